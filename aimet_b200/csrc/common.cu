// Error reporting, device queries and layout canonicalisation (host side).
#include <stdarg.h>
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace ab {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    // one cached value per device, filled on first use
    static int cached[64];
    static std::once_flag once[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::call_once(once[dev], [dev]() {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    });
    return cached[dev];
}

int canonicalize(const ab_layout *layout, Canon *out) {
    if (!layout) return fail(AB_ERR_INVALID, "layout is NULL");
    if (layout->ndim < 0 || layout->ndim > AB_MAX_DIMS)
        return fail(AB_ERR_INVALID, "layout.ndim=%d out of range [0, %d]", layout->ndim, AB_MAX_DIMS);

    int64_t size[AB_MAX_DIMS], block[AB_MAX_DIMS];
    int nd = 0;
    int64_t numel = 1;
    for (int k = 0; k < layout->ndim; ++k) {
        int64_t s = layout->size[k], b = layout->block[k];
        if (s < 0) return fail(AB_ERR_INVALID, "layout.size[%d]=%lld is negative", k, (long long)s);
        numel *= s;
        if (s == 0) continue;
        if (b <= 0 || s % b != 0)
            return fail(AB_ERR_INVALID, "layout.block[%d]=%lld does not divide size %lld", k,
                        (long long)b, (long long)s);
        if (s == 1) continue;
        // try to merge with the previous kept dim
        if (nd > 0) {
            int64_t ps = size[nd - 1], pb = block[nd - 1];
            if (pb == 1) {  // previous is per-channel: (i * s + j) / b indexes the merged parameter
                size[nd - 1] = ps * s;
                block[nd - 1] = b;
                continue;
            }
            if (b == s) {  // this dim broadcasts: previous block simply grows
                size[nd - 1] = ps * s;
                block[nd - 1] = pb * s;
                continue;
            }
        }
        size[nd] = s;
        block[nd] = b;
        ++nd;
    }

    Canon c;
    c.numel = numel;
    c.nd = nd;
    int64_t nparam = 1;
    for (int k = nd - 1; k >= 0; --k) {
        c.size[k] = size[k];
        c.block[k] = block[k];
        c.pstride[k] = nparam;
        nparam *= size[k] / block[k];
    }
    c.nparam = numel == 0 ? 0 : nparam;
    c.oci = false;
    c.O = c.C = c.I = 1;
    if (numel == 0) {
        c.oci = true;
        c.O = 0;
    } else if (nd == 0) {
        c.oci = true;
    } else if (nd == 1) {
        c.oci = true;
        c.I = block[0];
        c.C = size[0] / block[0];
    } else if (nd == 2 && block[0] == size[0]) {
        c.oci = true;
        c.O = size[0];
        c.I = block[1];
        c.C = size[1] / block[1];
    }
    *out = c;
    return AB_OK;
}

ChanMap make_chan_map(const Canon &c) {
    ChanMap m;
    m.I = c.I;
    m.C = c.C;
    m.shift = -1;
    if (c.I > 0 && (c.I & (c.I - 1)) == 0) {
        int s = 0;
        while (((int64_t)1 << s) < c.I) ++s;
        m.shift = s;
    }
    m.wrap = c.O > 1;
    m.narrow = c.numel < ((int64_t)1 << 31);
    return m;
}

GenMap make_gen_map(const Canon &c) {
    GenMap g;
    g.nd = c.nd;
    for (int k = 0; k < AB_MAX_DIMS; ++k) {
        g.size[k] = k < c.nd ? c.size[k] : 1;
        g.block[k] = k < c.nd ? c.block[k] : 1;
        g.pstride[k] = k < c.nd ? c.pstride[k] : 0;
    }
    return g;
}

static int pow2_ceil(int64_t v) {
    int r = 1;
    while (r < v) r <<= 1;
    return r;
}

ReducePlan plan_reduce(const Canon &c, int io_dtype, bool ptr_aligned, int chunk_mult, int ctas_per_sm) {
    ReducePlan p{};
    if (!c.oci) {
        p.mode = ReducePlan::GEN;
        return p;
    }
    const int vecw = 16 / dtype_size(io_dtype);
    const int64_t row_len = c.C * c.I;
    const int sms = sm_count();
    // column mode: many rows, short runs per parameter
    if (c.O > 1 && c.I < 64 * vecw) {
        p.mode = ReducePlan::COL;
        p.vect = ptr_aligned && (row_len % vecw == 0);
        const int v = p.vect ? vecw : 1;
        const int64_t gx = (row_len / v + kThreads - 1) / kThreads;
        int64_t tiles = (4 * (int64_t)sms + gx - 1) / gx;
        if (tiles > c.O) tiles = c.O;
        if (tiles > 65535) tiles = 65535;
        if (tiles < 1) tiles = 1;
        p.rows_per_tile = (c.O + tiles - 1) / tiles;
        p.row_tiles = (c.O + p.rows_per_tile - 1) / p.rows_per_tile;
        p.npartial = p.row_tiles * row_len;
        p.na = p.row_tiles;
        p.sa = row_len;
        p.sc = c.I;
        p.nb = c.I;
        return p;
    }
    p.mode = ReducePlan::SEG;
    p.vect = ptr_aligned && (c.I % vecw == 0);
    const int v = p.vect ? vecw : 1;
    const int64_t chunk = (int64_t)kThreads * kSegVecPerThread * v * chunk_mult;
    if (c.I > chunk) {
        p.seg_len = chunk;
        p.nchunk = (c.I + chunk - 1) / chunk;
        // one long run (per-tensor): cut it into a whole number of waves of CTAs so that the
        // last wave is not nearly empty
        const int64_t slots = (int64_t)sms * ctas_per_sm;
        if (ctas_per_sm > 0 && c.O * c.C == 1 && p.nchunk > slots) {
            int64_t waves = (p.nchunk + slots / 2) / slots;
            if (waves < 1) waves = 1;
            const int64_t want = waves * slots;
            const int64_t unit = 2 * (int64_t)v;  // two vectors: one loop iteration of a thread
            int64_t len = (c.I + want - 1) / want;
            len = (len + unit - 1) / unit * unit;
            p.seg_len = len;
            p.nchunk = (c.I + len - 1) / len;
        }
    } else {
        p.seg_len = c.I;
        p.nchunk = 1;
    }
    p.nseg = c.O * c.C * p.nchunk;
    const int64_t vec_per_seg = (p.seg_len + v - 1) / v;
    // aim at kSegVecPerThread vectors per thread (index arithmetic and the group reduction are paid per
    // thread)
    // small tensors: fewer vectors per thread, so that there are enough threads to fill the GPU
    // and a thread's chain of dependent memory latencies stays short
    const int64_t total_vec = vec_per_seg * p.nseg;
    int per_thread = kSegVecPerThread;
    while (per_thread > 2 && total_vec / per_thread < (int64_t)sms * 1024) per_thread >>= 1;
    int grp = pow2_ceil((vec_per_seg + per_thread - 1) / per_thread);
    // two neighbouring lanes read one 32-byte sector together
    const int floor_grp = vec_per_seg >= 2 ? 2 : 1;
    if (grp < floor_grp) grp = floor_grp;
    if (grp > kThreads) grp = kThreads;
    p.group = grp;
    p.direct = (c.O == 1 && p.nchunk == 1) ? 1 : 0;
    p.npartial = p.direct ? 0 : p.nseg;
    p.na = c.O;
    p.sa = c.C * p.nchunk;
    p.sc = p.nchunk;
    p.nb = p.nchunk;
    return p;
}

}  // namespace ab

extern "C" int aimet_b200_version(void) { return 1; }
extern "C" const char *aimet_b200_last_error(void) { return ab::g_error; }
extern "C" int64_t aimet_b200_launch_count(void) { return ab::g_launches.load(std::memory_order_relaxed); }
