// Calibration statistics: single-pass min/max, shared-memory histograms with
// the exact torch.histc binning rule, and the SQNR candidate sweep over a
// histogram.  Follows quantization/encoding_analyzer.py of the reference:
// _MinMaxObserver (:69-118), _HistogramObserver (:121-338) and
// _LpNormEncodingAnalyzer._estimate_clip_and_quant_noise (:822-899).
#include <math.h>

#include <mutex>

#include <type_traits>

#include "common.cuh"

namespace ab {
namespace {

// ---------------------------------------------------------------------------
// min / max
// ---------------------------------------------------------------------------
constexpr int kStatChunkMult = 4;  // read-only passes take longer runs per thread group
constexpr int kMaxBatch = 32;       // tensors of the same shape that one launch can take

template <typename T> struct MinMax {
    T lo, hi;
};

// torch.amin / amax semantics: NaN wins.
template <typename T> __device__ __forceinline__ void mm_update(MinMax<T> &m, T v, bool finite_only) {
    if (finite_only) {
        if (!isfinite(v)) return;
        m.lo = v < m.lo ? v : m.lo;
        m.hi = v > m.hi ? v : m.hi;
    } else {
        // once NaN, comparisons keep it: (v < NaN) is false and v != v picks up new NaNs
        m.lo = (v < m.lo || v != v) ? v : m.lo;
        m.hi = (v > m.hi || v != v) ? v : m.hi;
    }
}
template <typename T> __device__ __forceinline__ void mm_merge(MinMax<T> &m, T lo, T hi) {
    m.lo = (lo < m.lo || lo != lo) ? lo : m.lo;
    m.hi = (hi > m.hi || hi != hi) ? hi : m.hi;
}
template <typename T> __device__ __forceinline__ MinMax<T> mm_init() {
    MinMax<T> m;
    m.lo = (T)INFINITY;
    m.hi = (T)-INFINITY;
    return m;
}

template <int IO> struct StatT { using T = float; };
template <> struct StatT<AB_F64> { using T = double; };

template <typename T, typename E> __device__ __forceinline__ T stat_load(E v) { return (T)to_f32(v); }
template <> __device__ __forceinline__ double stat_load<double, double>(double v) { return v; }
template <> __device__ __forceinline__ double stat_load<double, float>(float v) { return (double)v; }

template <typename E> __device__ __forceinline__ E stat_store(double v);
template <> __device__ __forceinline__ float stat_store<float>(double v) { return (float)v; }
template <> __device__ __forceinline__ double stat_store<double>(double v) { return v; }
template <> __device__ __forceinline__ __half stat_store<__half>(double v) { return __float2half_rn((float)v); }
template <> __device__ __forceinline__ __nv_bfloat16 stat_store<__nv_bfloat16>(double v) {
    return __float2bfloat16_rn((float)v);
}

// Packed running min / max over the two 16-bit halves of each word: two instructions per pair of
// elements in the NaN-propagating mode, seven in the finite-only mode (non-finite halves are
// replaced by +inf / -inf before the comparison).
template <typename E> struct PackedMM { static constexpr bool ok = false; };
template <> struct PackedMM<__nv_bfloat16> {
    static constexpr bool ok = true;
    using H2 = __nv_bfloat162;
    static __device__ __forceinline__ H2 dup(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ float lo(H2 v) { return __low2float(v); }
    static __device__ __forceinline__ float hi(H2 v) { return __high2float(v); }
};
template <> struct PackedMM<__half> {
    static constexpr bool ok = true;
    using H2 = __half2;
    static __device__ __forceinline__ H2 dup(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ float lo(H2 v) { return __low2float(v); }
    static __device__ __forceinline__ float hi(H2 v) { return __high2float(v); }
};

template <typename H2> __device__ __forceinline__ H2 mm_bit_select(H2 a, H2 b, unsigned mask) {  // mask ? a : b
    const unsigned ua = *reinterpret_cast<unsigned *>(&a), ub = *reinterpret_cast<unsigned *>(&b);
    const unsigned r = (ua & mask) | (ub & ~mask);
    return *reinterpret_cast<const H2 *>(&r);
}

template <typename E, typename H2>
__device__ __forceinline__ void mm_update_packed(H2 &pmin, H2 &pmax, const Vec16<E> &v, bool finite_only, H2 pinf, H2 ninf) {
    const H2 *w = reinterpret_cast<const H2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (finite_only) {
            const unsigned bad = __hgeu2_mask(__habs2(w[i]), pinf);  // inf or NaN
            pmin = __hmin2(pmin, mm_bit_select(pinf, w[i], bad));
            pmax = __hmax2(pmax, mm_bit_select(ninf, w[i], bad));
        } else {
            pmin = __hmin2_nan(pmin, w[i]);
            pmax = __hmax2_nan(pmax, w[i]);
        }
    }
}

struct MinMaxArgs {
    const void *x;
    void *min_out, *max_out;  // io dtype, direct mode
    double *partial;          // [npartial][2]
    ChanMap cm;
    int64_t seg_len, nseg, nchunk;
    int group, direct;
    int64_t rows, row_len, rows_per_tile;
    int finite_only;
    int merge;  // direct mode: also take the values already in min_out / max_out
};

template <int IO, bool VECT> __global__ void __launch_bounds__(kThreads) k_minmax_seg(MinMaxArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using T = typename StatT<IO>::T;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    const int G = a.group;
    const int64_t s = (int64_t)blockIdx.x * (kThreads / G) + threadIdx.x / G;
    const int lane = threadIdx.x % G;
    const bool valid = s < a.nseg;
    MinMax<T> m = mm_init<T>();
    int64_t param = 0;
    if (valid) {
        int64_t ts = s, k = 0;
        if (a.nchunk > 1) {
            if (a.cm.narrow) {
                ts = (uint32_t)s / (uint32_t)a.nchunk;
                k = (uint32_t)s - (uint32_t)ts * (uint32_t)a.nchunk;
            } else {
                ts = s / a.nchunk;
                k = s - ts * a.nchunk;
            }
        }
        const int64_t start = ts * a.cm.I + k * a.seg_len;
        int64_t len = a.cm.I - k * a.seg_len;
        if (len > a.seg_len) len = a.seg_len;
        if (a.cm.C == 1)
            param = 0;
        else if (!a.cm.wrap)
            param = ts;
        else
            param = a.cm.narrow ? (int64_t)((uint32_t)ts % (uint32_t)a.cm.C) : ts % a.cm.C;
        const int64_t nv = len / VEC, v0 = start / VEC;
        for (int64_t v = lane; v < nv; v += 2 * (int64_t)G) {
            const bool hb = v + G < nv;
            if constexpr (VECT && PackedMM<E>::ok) {
                using PM = PackedMM<E>;
                const typename PM::H2 pinf = PM::dup(INFINITY), ninf = PM::dup(-INFINITY);
                typename PM::H2 pmin = pinf, pmax = ninf;
                // this path walks the whole run itself, four vectors in flight per thread
                for (int64_t w = v; w < nv; w += 4 * (int64_t)G) {
                    Vec16<E> xs[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (w + (int64_t)u * G < nv) xs[u] = reinterpret_cast<const Vec16<E> *>(xp)[v0 + w + (int64_t)u * G];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (w + (int64_t)u * G < nv) mm_update_packed<E>(pmin, pmax, xs[u], a.finite_only != 0, pinf, ninf);
                }
                mm_merge(m, (T)PM::lo(pmin), (T)PM::lo(pmax));
                mm_merge(m, (T)PM::hi(pmin), (T)PM::hi(pmax));
                break;
            } else if constexpr (VECT) {
                Vec16<E> xa = reinterpret_cast<const Vec16<E> *>(xp)[v0 + v], xb;
                if (hb) xb = reinterpret_cast<const Vec16<E> *>(xp)[v0 + v + G];
#pragma unroll
                for (int i = 0; i < VEC; ++i) mm_update(m, stat_load<T, E>(xa.v[i]), a.finite_only);
                if (hb) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) mm_update(m, stat_load<T, E>(xb.v[i]), a.finite_only);
                }
            } else {
                mm_update(m, stat_load<T, E>(xp[v0 + v]), a.finite_only);
                if (hb) mm_update(m, stat_load<T, E>(xp[v0 + v + G]), a.finite_only);
            }
        }
    }
    const int span = G < 32 ? G : 32;
    for (int o = span >> 1; o > 0; o >>= 1) {
        T lo = __shfl_xor_sync(0xffffffffu, m.lo, o);
        T hi = __shfl_xor_sync(0xffffffffu, m.hi, o);
        mm_merge(m, lo, hi);
    }
    if (G > 32) {
        __shared__ double sh[2][kThreads / 32];
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
            sh[0][warp] = (double)m.lo;
            sh[1][warp] = (double)m.hi;
        }
        __syncthreads();
        if (lane == 0) {
            const int w0 = (threadIdx.x / G) * (G / 32);
            for (int w = 1; w < G / 32; ++w) mm_merge(m, (T)sh[0][w0 + w], (T)sh[1][w0 + w]);
        }
    }
    if (valid && lane == 0) {
        if (a.direct) {
            if (a.merge)
                mm_merge(m, stat_load<T, E>(static_cast<E *>(a.min_out)[param]),
                         stat_load<T, E>(static_cast<E *>(a.max_out)[param]));
            static_cast<E *>(a.min_out)[param] = stat_store<E>((double)m.lo);
            static_cast<E *>(a.max_out)[param] = stat_store<E>((double)m.hi);
        } else {
            a.partial[2 * s] = (double)m.lo;
            a.partial[2 * s + 1] = (double)m.hi;
        }
    }
}

template <int IO, bool VECT> __global__ void __launch_bounds__(kThreads) k_minmax_col(MinMaxArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using T = typename StatT<IO>::T;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    const int64_t cv = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t ncv = a.row_len / VEC;
    if (cv >= ncv) return;
    const int64_t r0 = (int64_t)blockIdx.y * a.rows_per_tile;
    int64_t r1 = r0 + a.rows_per_tile;
    if (r1 > a.rows) r1 = a.rows;
    MinMax<T> m[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) m[i] = mm_init<T>();
    for (int64_t r = r0; r < r1; r += 2) {
        const bool hb = r + 1 < r1;
        Vec16<E> xa, xb;
        if (VECT) {
            xa = reinterpret_cast<const Vec16<E> *>(xp)[r * ncv + cv];
            if (hb) xb = reinterpret_cast<const Vec16<E> *>(xp)[(r + 1) * ncv + cv];
        } else {
            xa.v[0] = xp[r * ncv + cv];
            if (hb) xb.v[0] = xp[(r + 1) * ncv + cv];
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) mm_update(m[i], stat_load<T, E>(xa.v[i]), a.finite_only);
        if (hb) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) mm_update(m[i], stat_load<T, E>(xb.v[i]), a.finite_only);
        }
    }
    double *out = a.partial + 2 * ((int64_t)blockIdx.y * a.row_len + cv * VEC);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        out[2 * i] = (double)m[i].lo;
        out[2 * i + 1] = (double)m[i].hi;
    }
}

struct MinMaxFinishArgs {
    const double *partial;
    void *min_out, *max_out;
    int64_t nparam, na, sa, sc, nb;
    int merge;  // also take the values already in min_out / max_out (a running min / max over calls)
};

template <int IO, bool PER_CTA> __global__ void __launch_bounds__(kThreads) k_minmax_finish(MinMaxFinishArgs a) {
    pdl_prologue();
    // PER_CTA: one CTA per statistic (many partials each); else one warp per statistic
    using E = typename Elem<IO>::type;
    const int64_t c = PER_CTA ? (int64_t)blockIdx.x : (((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (c >= a.nparam) return;
    MinMax<double> m = mm_init<double>();
    const int64_t n = a.na * a.nb;
    const int step = PER_CTA ? kThreads : 32;
    for (int64_t t = PER_CTA ? threadIdx.x : lane; t < n; t += step) {
        const int64_t ia = t / a.nb, ib = t - ia * a.nb;
        const double *p = a.partial + 2 * (ia * a.sa + c * a.sc + ib);
        mm_merge(m, p[0], p[1]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        double lo = __shfl_xor_sync(0xffffffffu, m.lo, o);
        double hi = __shfl_xor_sync(0xffffffffu, m.hi, o);
        mm_merge(m, lo, hi);
    }
    if (PER_CTA) {
        __shared__ double sh[2][kThreads / 32];
        if (lane == 0) {
            sh[0][threadIdx.x >> 5] = m.lo;
            sh[1][threadIdx.x >> 5] = m.hi;
        }
        __syncthreads();
        if (threadIdx.x != 0) return;
        for (int w = 1; w < kThreads / 32; ++w) mm_merge(m, sh[0][w], sh[1][w]);
    }
    if (lane == 0) {
        if (a.merge) mm_merge(m, (double)stat_load<double, E>(static_cast<E *>(a.min_out)[c]),
                              (double)stat_load<double, E>(static_cast<E *>(a.max_out)[c]));
        static_cast<E *>(a.min_out)[c] = stat_store<E>(m.lo);
        static_cast<E *>(a.max_out)[c] = stat_store<E>(m.hi);
    }
}

template <int IO> void launch_minmax_finish(const MinMaxFinishArgs &f, cudaStream_t stream) {
    if (f.na * f.nb > 256) {
        launch_pdl(k_minmax_finish<IO, true>, (unsigned)f.nparam, kThreads, 0, stream, f);
    } else {
        const int64_t grid = (f.nparam * 32 + kThreads - 1) / kThreads;
        launch_pdl(k_minmax_finish<IO, false>, (unsigned)grid, kThreads, 0, stream, f);
    }
}

// One statistic over whole contiguous tensors (a per-tensor quantizer's calibration), several
// tensors of the same size per launch: chunks of 1024 vectors are dealt out round-robin to the
// CTAs, four loads in flight per thread, one partial pair per CTA.
struct MinMaxFlatArgs {
    const void *xs[kMaxBatch];
    int num_x;
    int64_t numel;
    int finite_only;
    double *partial;  // [gridDim.x][2]
};

template <int IO> __global__ void __launch_bounds__(kThreads) k_minmax_flat(MinMaxFlatArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using T = typename StatT<IO>::T;
    constexpr int VEC = 16 / (int)sizeof(E);
    constexpr int U = 4;
    const int64_t nvec = a.numel / VEC;
    const int64_t chunk = (int64_t)kThreads * U;
    const int64_t chunks_per_x = (nvec + chunk - 1) / chunk;
    const int64_t total = chunks_per_x * a.num_x;
    const bool fin = a.finite_only != 0;
    MinMax<T> m = mm_init<T>();
    [[maybe_unused]] auto packed = [&]() {
        if constexpr (PackedMM<E>::ok) {
            using PM = PackedMM<E>;
            const typename PM::H2 pinf = PM::dup(INFINITY), ninf = PM::dup(-INFINITY);
            typename PM::H2 pmin = pinf, pmax = ninf;
            for (int64_t ch = blockIdx.x; ch < total; ch += gridDim.x) {
                const int64_t xi = ch / chunks_per_x, lc = ch - xi * chunks_per_x;
                const Vec16<E> *xp = static_cast<const Vec16<E> *>(a.xs[xi]);
                const int64_t base = lc * chunk + threadIdx.x;
                Vec16<E> v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (base + (int64_t)u * kThreads < nvec) v[u] = xp[base + (int64_t)u * kThreads];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (base + (int64_t)u * kThreads < nvec) mm_update_packed<E>(pmin, pmax, v[u], fin, pinf, ninf);
            }
            mm_merge(m, (T)PM::lo(pmin), (T)PM::lo(pmax));
            mm_merge(m, (T)PM::hi(pmin), (T)PM::hi(pmax));
        }
    };
    if constexpr (PackedMM<E>::ok) {
        packed();
    } else {
        for (int64_t ch = blockIdx.x; ch < total; ch += gridDim.x) {
            const int64_t xi = ch / chunks_per_x, lc = ch - xi * chunks_per_x;
            const Vec16<E> *xp = static_cast<const Vec16<E> *>(a.xs[xi]);
            const int64_t base = lc * chunk + threadIdx.x;
            Vec16<E> v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (base + (int64_t)u * kThreads < nvec) v[u] = xp[base + (int64_t)u * kThreads];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (base + (int64_t)u * kThreads < nvec) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) mm_update(m, stat_load<T, E>(v[u].v[i]), fin);
                }
        }
    }
    // elements beyond the last whole vector of each tensor
    const int tail = (int)(a.numel - nvec * VEC);
    if (blockIdx.x == 0 && (int)threadIdx.x < tail * a.num_x) {
        const int xi = threadIdx.x / tail, i = threadIdx.x - xi * tail;
        mm_update(m, stat_load<T, E>(static_cast<const E *>(a.xs[xi])[nvec * VEC + i]), fin);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        T lo = __shfl_xor_sync(0xffffffffu, m.lo, o);
        T hi = __shfl_xor_sync(0xffffffffu, m.hi, o);
        mm_merge(m, lo, hi);
    }
    __shared__ double sh[2][kThreads / 32];
    if ((threadIdx.x & 31) == 0) {
        sh[0][threadIdx.x >> 5] = (double)m.lo;
        sh[1][threadIdx.x >> 5] = (double)m.hi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        MinMax<double> r = mm_init<double>();
        for (int w = 0; w < kThreads / 32; ++w) mm_merge(r, sh[0][w], sh[1][w]);
        a.partial[2 * blockIdx.x] = r.lo;
        a.partial[2 * blockIdx.x + 1] = r.hi;
    }
}

template <int IO>
int launch_minmax(const void *x, const Canon &canon, int finite_only, int merge, void *min_out, void *max_out,
                  void *scratch, int64_t scratch_bytes, cudaStream_t stream);

// a list of tensors of the same layout: min_out / max_out run over all of them
template <int IO>
int launch_minmax_list(const void *const *xs, int num_x, const Canon &canon, int finite_only, int merge, void *min_out,
                       void *max_out, void *scratch, int64_t scratch_bytes, cudaStream_t stream) {
    bool flat = canon.oci && canon.nparam == 1 && canon.numel >= (1 << 16);
    for (int i = 0; i < num_x; ++i) flat = flat && aligned16(xs[i]);
    if (!flat) {
        for (int i = 0; i < num_x; ++i) {
            const int rc = launch_minmax<IO>(xs[i], canon, finite_only, merge || i > 0, min_out, max_out, scratch,
                                             scratch_bytes, stream);
            if (rc != AB_OK) return rc;
        }
        return AB_OK;
    }
    const int vec = 16 / dtype_size(IO);
    for (int i0 = 0; i0 < num_x; i0 += kMaxBatch) {
        MinMaxFlatArgs a;
        a.num_x = num_x - i0 < kMaxBatch ? num_x - i0 : kMaxBatch;
        for (int i = 0; i < a.num_x; ++i) a.xs[i] = xs[i0 + i];
        a.numel = canon.numel;
        a.finite_only = finite_only;
        a.partial = static_cast<double *>(scratch);
        const int64_t chunks = ((canon.numel / vec + (int64_t)kThreads * 4 - 1) / ((int64_t)kThreads * 4)) * a.num_x;
        int64_t grid = (int64_t)sm_count() * 8;
        if (grid > chunks) grid = chunks;
        if (grid < 1) grid = 1;
        const int64_t need = grid * 2 * (int64_t)sizeof(double);
        if (!scratch || scratch_bytes < need)
            return fail(AB_ERR_SCRATCH, "min/max needs %lld bytes of scratch, got %lld", (long long)need,
                        (long long)scratch_bytes);
        launch_pdl(k_minmax_flat<IO>, (unsigned)grid, kThreads, 0, stream, a);
        AB_LAUNCH_OK();
        MinMaxFinishArgs f{a.partial, min_out, max_out, 1, 1, 0, grid, grid, (merge || i0 > 0) ? 1 : 0};
        launch_minmax_finish<IO>(f, stream);
        AB_LAUNCH_OK();
    }
    return AB_OK;
}

template <int IO>
int launch_minmax(const void *x, const Canon &canon, int finite_only, int merge, void *min_out, void *max_out,
                  void *scratch, int64_t scratch_bytes, cudaStream_t stream) {
    const ReducePlan p = plan_reduce(canon, IO, aligned16(x), kStatChunkMult);
    if (p.mode == ReducePlan::GEN)
        return fail(AB_ERR_UNSUPPORTED, "statistics need a layout that reduces to (outer, channel, inner)");
    const int64_t need = p.npartial * 2 * (int64_t)sizeof(double);
    if (need > 0 && (!scratch || scratch_bytes < need))
        return fail(AB_ERR_SCRATCH, "min/max needs %lld bytes of scratch, got %lld", (long long)need,
                    (long long)scratch_bytes);
    MinMaxArgs a;
    a.x = x;
    a.min_out = min_out;
    a.max_out = max_out;
    a.partial = static_cast<double *>(scratch);
    a.cm = make_chan_map(canon);
    a.seg_len = p.seg_len;
    a.nseg = p.nseg;
    a.nchunk = p.nchunk;
    a.group = p.group;
    a.direct = p.direct;
    a.rows = canon.O;
    a.row_len = canon.C * canon.I;
    a.rows_per_tile = p.rows_per_tile;
    a.finite_only = finite_only;
    a.merge = merge;
    if (p.mode == ReducePlan::SEG) {
        const int gpc = kThreads / p.group;
        const int64_t grid = (p.nseg + gpc - 1) / gpc;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (p.vect)
            launch_pdl(k_minmax_seg<IO, true>, (unsigned)grid, kThreads, 0, stream, a);
        else
            launch_pdl(k_minmax_seg<IO, false>, (unsigned)grid, kThreads, 0, stream, a);
    } else {
        const int v = p.vect ? 16 / dtype_size(IO) : 1;
        const int64_t gx = (a.row_len / v + kThreads - 1) / kThreads;
        dim3 grid((unsigned)gx, (unsigned)p.row_tiles);
        if (p.vect)
            launch_pdl(k_minmax_col<IO, true>, grid, kThreads, 0, stream, a);
        else
            launch_pdl(k_minmax_col<IO, false>, grid, kThreads, 0, stream, a);
    }
    AB_LAUNCH_OK();
    if (p.npartial > 0) {
        MinMaxFinishArgs f{a.partial, min_out, max_out, canon.nparam, p.na, p.sa, p.sc, p.nb, merge};
        launch_minmax_finish<IO>(f, stream);
        AB_LAUNCH_OK();
    }
    return AB_OK;
}

// ---------------------------------------------------------------------------
// histogram
// ---------------------------------------------------------------------------
constexpr int kHistUnroll = 4;

struct HistArgs {
    const void *x;
    const float *lo, *hi, *below, *above;
    unsigned long long *counts;  // [C][num_bins]
    double *mm_partial;          // [C][tiles][2] or NULL
    int64_t O, C, I;
    int64_t chan_elems;          // O * I
    int64_t tile_elems;          // elements of one channel handled by one CTA (multiple of 16)
    int num_bins;
    int tiles;                   // CTAs per channel
    const int *run_if;           // NULL, or one device flag per histogram: nothing is done for those that are zero
};

// torch.histc's bin of v over [lo, hi] (CPU and CUDA kernels agree):
//   bin = (int)((v - lo) * num_bins / (hi - lo)), with v == hi folded into the last bin.
__device__ __forceinline__ int histc_bin(float v, float lo, float range, float nbins_f, int nbins) {
    int b = __float2int_rz(__fdiv_rn(__fmul_rn(__fsub_rn(v, lo), nbins_f), range));
    return b >= nbins ? nbins - 1 : b;
}

// One CTA bins one tile of one channel into a shared-memory histogram.  Values
// of a calibration batch pile up in a handful of bins, so a warp whose lanes all
// hit the same bin issues a single shared-memory atomic.
template <int IO, bool VECT> __global__ void __launch_bounds__(kThreads) k_histogram(HistArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    extern __shared__ unsigned int sh_hist[];
    __shared__ unsigned long long sh_edge[2];
    __shared__ float sh_mm[2][kThreads / 32];

    if (a.run_if && a.run_if[blockIdx.y] == 0) return;
    const int64_t c = blockIdx.y;
    const int tile = blockIdx.x;
    for (int b = threadIdx.x; b < a.num_bins; b += kThreads) sh_hist[b] = 0;
    if (threadIdx.x < 2) sh_edge[threadIdx.x] = 0;
    __syncthreads();

    const float lo = a.lo[c], hi = a.hi[c];
    const float range = __fsub_rn(hi, lo);
    const float nbf = (float)a.num_bins;
    const float below = a.below[c], above = a.above[c];
    const E *__restrict__ xp = static_cast<const E *>(a.x);

    const int64_t e0 = (int64_t)tile * a.tile_elems;
    int64_t e1 = e0 + a.tile_elems;
    if (e1 > a.chan_elems) e1 = a.chan_elems;

    unsigned int n_below = 0, n_above = 0;
    float fmin_ = INFINITY, fmax_ = -INFINITY;
    const bool want_mm = a.mm_partial != nullptr;
    const unsigned full = 0xffffffffu;
    const int lane = threadIdx.x & 31;

    auto consume = [&](float v, int &run_bin, unsigned int &run_cnt) {
        if (v < below) ++n_below;
        if (v > above) ++n_above;
        if (want_mm && isfinite(v)) {
            fmin_ = fminf(fmin_, v);
            fmax_ = fmaxf(fmax_, v);
        }
        if (v >= lo && v <= hi) {
            const int b = histc_bin(v, lo, range, nbf, a.num_bins);
            if (b == run_bin) {
                ++run_cnt;
            } else {
                if (run_cnt) atomicAdd(&sh_hist[run_bin], run_cnt);
                run_bin = b;
                run_cnt = 1;
            }
        }
    };

    // element index within the channel -> address: (o * C + c) * I + i
    const bool flat = (a.C == 1);
    const int64_t nvec = (e1 - e0) / VEC;  // tiles and runs are multiples of VEC when VECT
    // the trip count is the same for every thread of the CTA: the warp-wide votes below need all lanes
    for (int64_t base = 0; base < nvec; base += kThreads * kHistUnroll) {
        const int64_t v0 = base + threadIdx.x;
        Vec16<E> xv[kHistUnroll];
        bool ok[kHistUnroll];
#pragma unroll
        for (int u = 0; u < kHistUnroll; ++u) {
            const int64_t v = v0 + (int64_t)u * kThreads;
            ok[u] = v < nvec;
            if (ok[u]) {
                const int64_t e = e0 + v * VEC;
                int64_t addr;
                if (flat) {
                    addr = e;
                } else {
                    const int64_t o = e / a.I, i = e - o * a.I;
                    addr = (o * a.C + c) * a.I + i;
                }
                if (VECT)
                    xv[u] = *reinterpret_cast<const Vec16<E> *>(xp + addr);
                else
                    xv[u].v[0] = xp[addr];
            }
        }
#pragma unroll
        for (int u = 0; u < kHistUnroll; ++u) {
            int run_bin = -1;
            unsigned int run_cnt = 0;
            if (ok[u]) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) consume(to_f32(xv[u].v[i]), run_bin, run_cnt);
            }
            // warp-uniform fast path: every lane ended on the same bin
            const int b0 = __shfl_sync(full, run_bin, 0);
            if (__all_sync(full, run_bin == b0)) {
                const unsigned int tot = __reduce_add_sync(full, run_cnt);
                if (lane == 0 && tot) atomicAdd(&sh_hist[b0], tot);
            } else if (run_cnt) {
                atomicAdd(&sh_hist[run_bin], run_cnt);
            }
        }
    }

    // below / above counts
    n_below = __reduce_add_sync(full, n_below);
    n_above = __reduce_add_sync(full, n_above);
    if (lane == 0) {
        if (n_below) atomicAdd(&sh_edge[0], (unsigned long long)n_below);
        if (n_above) atomicAdd(&sh_edge[1], (unsigned long long)n_above);
    }
    if (want_mm) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            fmin_ = fminf(fmin_, __shfl_xor_sync(full, fmin_, o));
            fmax_ = fmaxf(fmax_, __shfl_xor_sync(full, fmax_, o));
        }
        if (lane == 0) {
            sh_mm[0][threadIdx.x >> 5] = fmin_;
            sh_mm[1][threadIdx.x >> 5] = fmax_;
        }
    }
    __syncthreads();
    unsigned long long *out = a.counts + c * (int64_t)a.num_bins;
    for (int b = threadIdx.x; b < a.num_bins; b += kThreads) {
        unsigned long long n = sh_hist[b];
        if (b == 0) n += sh_edge[0];
        if (b == a.num_bins - 1) n += sh_edge[1];
        if (n) atomicAdd(out + b, n);
    }
    if (want_mm && threadIdx.x == 0) {
        float mn = sh_mm[0][0], mx = sh_mm[1][0];
        for (int w = 1; w < kThreads / 32; ++w) {
            mn = fminf(mn, sh_mm[0][w]);
            mx = fmaxf(mx, sh_mm[1][w]);
        }
        double *p = a.mm_partial + 2 * (c * (int64_t)a.tiles + tile);
        p[0] = (double)mn;
        p[1] = (double)mx;
    }
}

// ---------------------------------------------------------------------------
// Large histograms.  The pass over the tensor is instruction-bound (2-4 bytes per element), so
// the common case is kept to a handful of instructions per element:
//  * the bin is computed arithmetically with the exact torch.histc formula,
//    (v - lo) * bins / (hi - lo), the division by reciprocal and exact remainder (see div_fast in
//    the affine kernels), the truncation by an add of 2^23 rounded toward zero, two elements per
//    instruction (FADD2 / FMUL2 / FFMA2);
//  * a 16-byte vector is checked as a whole (packed min / max, NaN-propagating): when all its
//    values lie inside the binning range and inside the outlier thresholds they are counted
//    without any per-element predicate; otherwise the vector takes the element-wise general body;
//  * 16 replicas of the histogram, counter (bin, lane mod 16) at (bin * 16 + lane mod 16) * 4:
//    calibration batches pile up in a handful of bins, and with replicas a warp's increments of
//    one bin collide at most two-fold (measured: peaked and flat data take the same time, and
//    counting the most frequent bins in registers instead did not pay for its instructions);
//  * the next iteration's loads are issued before this one's arithmetic: the warps of the one
//    1024-thread CTA per SM run in step and would otherwise all wait on memory together.
// ---------------------------------------------------------------------------
constexpr int kPrivThreads = 1024;
constexpr int kPrivCopies = 16;
constexpr int kPrivMaxBins = 3072;                    // (bins + 1) * 64 B of counters: 192 KB
constexpr size_t kPrivSmemMax = 232448 - 1024;        // dynamic shared memory one CTA may ask for
constexpr int64_t kPrivMinElems = 1 << 20;            // per histogram; below this the plain kernel

struct HistPrivArgs {
    const void *x;
    const void *xs[kMaxBatch];  // num_x tensors of the same shape (a single contiguous statistic only)
    int num_x;
    const float *lo, *hi, *below, *above;
    unsigned long long *counts;
    double *mm_partial;  // [C][tiles][2] finite min / max of each CTA's tile, or NULL
    int64_t O, C, I;
    int64_t chan_elems, tile_elems;
    int num_bins;
    int tiles;
    const int *run_if;   // NULL, or one device flag per histogram: nothing is done for those that are zero
};

// all values of the vector inside [plo, phi] (false if any is NaN); the packed minimum and maximum
// of a 16-bit vector are handed back for the running min / max
struct RangeF32 {
    float plo, phi;
    __device__ __forceinline__ void init(float lo, float hi) {
        plo = lo;
        phi = hi;
    }
    __device__ __forceinline__ bool inside(const Vec16<float> &v, float &mn, float &mx) const {
        float mn2, mx2;
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(mn) : "f"(v.v[0]), "f"(v.v[1]));
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(mx) : "f"(v.v[0]), "f"(v.v[1]));
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(mn2) : "f"(v.v[2]), "f"(v.v[3]));
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(mx2) : "f"(v.v[2]), "f"(v.v[3]));
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(mn) : "f"(mn), "f"(mn2));
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(mx) : "f"(mx), "f"(mx2));
        return mn >= plo && mx <= phi;
    }
};
// For 16-bit elements the thresholds are moved onto the element grid (the lower one rounded up, the
// upper one rounded down): a 16-bit value is >= plo exactly when it is >= the smallest 16-bit value
// that is, so the whole test is two packed comparisons.
template <typename E> struct Range16 {
    using H2 = typename std::conditional<std::is_same<E, __half>::value, __half2, __nv_bfloat162>::type;
    H2 plo, phi;
    __device__ __forceinline__ void init(float lo, float hi) {
        if constexpr (std::is_same<E, __half>::value) {
            plo = __half2half2(__float2half_ru(lo));
            phi = __half2half2(__float2half_rd(hi));
        } else {
            plo = __bfloat162bfloat162(__float2bfloat16_ru(lo));
            phi = __bfloat162bfloat162(__float2bfloat16_rd(hi));
        }
    }
    __device__ __forceinline__ bool inside(const Vec16<E> &v, H2 &mn, H2 &mx) const {
        const H2 *w = reinterpret_cast<const H2 *>(&v);
        mn = __hmin2_nan(__hmin2_nan(w[0], w[1]), __hmin2_nan(w[2], w[3]));
        mx = __hmax2_nan(__hmax2_nan(w[0], w[1]), __hmax2_nan(w[2], w[3]));
        return __hbge2(mn, plo) && __hble2(mx, phi);
    }
};

// MM: also produce the finite minimum and maximum of the tile (for the pass that bins a batch
// against a range known beforehand and learns the batch's own range on the way).
template <int IO, bool MM, bool POW2, int RING>
__global__ void __launch_bounds__(kPrivThreads, 1) k_hist_private(HistPrivArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    constexpr int NV = 16 / (int)sizeof(E);
    constexpr bool F32 = std::is_same<E, float>::value;
    using Range = typename std::conditional<F32, RangeF32, Range16<E>>::type;
    using Ext = typename std::conditional<F32, float, typename Range16<typename std::conditional<F32, __half, E>::type>::H2>::type;
    extern __shared__ __align__(16) unsigned int sh_cnt[];  // [num_bins + 1][16]; row num_bins: v == hi
    __shared__ unsigned long long sh_edge[2];
    __shared__ float sh_mm[2][kPrivThreads / 32];
    if (a.run_if && a.run_if[blockIdx.y] == 0) return;
    const int64_t c = blockIdx.y;
    for (int i = threadIdx.x; i < (a.num_bins + 1) * kPrivCopies; i += kPrivThreads) sh_cnt[i] = 0;
    if (threadIdx.x < 2) sh_edge[threadIdx.x] = 0;
    __syncthreads();

    const float lo = a.lo[c], hi = a.hi[c], below = a.below[c], above = a.above[c];
    const float range = __fsub_rn(hi, lo), nbf = (float)a.num_bins;
    // a power-of-two bin count scales exactly: (v - lo) * bins / range == (v - lo) / (range / bins)
    const float dvs = POW2 ? __fdiv_rn(range, nbf) : range;  // divisor of the quick body
    const float mul = POW2 ? 1.0f : nbf;
    const float r = __frcp_rn(dvs);
    // the quick body needs a moderate range (exact reciprocal division, no underflow in the remainder)
    const bool quick = range > 1.0e-25f && range < 1.2676506e30f && fabsf(lo) < 1.2676506e30f &&
                       fabsf(hi) < 1.2676506e30f;
    // "plain" values lie inside the binning range and inside the outlier thresholds: they count in
    // their bin and nowhere else
    Range rng;
    rng.init(fmaxf(lo, below), fminf(hi, above));
    const int lane = threadIdx.x & 31;
    // counter (bin, lane mod 16) lives at base + 64 * bin + 4 * (lane mod 16).  The quick body gets the
    // bin as the low bits of the float 2^23 + bin (0x4B000000 + bin), so the address is one
    // multiply-add on those bits with the constant part folded into the base.
    const unsigned base = (unsigned)__cvta_generic_to_shared(sh_cnt) + 4u * (lane & (kPrivCopies - 1));
    const unsigned base_q = base - (0x4B000000u << 6);
    unsigned int n_below = 0, n_above = 0;
    float fmn = INFINITY, fmx = -INFINITY;  // general body's finite min / max
    Ext rmn, rmx;                            // quick body's running (packed) min / max
    if constexpr (F32) {
        rmn = INFINITY;
        rmx = -INFINITY;
    } else if constexpr (std::is_same<E, __half>::value) {
        rmn = __float2half2_rn(INFINITY);
        rmx = __float2half2_rn(-INFINITY);
    } else {
        rmn = __float2bfloat162_rn(INFINITY);
        rmx = __float2bfloat162_rn(-INFINITY);
    }

    auto count = [&](int b) {  // b in [0, num_bins]
        asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(base + ((unsigned)b << 6)), "r"(1u) : "memory");
    };
    const float2 nlo2 = make_float2(-lo, -lo), mul2 = make_float2(mul, mul), r2 = make_float2(r, r),
                 ndv2 = make_float2(-dvs, -dvs), one2 = make_float2(1.0f, 1.0f),
                 magic2 = make_float2(8388608.0f, 8388608.0f);
    auto quick_pair = [&](float fx, float fy) {
        float2 t = __fadd2_rn(make_float2(fx, fy), nlo2);
        if (!POW2) t = __fmul2_rn(t, mul2);
        const float2 q0 = __fmul2_rn(t, r2);
        const float2 rem = __ffma2_rn(q0, ndv2, t);
        const float2 q = __ffma2_rn(rem, r2, q0);
        const float2 tb = __ffma2_rz(q, one2, magic2);
        asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(__float_as_uint(tb.x) * 64u + base_q), "r"(1u) : "memory");
        asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(__float_as_uint(tb.y) * 64u + base_q), "r"(1u) : "memory");
    };
    auto general_vec = [&](unsigned slot_addr) {  // rare: the vector is read back from its ring slot
#pragma unroll 1
        for (int i = 0; i < NV; ++i) {
            E e;
            if constexpr (F32) {
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(e) : "r"(slot_addr + 4u * i) : "memory");
            } else {
                unsigned short bits;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(bits) : "r"(slot_addr + 2u * i) : "memory");
                e = *reinterpret_cast<const E *>(&bits);
            }
            const float v = to_f32(e);
            if (v >= lo && v <= hi) count(histc_bin(v, lo, range, nbf, a.num_bins));
            n_below += v < below;
            n_above += v > above;
            if (MM && isfinite(v)) {
                fmn = fminf(fmn, v);
                fmx = fmaxf(fmx, v);
            }
        }
    };
    auto feed = [&](const Vec16<E> &w, unsigned slot_addr) {
        Ext mn, mx;
        if (quick && rng.inside(w, mn, mx)) {
            if constexpr (MM) {
                if constexpr (F32) {
                    rmn = fminf(rmn, mn);
                    rmx = fmaxf(rmx, mx);
                } else {
                    rmn = __hmin2(rmn, mn);
                    rmx = __hmax2(rmx, mx);
                }
            }
            if constexpr (F32) {
                quick_pair(w.v[0], w.v[1]);
                quick_pair(w.v[2], w.v[3]);
            } else if constexpr (std::is_same<E, __nv_bfloat16>::value) {
                const uint32_t *u = reinterpret_cast<const uint32_t *>(&w);
#pragma unroll
                for (int i = 0; i < 4; ++i) quick_pair(__uint_as_float(u[i] << 16), __uint_as_float(u[i] & 0xffff0000u));
            } else {
                const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h[i]);
                    quick_pair(f.x, f.y);
                }
            }
        } else {
            general_vec(slot_addr);
        }
    };

    // Which vectors this CTA bins.  A single histogram over one contiguous run (the usual case: a
    // per-tensor statistic), possibly of several tensors of the same shape, is dealt out in rounds of
    // RING * 1024 vectors, round r going to CTA r mod gridDim.x: every SM then reads from all over
    // the tensors and sees the same mix of memory channels as the others (with one contiguous tile
    // per CTA some SMs finished 15 % early).  Otherwise a CTA walks its own tile of the channel.
    const bool flat = a.C == 1;
    const int64_t e0 = flat ? 0 : (int64_t)blockIdx.x * a.tile_elems;
    int64_t e1 = flat ? a.chan_elems : e0 + a.tile_elems;
    if (e1 > a.chan_elems) e1 = a.chan_elems;
    const int64_t nvec = (e1 - e0) / NV;
    constexpr int T = kPrivThreads;
    const int64_t rounds_per_x = (nvec + RING * T - 1) / (RING * T);
    const int64_t num_runs = flat ? (int64_t)a.num_x : 1;  // tensors walked one after the other
    const int64_t G = flat ? gridDim.x : 1, bidx = flat ? blockIdx.x : 0;
    // The input reaches the thread through its own ring of RING 16-byte slots in shared memory,
    // filled by cp.async: RING - 1 vectors per thread (80 KB per SM with six slots) are in flight
    // while one is binned, however the compiler orders the rest -- the pass is bound by memory
    // latency otherwise, the warps of the one 1024-thread CTA per SM running in step.  A thread only
    // ever touches its own slots, so no barrier is involved.
    constexpr unsigned kSlotBytes = T * 16u;
    const unsigned ring = (unsigned)__cvta_generic_to_shared(sh_cnt) + (unsigned)(a.num_bins + 1) * (kPrivCopies * 4u) +
                          16u * threadIdx.x;
    // a round: the tensor it reads and this thread's first vector in it
    struct Round {
        const Vec16<E> *x;
        int64_t v;
    };
    // rounds are walked in steps of G: the tensor index and the round inside it advance by
    // additions (a 64-bit division per round costs about two instructions per element)
    int64_t r_xi = rounds_per_x > 0 ? bidx / rounds_per_x : num_runs;
    int64_t r_lr = rounds_per_x > 0 ? bidx - r_xi * rounds_per_x : 0;
    auto next_round = [&]() -> Round {
        Round rd;
        if (r_xi >= num_runs) {
            rd.x = nullptr;
            rd.v = nvec;  // beyond the end: nothing is fetched or binned
            return rd;
        }
        rd.x = static_cast<const Vec16<E> *>(flat ? a.xs[r_xi] : a.x);
        rd.v = r_lr * (RING * T) + threadIdx.x;
        r_lr += G;
        while (r_lr >= rounds_per_x && r_xi < num_runs) {
            r_lr -= rounds_per_x;
            ++r_xi;
        }
        return rd;
    };
    auto src = [&](const Round &rd, int64_t v) -> const Vec16<E> * {
        if (flat) return rd.x + v;
        const int64_t e = e0 + v * NV;
        const int64_t o = e / a.I;
        return rd.x + ((o * a.C + c) * a.I + (e - o * a.I)) / NV;
    };
    auto fill = [&](unsigned slot_addr, const Round &rd, int64_t v) {
        if (v < nvec) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slot_addr), "l"(src(rd, v)) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per slot, empty or not
    };
    auto take = [&](unsigned slot_addr, int64_t v) {  // the oldest group has landed: bin its vector
        asm volatile("cp.async.wait_group %0;" ::"n"(RING - 1) : "memory");
        if (v < nvec) {
            Vec16<E> w;
            uint32_t *wr = reinterpret_cast<uint32_t *>(&w);
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(wr[0]), "=r"(wr[1]), "=r"(wr[2]), "=r"(wr[3])
                         : "r"(slot_addr)
                         : "memory");
            feed(w, slot_addr);
        }
    };
    Round cur = next_round();
#pragma unroll
    for (int j = 0; j < RING - 1; ++j) fill(ring + j * kSlotBytes, cur, cur.v + j * T);
    while (cur.x != nullptr) {
        const Round nxt = next_round();
#pragma unroll
        for (int j = 0; j < RING; ++j) {
            // the slot emptied one step ago takes the vector RING - 1 steps ahead
            const int rs = (j + RING - 1) % RING;
            if (j == 0)
                fill(ring + rs * kSlotBytes, cur, cur.v + (RING - 1) * T);
            else
                fill(ring + rs * kSlotBytes, nxt, nxt.v + (j - 1) * T);
            take(ring + j * kSlotBytes, cur.v + j * T);
        }
        cur = nxt;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    n_below = __reduce_add_sync(0xffffffffu, n_below);
    n_above = __reduce_add_sync(0xffffffffu, n_above);
    if (lane == 0) {
        if (n_below) atomicAdd(&sh_edge[0], (unsigned long long)n_below);
        if (n_above) atomicAdd(&sh_edge[1], (unsigned long long)n_above);
    }
    if constexpr (MM) {
        if constexpr (F32) {
            fmn = fminf(fmn, rmn);
            fmx = fmaxf(fmx, rmx);
        } else if constexpr (std::is_same<E, __half>::value) {
            fmn = fminf(fmn, fminf(__low2float(rmn), __high2float(rmn)));
            fmx = fmaxf(fmx, fmaxf(__low2float(rmx), __high2float(rmx)));
        } else {
            fmn = fminf(fmn, fminf(__low2float(rmn), __high2float(rmn)));
            fmx = fmaxf(fmx, fmaxf(__low2float(rmx), __high2float(rmx)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            fmn = fminf(fmn, __shfl_xor_sync(0xffffffffu, fmn, o));
            fmx = fmaxf(fmx, __shfl_xor_sync(0xffffffffu, fmx, o));
        }
        if (lane == 0) {
            sh_mm[0][threadIdx.x >> 5] = fmn;
            sh_mm[1][threadIdx.x >> 5] = fmx;
        }
    }
    __syncthreads();
    // merge the replicas: half a warp per bin
    unsigned long long *out = a.counts + c * (int64_t)a.num_bins;
    const int last = a.num_bins - 1;
    for (int b0i = (threadIdx.x >> 5) * 2; b0i <= a.num_bins; b0i += kPrivThreads / 16) {
        const int b = b0i + (lane >> 4);
        unsigned int n32 = b <= a.num_bins ? sh_cnt[b * kPrivCopies + (lane & 15)] : 0u;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) n32 += __shfl_xor_sync(0xffffffffu, n32, o);
        if ((lane & 15) == 0 && b <= a.num_bins) {
            unsigned long long n = n32;
            const int dst = b > last ? last : b;  // row num_bins (v == hi) belongs to the last bin
            if (b == 0) n += sh_edge[0];
            if (b == last) n += sh_edge[1];
            if (n) atomicAdd(out + dst, n);
        }
    }
    if (MM && threadIdx.x == 0) {
        float mn = sh_mm[0][0], mx = sh_mm[1][0];
        for (int w = 1; w < kPrivThreads / 32; ++w) {
            mn = fminf(mn, sh_mm[0][w]);
            mx = fmaxf(mx, sh_mm[1][w]);
        }
        double *p = a.mm_partial + 2 * (c * (int64_t)a.tiles + blockIdx.x);
        p[0] = (double)mn;
        p[1] = (double)mx;
    }
}

// Zeroes the count array.  A kernel rather than a memset node, so that the chain of launches stays
// kernel -> kernel and the programmatic dependency of the histogram kernel has a grid to wait for.
__global__ void __launch_bounds__(kThreads) k_zero_counts(unsigned long long *p, int64_t n) {
    pdl_prologue();
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) p[i] = 0ull;
}
inline int zero_counts(int64_t *counts, int64_t n, cudaStream_t stream) {
    launch_pdl(k_zero_counts, (unsigned)((n + kThreads - 1) / kThreads), kThreads, 0, stream,
               reinterpret_cast<unsigned long long *>(counts), n);
    AB_LAUNCH_OK();
    return AB_OK;
}

constexpr int AB_HIST_ACCUMULATE = 1;   // add to counts instead of overwriting them
constexpr int AB_HIST_MERGE_MINMAX = 2; // fin_min / fin_max: running values over calls

template <int IO>
int launch_histogram_one(const void *const *xs, int num_x, const Canon &canon, int32_t num_bins, const float *lo,
                         const float *hi, const float *below, const float *above, int64_t *counts, void *fin_min,
                         void *fin_max, int flags, const int *run_if, void *scratch, int64_t scratch_bytes,
                         cudaStream_t stream, int *consumed) {
    // bins xs[0] (and, where one launch can take several tensors, up to kMaxBatch of them);
    // *consumed tells how many
    *consumed = 1;
    const void *x = xs[0];
    const int vecw = 16 / dtype_size(IO);
    const bool vect = aligned16(x) && (canon.I % vecw == 0);
    const int v = vect ? vecw : 1;
    const int64_t chan_elems = canon.O * canon.I;
    const int64_t grain = (int64_t)kThreads * kHistUnroll * v;  // elements per CTA sweep
    int64_t tiles = ((int64_t)sm_count() * 8 + canon.C - 1) / canon.C;
    const int64_t max_tiles = (chan_elems + grain - 1) / grain;
    if (tiles > max_tiles) tiles = max_tiles;
    if (tiles < 1) tiles = 1;
    int64_t tile_elems = (chan_elems + tiles - 1) / tiles;
    tile_elems = ((tile_elems + 15) / 16) * 16;
    tiles = (chan_elems + tile_elems - 1) / tile_elems;

    const bool want_mm = fin_min && fin_max;
    const bool accumulate = (flags & AB_HIST_ACCUMULATE) != 0;
    const int merge_mm = (flags & AB_HIST_MERGE_MINMAX) ? 1 : 0;
    // lane-private counters for large histograms
    if constexpr (IO == AB_BF16 || IO == AB_F16 || IO == AB_F32) {
        if (vect && num_bins <= kPrivMaxBins && chan_elems >= kPrivMinElems && canon.C <= 1024) {
            // counters, then the input ring: six slots of 16 bytes per thread when they fit, else two
            const size_t counters = (size_t)(num_bins + 1) * kPrivCopies * sizeof(unsigned int);
            const int ring = counters + 6 * (size_t)kPrivThreads * 16 <= kPrivSmemMax ? 6 : 2;
            const size_t smem = counters + (size_t)ring * kPrivThreads * 16;
            const bool pow2 = (num_bins & (num_bins - 1)) == 0;
            using KernelFn = void (*)(HistPrivArgs);
            KernelFn kernel = nullptr;
            int rc = AB_OK;
#define AB_PICK(MMV, P2V, RV)                                                       \
    if (want_mm == MMV && pow2 == P2V && ring == RV) {                              \
        kernel = k_hist_private<IO, MMV, P2V, RV>;                                  \
        rc = opt_in_smem<k_hist_private<IO, MMV, P2V, RV>>(kPrivSmemMax);           \
    }
            AB_PICK(false, false, 2) AB_PICK(false, false, 6) AB_PICK(false, true, 2) AB_PICK(false, true, 6)
            AB_PICK(true, false, 2) AB_PICK(true, false, 6) AB_PICK(true, true, 2) AB_PICK(true, true, 6)
#undef AB_PICK
            if (rc != AB_OK) return rc;
            int64_t ptiles = (sm_count() + canon.C - 1) / canon.C;
            if (ptiles < 1) ptiles = 1;
            int64_t pt_elems = (chan_elems + ptiles - 1) / ptiles;
            pt_elems = ((pt_elems + 15) / 16) * 16;
            ptiles = (chan_elems + pt_elems - 1) / pt_elems;
            const int64_t need = want_mm ? canon.C * ptiles * 2 * (int64_t)sizeof(double) : 0;
            if (need > 0 && (!scratch || scratch_bytes < need))
                return fail(AB_ERR_SCRATCH, "histogram needs %lld bytes of scratch, got %lld", (long long)need,
                            (long long)scratch_bytes);
            if (!accumulate) {
                rc = zero_counts(counts, canon.C * (int64_t)num_bins, stream);
                if (rc != AB_OK) return rc;
            }
            HistPrivArgs h;
            h.x = x;
            h.num_x = 1;
            h.xs[0] = x;
            if (canon.C == 1) {  // one contiguous statistic: several tensors in one launch
                int n = 1;
                for (; n < num_x && n < kMaxBatch && aligned16(xs[n]); ++n) h.xs[n] = xs[n];
                h.num_x = n;
                *consumed = n;
            }
            h.lo = lo;
            h.hi = hi;
            h.below = below;
            h.above = above;
            h.counts = reinterpret_cast<unsigned long long *>(counts);
            h.mm_partial = want_mm ? static_cast<double *>(scratch) : nullptr;
            h.O = canon.O;
            h.C = canon.C;
            h.I = canon.I;
            h.chan_elems = chan_elems;
            h.tile_elems = pt_elems;
            h.num_bins = num_bins;
            h.tiles = (int)ptiles;
            h.run_if = run_if;
            dim3 grid((unsigned)ptiles, (unsigned)canon.C);
            launch_pdl(kernel, grid, kPrivThreads, smem, stream, h);
            AB_LAUNCH_OK();
            if (want_mm) {
                MinMaxFinishArgs f{h.mm_partial, fin_min, fin_max, canon.C, 1, 0, ptiles, ptiles, merge_mm};
                launch_minmax_finish<IO>(f, stream);
                AB_LAUNCH_OK();
            }
            return AB_OK;
        }
    }
    const int64_t need = want_mm ? canon.C * tiles * 2 * (int64_t)sizeof(double) : 0;
    if (need > 0 && (!scratch || scratch_bytes < need))
        return fail(AB_ERR_SCRATCH, "histogram needs %lld bytes of scratch, got %lld", (long long)need,
                    (long long)scratch_bytes);

    if (!accumulate) {
        const int zrc = zero_counts(counts, canon.C * (int64_t)num_bins, stream);
        if (zrc != AB_OK) return zrc;
    }
    HistArgs a;
    a.x = x;
    a.lo = lo;
    a.hi = hi;
    a.below = below;
    a.above = above;
    a.counts = reinterpret_cast<unsigned long long *>(counts);
    a.mm_partial = want_mm ? static_cast<double *>(scratch) : nullptr;
    a.O = canon.O;
    a.C = canon.C;
    a.I = canon.I;
    a.chan_elems = chan_elems;
    a.tile_elems = tile_elems;
    a.num_bins = num_bins;
    a.tiles = (int)tiles;
    a.run_if = run_if;
    dim3 grid((unsigned)tiles, (unsigned)canon.C);
    const size_t smem = sizeof(unsigned int) * (size_t)num_bins;
    if (vect)
        launch_pdl(k_histogram<IO, true>, grid, kThreads, smem, stream, a);
    else
        launch_pdl(k_histogram<IO, false>, grid, kThreads, smem, stream, a);
    AB_LAUNCH_OK();
    if (want_mm) {
        MinMaxFinishArgs f{a.mm_partial, fin_min, fin_max, canon.C, 1, 0, tiles, tiles, merge_mm};
        launch_minmax_finish<IO>(f, stream);
        AB_LAUNCH_OK();
    }
    return AB_OK;
}

// all tensors of the list, the counts (and the min / max) running over them
template <int IO>
int launch_histogram(const void *const *xs, int num_x, const Canon &canon, int32_t num_bins, const float *lo,
                     const float *hi, const float *below, const float *above, int64_t *counts, void *fin_min,
                     void *fin_max, int flags, const int *run_if, void *scratch, int64_t scratch_bytes,
                     cudaStream_t stream) {
    if (!canon.oci)
        return fail(AB_ERR_UNSUPPORTED, "statistics need a layout that reduces to (outer, channel, inner)");
    if (canon.C > 65535) return fail(AB_ERR_UNSUPPORTED, "at most 65535 histograms per call, got %lld", (long long)canon.C);
    if (run_if && (fin_min || fin_max))
        return fail(AB_ERR_INVALID, "a conditional launch cannot also produce min / max");
    for (int i = 0; i < num_x;) {
        int used = 1;
        const int rc = launch_histogram_one<IO>(xs + i, num_x - i, canon, num_bins, lo, hi, below, above, counts, fin_min,
                                                fin_max, flags, run_if, scratch, scratch_bytes, stream, &used);
        if (rc != AB_OK) return rc;
        i += used;
        flags |= AB_HIST_ACCUMULATE | AB_HIST_MERGE_MINMAX;  // the rest of the list adds to what is there
    }
    return AB_OK;
}

// ---------------------------------------------------------------------------
// Merging an accumulated histogram into a (possibly wider) range, one CTA per histogram: the
// body of _HistogramObserver.merge_stats (encoding_analyzer.py:231-323 of the reference) as one
// launch instead of some sixty small tensor operations.  Every float operation is the one the
// tensor expression performs, in the same order and without contraction: the updated range is
// the batch's range clamped between the growth limit and the current edges; a source bin that
// straddles a destination edge is split proportionally, the first part rounded half to even;
// the new edges are ticks * step + lo.
// ---------------------------------------------------------------------------
// round to the dtype the statistics are kept in, as a tensor operation on that dtype would
__device__ __forceinline__ float rnd_dt(float v, int dt) {
    if (dt == AB_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (dt == AB_F16) return __half2float(__float2half_rn(v));
    return v;
}

struct MergeArgs {
    const float *new_min, *new_max, *cur_min, *cur_max;
    const float *cur_edges;  // [H][n + 1]
    const float *cur_hist;   // [H][n]
    const float *limit;      // [H][2]
    float *out_min, *out_max;
    float *out_carry;        // [H][n]
    float *out_edges;        // [H][n + 1]
    int num_bins;
    int *out_moved;          // [H] or NULL: 1 when the updated range differs from the current edges
    float *out_range;        // [H][4] or NULL: first edge, last edge, and the two rounded to stat_dtype
    int stat_dtype;
    // the batch's min / max in the tensor's own dtype (new_raw_dtype), used when new_min is NULL
    const void *new_raw_min = nullptr, *new_raw_max = nullptr;
    int new_raw_dtype = AB_F32;
};

__device__ __forceinline__ float load_stat(const void *p, int dt, int64_t i) {
    if (dt == AB_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    if (dt == AB_F16) return __half2float(static_cast<const __half *>(p)[i]);
    return static_cast<const float *>(p)[i];
}

__device__ __forceinline__ float min_prop(float a, float b) {  // torch.minimum: NaN propagates
    return (a != a) ? a : ((b != b) ? b : (a < b ? a : b));
}

__global__ void __launch_bounds__(kThreads) k_hist_merge(MergeArgs a) {
    pdl_prologue();
    extern __shared__ float sh_carry[];
    const int n = a.num_bins;
    const int64_t h = blockIdx.x;
    const float *edges = a.cur_edges + h * (int64_t)(n + 1);
    const float *hist = a.cur_hist + h * (int64_t)n;
    const float e0 = edges[0], e_last = edges[n];
    const float bmin = a.new_min ? a.new_min[h] : load_stat(a.new_raw_min, a.new_raw_dtype, h);
    const float bmax = a.new_max ? a.new_max[h] : load_stat(a.new_raw_max, a.new_raw_dtype, h);
    const float umin = clamp_nan(bmin, a.limit[2 * h], e0);
    const float umax = clamp_nan(bmax, e_last, a.limit[2 * h + 1]);
    const bool keep = (umin == a.cur_min[h]) && (umax == a.cur_max[h]);
    const float nf = (float)n;
    const float dw = __fdiv_rn(__fsub_rn(umax, umin), nf);
    const float sw = __fsub_rn(edges[1], edges[0]);
    for (int j = threadIdx.x; j < n; j += kThreads) sh_carry[j] = 0.0f;
    __syncthreads();
    if (!keep) {
        for (int j = threadIdx.x; j < n; j += kThreads) {
            const float src = edges[j], cnt = hist[j];
            int d1 = __float2int_rz(__fdiv_rn(__fsub_rn(src, umin), dw));
            d1 = d1 > n - 1 ? n - 1 : d1;
            const float d1_end = __fadd_rn(umin, __fmul_rn(dw, (float)(d1 + 1)));
            const float part = __fmul_rn(__fdiv_rn(__fsub_rn(d1_end, src), sw), cnt);
            const float first = min_prop(rintf(part), cnt);
            int d2 = __float2int_rz(__fdiv_rn(__fsub_rn(__fadd_rn(src, dw), umin), dw));
            d2 = d2 > n - 1 ? n - 1 : d2;
            const float rest = __fsub_rn(cnt, first);
            const int i1 = d1 < 0 ? 0 : d1, i2 = d2 < 0 ? 0 : d2;
            atomicAdd(&sh_carry[i1], first);
            if (first < cnt) atomicAdd(&sh_carry[i2], rest);
        }
    }
    __syncthreads();
    float *carry = a.out_carry + h * (int64_t)n;
    for (int j = threadIdx.x; j < n; j += kThreads) carry[j] = keep ? hist[j] : sh_carry[j];
    // edges of the merged range; a degenerate range is widened by 0.5 on each side
    const bool same = umin == umax;
    const float lo = same ? __fsub_rn(umin, 0.5f) : umin, hi = same ? __fadd_rn(umax, 0.5f) : umax;
    const float step = __fdiv_rn(__fsub_rn(hi, lo), nf);
    float *oe = a.out_edges + h * (int64_t)(n + 1);
    for (int j = threadIdx.x; j <= n; j += kThreads) oe[j] = __fadd_rn(__fmul_rn((float)j, step), lo);
    if (threadIdx.x == 0) {
        a.out_min[h] = umin;
        a.out_max[h] = umax;
        // counts taken over [edges[0], edges[n]] are the counts over the updated range exactly when
        // the range still ends where the edges do
        if (a.out_moved) a.out_moved[h] = (umin == e0 && umax == e_last) ? 0 : 1;
        if (a.out_range) {
            const float first = __fadd_rn(__fmul_rn(0.0f, step), lo), last = __fadd_rn(__fmul_rn(nf, step), lo);
            a.out_range[4 * h] = first;
            a.out_range[4 * h + 1] = last;
            a.out_range[4 * h + 2] = rnd_dt(first, a.stat_dtype);
            a.out_range[4 * h + 3] = rnd_dt(last, a.stat_dtype);
        }
    }
}

// hist[h][b] = carry[h][b] + (moved[h] ? redo : counts)[h][b]: the accumulated counts moved into the
// updated range plus the batch's counts from whichever pass is valid for it
__global__ void __launch_bounds__(kThreads) k_hist_combine(const long long *counts, const long long *redo, const float *carry,
                                                           const int *moved, float *hist, int num_bins) {
    pdl_prologue();
    const int h = blockIdx.y;
    const int b = blockIdx.x * kThreads + threadIdx.x;
    if (b >= num_bins) return;
    const int64_t i = (int64_t)h * num_bins + b;
    const long long n = moved[h] ? redo[i] : counts[i];
    hist[i] = __fadd_rn((float)n, carry[i]);
}

// ---------------------------------------------------------------------------
// SQNR sweep: noise of every (delta, offset) candidate against a histogram
// ---------------------------------------------------------------------------
struct SweepArgs {
    const float *hist, *edge0, *width, *deltas, *offsets;
    int offsets_per_hist;
    int num_bins, num_cand;
    float num_steps, gamma;
    int use_gamma;
    float p;  // exponent of the error
    float *noise;
};

constexpr int kSweepThreads = 128;

// |err|^p the way torch.pow evaluates a scalar exponent: 2 and 3 by multiplication, 0.5 as a
// square root, 1 as the value itself, anything else through pow
__device__ __forceinline__ float lp_error(float err, float p) {
    if (p == 2.0f) return __fmul_rn(err, err);
    if (p == 1.0f) return err;
    if (p == 3.0f) return __fmul_rn(__fmul_rn(err, err), err);
    if (p == 0.5f) return __fsqrt_rn(err);
    return powf(err, p);
}

__global__ void __launch_bounds__(kSweepThreads) k_sqnr_sweep(SweepArgs a) {
    pdl_prologue();
    const int cand = blockIdx.x, h = blockIdx.y;
    const float delta = a.deltas[(int64_t)h * a.num_cand + cand];
    const float offset = a.offsets[(a.offsets_per_hist ? (int64_t)h * a.num_cand : 0) + cand];
    const float width = a.width[h];
    const float mid0 = __fadd_rn(a.edge0[h], __fdiv_rn(width, 2.0f));
    const float *hist = a.hist + (int64_t)h * a.num_bins;
    double acc = 0.0;
    for (int b = threadIdx.x; b < a.num_bins; b += kSweepThreads) {
        const float mid = __fadd_rn(mid0, __fmul_rn(width, (float)b));
        float q = rintf(__fsub_rn(__fdiv_rn(mid, delta), offset));
        const bool clipped = (q < 0.0f) || (q > a.num_steps);
        q = clamp_nan(q, 0.0f, a.num_steps);
        q = __fmul_rn(__fadd_rn(q, offset), delta);
        float err = fabsf(__fsub_rn(q, mid));
        err = __fmul_rn(lp_error(err, a.p), hist[b]);
        if (a.use_gamma && clipped) err = __fmul_rn(err, a.gamma);
        acc += (double)err;
    }
    acc = warp_sum(acc);
    __shared__ double sh[kSweepThreads / 32];
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < kSweepThreads / 32; ++w) t += sh[w];
        a.noise[(int64_t)h * a.num_cand + cand] = (float)t;
    }
}

__global__ void __launch_bounds__(kSweepThreads) k_argmin(const float *noise, int num_cand, int *best) {
    pdl_prologue();
    const int h = blockIdx.x;
    const float *n = noise + (int64_t)h * num_cand;
    float bv = INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < num_cand; i += kSweepThreads) {
        const float v = n[i];
        if (v < bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    __shared__ float sv[kSweepThreads];
    __shared__ int si[kSweepThreads];
    sv[threadIdx.x] = bv;
    si[threadIdx.x] = bi;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int t = 1; t < kSweepThreads; ++t) {
            const float v = sv[t];
            const int i = si[t];
            if (i == 0x7fffffff) continue;
            if (bi == 0x7fffffff || v < bv || (v == bv && i < bi)) {
                bv = v;
                bi = i;
            }
        }
        best[h] = bi == 0x7fffffff ? 0 : bi;
    }
}


// ---------------------------------------------------------------------------
// Small-tensor bookkeeping of a calibration as single launches (it is what a many-GPU calibration
// spends its time on once the passes over the data are short)
// ---------------------------------------------------------------------------
struct EdgesArgs {
    const float *mn, *mx;  // [H] observed range (finite min / max), exact in the statistics dtype
    int num_hist, num_bins, stat_dtype;
    float growth;          // range limit = edges -/+ span * growth / 2
    float *edges;          // [H][num_bins + 1]
    float *lo, *hi, *below, *above, *limit;  // [H], [H], [H], [H], [H][2]; limit may be NULL
};

// _HistogramObserver._create_bin_edges (encoding_analyzer.py:221-229) and what the histogram pass
// needs from it: first / last edge, the same two rounded to the tensor dtype for the outlier
// comparisons, and the growth limit of the range (:244-257).  One thread per edge.
__global__ void __launch_bounds__(kThreads) k_hist_edges(EdgesArgs a) {
    pdl_prologue();
    const int h = blockIdx.y;
    const float mn = a.mn[h], mx = a.mx[h];
    const bool same = mn == mx;
    const float lo = same ? rnd_dt(__fsub_rn(mn, 0.5f), a.stat_dtype) : mn;
    const float hi = same ? rnd_dt(__fadd_rn(mx, 0.5f), a.stat_dtype) : mx;
    const float step = __fdiv_rn(__fsub_rn(hi, lo), (float)a.num_bins);
    const int j = blockIdx.x * kThreads + threadIdx.x;
    if (j <= a.num_bins) a.edges[(int64_t)h * (a.num_bins + 1) + j] = __fadd_rn(__fmul_rn((float)j, step), lo);
    if (j == 0) {
        const float e0 = __fadd_rn(__fmul_rn(0.0f, step), lo);
        const float e1 = __fadd_rn(__fmul_rn((float)a.num_bins, step), lo);
        a.lo[h] = e0;
        a.hi[h] = e1;
        a.below[h] = rnd_dt(e0, a.stat_dtype);
        a.above[h] = rnd_dt(e1, a.stat_dtype);
        if (a.limit) {
            const float half = __fmul_rn(__fmul_rn(__fsub_rn(e1, e0), a.growth), 0.5f);
            a.limit[2 * h] = __fsub_rn(e0, half);
            a.limit[2 * h + 1] = __fadd_rn(e1, half);
        }
    }
}

// The (delta, offset) test candidates of the SQNR / TF-enhanced analyzers, formed on the device with
// the reference's operations in the reference's order (_pick_test_candidates,
// _pick_test_candidates_asymmetric / _symmetric, _clamp_delta_offset_values,
// encoding_analyzer.py:728-820).
struct CandArgs {
    const float *stat_min, *stat_max;  // [H]
    const float *base_offsets;         // [n_base] asymmetric offsets before the observed one is appended
    int n_base, n_delta, symmetric, stat_dtype;
    float num_steps, min_scale, widen;  // widen = (float)(min_scale * num_steps)
    float sym_offset;
};

__device__ __forceinline__ void sqnr_candidate(const CandArgs &c, int h, int cand, float &delta, float &offset) {
    const int dt = c.stat_dtype;
    float mn = fminf(c.stat_min[h], 0.0f), mx = fmaxf(c.stat_max[h], 0.0f);
    mx = fmaxf(mx, rnd_dt(__fadd_rn(mn, c.widen), dt));
    if (c.symmetric) {
        const float max_delta = __fdiv_rn(rnd_dt(__fmul_rn(2.0f, fmaxf(mx, -mn)), dt), c.num_steps);
        const float d = __fdiv_rn(__fmul_rn(max_delta, (float)(cand + 1)), (float)(c.n_delta - 1));
        delta = fmaxf(d, c.min_scale);
        offset = c.sym_offset;
        return;
    }
    const int n_off = c.n_base + 1;
    const int k = cand / n_off, o = cand - k * n_off;
    const float max_delta = __fdiv_rn(rnd_dt(__fsub_rn(mx, mn), dt), c.num_steps);
    const float obs_offset = rintf(__fdiv_rn(mn, max_delta));
    const float obs_min = __fmul_rn(max_delta, obs_offset);
    const float obs_max = __fadd_rn(obs_min, __fmul_rn(max_delta, c.num_steps));
    const float dk = __fdiv_rn(__fmul_rn(max_delta, (float)(k + 1)), (float)(c.n_delta - 1));
    const float off = o < c.n_base ? c.base_offsets[o] : obs_offset;
    float tmin = __fmul_rn(dk, off);
    float tmax = __fadd_rn(tmin, __fmul_rn(dk, c.num_steps));
    tmin = fmaxf(obs_min, tmin);
    tmax = fminf(obs_max, tmax);
    delta = fmaxf(__fdiv_rn(__fsub_rn(tmax, tmin), c.num_steps), c.min_scale);
    offset = rintf(__fdiv_rn(tmin, delta));
}

struct SweepGenArgs {
    CandArgs cand;
    const float *hist;   // [H][num_bins]
    const float *edges;  // [H][num_bins + 1]
    int num_bins, num_cand;
    float gamma;
    int use_gamma;
    float p;                   // exponent of the error
    float *noise;              // [H][num_cand]
    float *deltas, *offsets;   // [H][num_cand] or NULL
    float *enc_min, *enc_max;  // [H]
    int *best;                 // [H]
};

__global__ void __launch_bounds__(kSweepThreads) k_sqnr_sweep_gen(SweepGenArgs a) {
    pdl_prologue();
    const int cand = blockIdx.x, h = blockIdx.y;
    float delta, offset;
    sqnr_candidate(a.cand, h, cand, delta, offset);
    if (threadIdx.x == 0 && a.deltas) {
        a.deltas[(int64_t)h * a.num_cand + cand] = delta;
        a.offsets[(int64_t)h * a.num_cand + cand] = offset;
    }
    const float *edges = a.edges + (int64_t)h * (a.num_bins + 1);
    const float width = __fsub_rn(edges[1], edges[0]);
    const float mid0 = __fadd_rn(edges[0], __fdiv_rn(width, 2.0f));
    const float *hist = a.hist + (int64_t)h * a.num_bins;
    const float num_steps = a.cand.num_steps;
    double acc = 0.0;
    for (int b = threadIdx.x; b < a.num_bins; b += kSweepThreads) {
        const float mid = __fadd_rn(mid0, __fmul_rn(width, (float)b));
        float q = rintf(__fsub_rn(__fdiv_rn(mid, delta), offset));
        const bool clipped = (q < 0.0f) || (q > num_steps);
        q = clamp_nan(q, 0.0f, num_steps);
        q = __fmul_rn(__fadd_rn(q, offset), delta);
        float err = fabsf(__fsub_rn(q, mid));
        err = __fmul_rn(lp_error(err, a.p), hist[b]);
        if (a.use_gamma && clipped) err = __fmul_rn(err, a.gamma);
        acc += (double)err;
    }
    acc = warp_sum(acc);
    __shared__ double sh[kSweepThreads / 32];
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < kSweepThreads / 32; ++w) t += sh[w];
        a.noise[(int64_t)h * a.num_cand + cand] = (float)t;
    }
}

// arg-min over the candidates of one histogram (lowest index among equal minima) and the encoding
// range of the winner: min = offset * delta, max = min + num_steps * delta (:718-726)
__global__ void __launch_bounds__(kSweepThreads) k_sqnr_pick(SweepGenArgs a) {
    pdl_prologue();
    const int h = blockIdx.x;
    const float *n = a.noise + (int64_t)h * a.num_cand;
    float bv = INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < a.num_cand; i += kSweepThreads) {
        const float v = n[i];
        if (v < bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    __shared__ float sv[kSweepThreads];
    __shared__ int si[kSweepThreads];
    sv[threadIdx.x] = bv;
    si[threadIdx.x] = bi;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int t = 1; t < kSweepThreads; ++t) {
            const float v = sv[t];
            const int i = si[t];
            if (i == 0x7fffffff) continue;
            if (bi == 0x7fffffff || v < bv || (v == bv && i < bi)) {
                bv = v;
                bi = i;
            }
        }
        if (bi == 0x7fffffff) bi = 0;
        float delta, offset;
        sqnr_candidate(a.cand, h, bi, delta, offset);
        const float emin = __fmul_rn(offset, delta);
        a.best[h] = bi;
        a.enc_min[h] = emin;
        a.enc_max[h] = __fadd_rn(emin, __fmul_rn(a.cand.num_steps, delta));
    }
}

}  // namespace
}  // namespace ab

extern "C" int64_t aimet_b200_stats_scratch_bytes(const ab_layout *layout, int io_dtype) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (ab::dtype_size(io_dtype) == 0) return ab::fail(AB_ERR_INVALID, "unknown io_dtype %d", io_dtype);
    if (canon.numel == 0 || !canon.oci) return 0;
    const ab::ReducePlan pa = ab::plan_reduce(canon, io_dtype, true, ab::kStatChunkMult);
    const ab::ReducePlan pb = ab::plan_reduce(canon, io_dtype, false, ab::kStatChunkMult);
    int64_t n = pa.npartial > pb.npartial ? pa.npartial : pb.npartial;
    // histogram min/max partials: at most 8 * SMs tiles in total, plus one per channel
    const int64_t hist = (int64_t)ab::sm_count() * 8 + 2 * canon.C;
    if (hist > n) n = hist;
    int64_t bytes = n * 2 * (int64_t)sizeof(double);
    return bytes;
}

static int minmax_entry(const void *x, const ab_layout *layout, int io_dtype, int finite_only, int merge,
                        void *min_out, void *max_out, void *scratch, int64_t scratch_bytes, void *stream) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (canon.numel == 0) return ab::fail(AB_ERR_INVALID, "min/max of an empty tensor is undefined");
    if (!x || !min_out || !max_out) return ab::fail(AB_ERR_INVALID, "x, min_out and max_out must not be NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (io_dtype) {
        case AB_F32: return ab::launch_minmax<AB_F32>(x, canon, finite_only, merge, min_out, max_out, scratch, scratch_bytes, st);
        case AB_F16: return ab::launch_minmax<AB_F16>(x, canon, finite_only, merge, min_out, max_out, scratch, scratch_bytes, st);
        case AB_BF16: return ab::launch_minmax<AB_BF16>(x, canon, finite_only, merge, min_out, max_out, scratch, scratch_bytes, st);
        case AB_F64: return ab::launch_minmax<AB_F64>(x, canon, finite_only, merge, min_out, max_out, scratch, scratch_bytes, st);
    }
    return ab::fail(AB_ERR_INVALID, "unknown io_dtype %d", io_dtype);
}

extern "C" int aimet_b200_minmax_batches(const void *const *xs, int32_t num_tensors, const ab_layout *layout,
                                         int io_dtype, int finite_only, int merge, void *min_io, void *max_io,
                                         void *scratch, int64_t scratch_bytes, void *stream) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (canon.numel == 0) return ab::fail(AB_ERR_INVALID, "min/max of an empty tensor is undefined");
    if (num_tensors <= 0 || !xs || !min_io || !max_io)
        return ab::fail(AB_ERR_INVALID, "need at least one tensor and both outputs");
    for (int i = 0; i < num_tensors; ++i)
        if (!xs[i]) return ab::fail(AB_ERR_INVALID, "tensor %d of the list is NULL", i);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (io_dtype) {
        case AB_F32: return ab::launch_minmax_list<AB_F32>(xs, num_tensors, canon, finite_only, merge, min_io, max_io, scratch, scratch_bytes, st);
        case AB_F16: return ab::launch_minmax_list<AB_F16>(xs, num_tensors, canon, finite_only, merge, min_io, max_io, scratch, scratch_bytes, st);
        case AB_BF16: return ab::launch_minmax_list<AB_BF16>(xs, num_tensors, canon, finite_only, merge, min_io, max_io, scratch, scratch_bytes, st);
        case AB_F64: return ab::launch_minmax_list<AB_F64>(xs, num_tensors, canon, finite_only, merge, min_io, max_io, scratch, scratch_bytes, st);
    }
    return ab::fail(AB_ERR_INVALID, "unknown io_dtype %d", io_dtype);
}

extern "C" int aimet_b200_minmax(const void *x, const ab_layout *layout, int io_dtype, int finite_only,
                                 void *min_out, void *max_out, void *scratch, int64_t scratch_bytes,
                                 void *stream) {
    return minmax_entry(x, layout, io_dtype, finite_only, 0, min_out, max_out, scratch, scratch_bytes, stream);
}

extern "C" int aimet_b200_minmax_running(const void *x, const ab_layout *layout, int io_dtype, int finite_only,
                                         void *min_io, void *max_io, void *scratch, int64_t scratch_bytes,
                                         void *stream) {
    return minmax_entry(x, layout, io_dtype, finite_only, 1, min_io, max_io, scratch, scratch_bytes, stream);
}

extern "C" int aimet_b200_histogram_batches(const void *const *xs, int32_t num_tensors, const ab_layout *layout,
                                            int io_dtype, int32_t num_bins, const float *lo, const float *hi,
                                            const float *below, const float *above, int64_t *counts, void *fin_min,
                                            void *fin_max, int32_t flags, const int32_t *run_if_nonzero, void *scratch,
                                            int64_t scratch_bytes, void *stream) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (num_bins <= 0 || num_bins > 8192)
        return ab::fail(AB_ERR_UNSUPPORTED, "num_bins must be in [1, 8192], got %d", num_bins);
    if (canon.numel == 0) return ab::fail(AB_ERR_INVALID, "histogram of an empty tensor is undefined");
    if (num_tensors <= 0 || !xs) return ab::fail(AB_ERR_INVALID, "need at least one tensor");
    for (int i = 0; i < num_tensors; ++i)
        if (!xs[i]) return ab::fail(AB_ERR_INVALID, "tensor %d of the list is NULL", i);
    if (!lo || !hi || !below || !above || !counts)
        return ab::fail(AB_ERR_INVALID, "lo, hi, below, above and counts must not be NULL");
    if (flags & ~3) return ab::fail(AB_ERR_INVALID, "unknown flags %d", (int)flags);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (io_dtype) {
        case AB_F32:
            return ab::launch_histogram<AB_F32>(xs, num_tensors, canon, num_bins, lo, hi, below, above, counts, fin_min, fin_max, flags, run_if_nonzero, scratch, scratch_bytes, st);
        case AB_F16:
            return ab::launch_histogram<AB_F16>(xs, num_tensors, canon, num_bins, lo, hi, below, above, counts, fin_min, fin_max, flags, run_if_nonzero, scratch, scratch_bytes, st);
        case AB_BF16:
            return ab::launch_histogram<AB_BF16>(xs, num_tensors, canon, num_bins, lo, hi, below, above, counts, fin_min, fin_max, flags, run_if_nonzero, scratch, scratch_bytes, st);
    }
    return ab::fail(AB_ERR_UNSUPPORTED, "histogram supports float32, float16 and bfloat16 inputs");
}

extern "C" int aimet_b200_histogram_ex(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                                       const float *lo, const float *hi, const float *below,
                                       const float *above, int64_t *counts, void *fin_min, void *fin_max,
                                       int32_t flags, void *scratch, int64_t scratch_bytes, void *stream) {
    if (!x) return ab::fail(AB_ERR_INVALID, "x must not be NULL");
    return aimet_b200_histogram_batches(&x, 1, layout, io_dtype, num_bins, lo, hi, below, above, counts, fin_min,
                                        fin_max, flags, nullptr, scratch, scratch_bytes, stream);
}

extern "C" int aimet_b200_histogram(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                                    const float *lo, const float *hi, const float *below,
                                    const float *above, int64_t *counts, void *fin_min, void *fin_max,
                                    void *scratch, int64_t scratch_bytes, void *stream) {
    return aimet_b200_histogram_ex(x, layout, io_dtype, num_bins, lo, hi, below, above, counts, fin_min, fin_max, 0,
                                   scratch, scratch_bytes, stream);
}

extern "C" int aimet_b200_sqnr_sweep(const float *hist, const float *edge0, const float *width,
                                     const float *deltas, const float *offsets, int32_t offsets_per_hist,
                                     int32_t num_hist, int32_t num_bins, int32_t num_cand, double num_steps,
                                     double gamma, double p, float *noise_out, int32_t *best_out, void *stream) {
    if (num_hist <= 0 || num_bins <= 0 || num_cand <= 0)
        return ab::fail(AB_ERR_INVALID, "num_hist, num_bins and num_cand must be positive");
    if (!(p > 0)) return ab::fail(AB_ERR_INVALID, "the error exponent p must be positive");
    if (num_hist > 65535) return ab::fail(AB_ERR_UNSUPPORTED, "at most 65535 histograms per call");
    if (!hist || !edge0 || !width || !deltas || !offsets || !noise_out || !best_out)
        return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ab::SweepArgs a;
    a.hist = hist;
    a.edge0 = edge0;
    a.width = width;
    a.deltas = deltas;
    a.offsets = offsets;
    a.offsets_per_hist = offsets_per_hist;
    a.num_bins = num_bins;
    a.num_cand = num_cand;
    a.num_steps = (float)num_steps;
    a.gamma = (float)gamma;
    a.use_gamma = gamma != 1.0;
    a.p = (float)p;
    a.noise = noise_out;
    dim3 grid((unsigned)num_cand, (unsigned)num_hist);
    ab::launch_pdl(ab::k_sqnr_sweep, grid, ab::kSweepThreads, 0, st, a);
    AB_LAUNCH_OK();
    ab::launch_pdl(ab::k_argmin, (unsigned)num_hist, ab::kSweepThreads, 0, st, noise_out, num_cand, best_out);
    AB_LAUNCH_OK();
    return AB_OK;
}

extern "C" int aimet_b200_histogram_merge_ex(const float *new_min, const float *new_max, const float *cur_min,
                                             const float *cur_max, const float *cur_edges, const float *cur_hist,
                                             const float *range_limit, int32_t num_hist, int32_t num_bins,
                                             float *out_min, float *out_max, float *out_carry, float *out_edges,
                                             int32_t *out_moved, float *out_range, int stat_dtype, void *stream) {
    if (num_hist <= 0 || num_bins <= 0) return ab::fail(AB_ERR_INVALID, "num_hist and num_bins must be positive");
    if (num_bins > 8192) return ab::fail(AB_ERR_UNSUPPORTED, "at most 8192 bins, got %d", (int)num_bins);
    if (!new_min || !new_max || !cur_min || !cur_max || !cur_edges || !cur_hist || !range_limit || !out_min || !out_max ||
        !out_carry || !out_edges)
        return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    ab::MergeArgs a{new_min, new_max, cur_min, cur_max, cur_edges, cur_hist, range_limit,
                    out_min, out_max, out_carry, out_edges, num_bins, out_moved, out_range, stat_dtype};
    ab::launch_pdl(ab::k_hist_merge, (unsigned)num_hist, ab::kThreads, sizeof(float) * (size_t)num_bins,
                   static_cast<cudaStream_t>(stream), a);
    AB_LAUNCH_OK();
    return AB_OK;
}

extern "C" int aimet_b200_histogram_update(const void *x, const ab_layout *layout, int io_dtype, int32_t num_bins,
                                           const float *cur_hist, const float *cur_edges, const float *cur_min,
                                           const float *cur_max, const float *cur_range, const float *range_limit,
                                           float *new_hist, float *new_edges, float *new_min, float *new_max,
                                           float *new_range, void *batch_min, void *batch_max, int64_t *counts,
                                           int64_t *redo, float *carry, int32_t *moved, void *scratch,
                                           int64_t scratch_bytes, void *stream) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (num_bins <= 0 || num_bins > 8192)
        return ab::fail(AB_ERR_UNSUPPORTED, "num_bins must be in [1, 8192], got %d", num_bins);
    if (canon.numel == 0) return ab::fail(AB_ERR_INVALID, "histogram of an empty tensor is undefined");
    if (!canon.oci || canon.C != 1)
        return ab::fail(AB_ERR_UNSUPPORTED, "the one-call update serves a single (per-tensor) histogram");
    if (io_dtype != AB_F32 && io_dtype != AB_F16 && io_dtype != AB_BF16)
        return ab::fail(AB_ERR_UNSUPPORTED, "the one-call update takes float32, float16 or bfloat16 tensors");
    if (!x || !cur_hist || !cur_edges || !cur_min || !cur_max || !cur_range || !range_limit || !new_hist || !new_edges ||
        !new_min || !new_max || !new_range || !batch_min || !batch_max || !counts || !redo || !carry || !moved)
        return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // 1. the batch against the current range, and its own finite min / max
    const void *xs[1] = {x};
#define AB_BIN(LO, COUNTS, MN, MX, RUN_IF)                                                                              \
    (io_dtype == AB_F32    ? ab::launch_histogram<AB_F32>(xs, 1, canon, num_bins, (LO), (LO) + 1, (LO) + 2, (LO) + 3,   \
                                                          (COUNTS), (MN), (MX), 0, (RUN_IF), scratch, scratch_bytes, st) \
     : io_dtype == AB_F16  ? ab::launch_histogram<AB_F16>(xs, 1, canon, num_bins, (LO), (LO) + 1, (LO) + 2, (LO) + 3,   \
                                                          (COUNTS), (MN), (MX), 0, (RUN_IF), scratch, scratch_bytes, st) \
                           : ab::launch_histogram<AB_BF16>(xs, 1, canon, num_bins, (LO), (LO) + 1, (LO) + 2, (LO) + 3,  \
                                                           (COUNTS), (MN), (MX), 0, (RUN_IF), scratch, scratch_bytes, st))
    rc = AB_BIN(cur_range, counts, batch_min, batch_max, nullptr);
    if (rc != AB_OK) return rc;
    // 2. the accumulated histogram moved into the range that also covers the batch
    ab::MergeArgs m{nullptr, nullptr, cur_min, cur_max, cur_edges, cur_hist, range_limit,
                    new_min, new_max, carry, new_edges, num_bins, moved, new_range, io_dtype};
    m.new_raw_min = batch_min;
    m.new_raw_max = batch_max;
    m.new_raw_dtype = io_dtype;
    ab::launch_pdl(ab::k_hist_merge, 1u, ab::kThreads, sizeof(float) * (size_t)num_bins, st, m);
    AB_LAUNCH_OK();
    // 3. if the range moved, the batch again over the new range (skipped on the device otherwise)
    rc = AB_BIN(new_range, redo, nullptr, nullptr, moved);
    if (rc != AB_OK) return rc;
#undef AB_BIN
    // 4. counts of the batch + carried counts
    return aimet_b200_histogram_combine(counts, redo, carry, moved, 1, num_bins, new_hist, stream);
}

extern "C" int aimet_b200_histogram_edges(const float *min, const float *max, int32_t num_hist, int32_t num_bins,
                                          int stat_dtype, double growth_limit, float *edges, float *lo, float *hi,
                                          float *below, float *above, float *range_limit, void *stream) {
    if (num_hist <= 0 || num_bins <= 0) return ab::fail(AB_ERR_INVALID, "num_hist and num_bins must be positive");
    if (num_hist > 65535) return ab::fail(AB_ERR_UNSUPPORTED, "at most 65535 histograms per call");
    if (!min || !max || !edges || !lo || !hi || !below || !above) return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    ab::EdgesArgs a{min, max, num_hist, num_bins, stat_dtype, (float)growth_limit, edges, lo, hi, below, above, range_limit};
    dim3 grid((unsigned)((num_bins + 1 + ab::kThreads - 1) / ab::kThreads), (unsigned)num_hist);
    ab::launch_pdl(ab::k_hist_edges, grid, ab::kThreads, 0, static_cast<cudaStream_t>(stream), a);
    AB_LAUNCH_OK();
    return AB_OK;
}

extern "C" int aimet_b200_sqnr_encodings(const float *hist, const float *edges, const float *stat_min,
                                         const float *stat_max, const float *base_offsets, int32_t num_base_offsets,
                                         int32_t num_deltas, int32_t symmetric, int stat_dtype, int32_t num_hist,
                                         int32_t num_bins, double num_steps, double gamma, double p, double min_scale,
                                         float *noise_out, float *deltas_out, float *offsets_out, float *enc_min_out,
                                         float *enc_max_out, int32_t *best_out, void *stream) {
    if (num_hist <= 0 || num_bins <= 0 || num_deltas < 2)
        return ab::fail(AB_ERR_INVALID, "num_hist and num_bins must be positive, num_deltas at least 2");
    if (!(p > 0)) return ab::fail(AB_ERR_INVALID, "the error exponent p must be positive");
    if (num_hist > 65535) return ab::fail(AB_ERR_UNSUPPORTED, "at most 65535 histograms per call");
    if (!symmetric && (num_base_offsets <= 0 || !base_offsets))
        return ab::fail(AB_ERR_INVALID, "asymmetric candidates need the offset grid");
    if (!hist || !edges || !stat_min || !stat_max || !noise_out || !enc_min_out || !enc_max_out || !best_out)
        return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    if ((deltas_out == nullptr) != (offsets_out == nullptr))
        return ab::fail(AB_ERR_INVALID, "deltas_out and offsets_out go together");
    ab::SweepGenArgs a;
    a.cand.stat_min = stat_min;
    a.cand.stat_max = stat_max;
    a.cand.base_offsets = base_offsets;
    a.cand.n_base = symmetric ? 0 : num_base_offsets;
    a.cand.n_delta = num_deltas;
    a.cand.symmetric = symmetric;
    a.cand.stat_dtype = stat_dtype;
    a.cand.num_steps = (float)num_steps;
    a.cand.min_scale = (float)min_scale;
    a.cand.widen = (float)(min_scale * num_steps);
    a.cand.sym_offset = (float)floor(-num_steps / 2.0);
    a.hist = hist;
    a.edges = edges;
    a.num_bins = num_bins;
    a.num_cand = symmetric ? num_deltas : num_deltas * (num_base_offsets + 1);
    a.gamma = (float)gamma;
    a.use_gamma = gamma != 1.0;
    a.p = (float)p;
    a.noise = noise_out;
    a.deltas = deltas_out;
    a.offsets = offsets_out;
    a.enc_min = enc_min_out;
    a.enc_max = enc_max_out;
    a.best = best_out;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)a.num_cand, (unsigned)num_hist);
    ab::launch_pdl(ab::k_sqnr_sweep_gen, grid, ab::kSweepThreads, 0, st, a);
    AB_LAUNCH_OK();
    ab::launch_pdl(ab::k_sqnr_pick, (unsigned)num_hist, ab::kSweepThreads, 0, st, a);
    AB_LAUNCH_OK();
    return AB_OK;
}

extern "C" int aimet_b200_histogram_merge(const float *new_min, const float *new_max, const float *cur_min,
                                          const float *cur_max, const float *cur_edges, const float *cur_hist,
                                          const float *range_limit, int32_t num_hist, int32_t num_bins, float *out_min,
                                          float *out_max, float *out_carry, float *out_edges, void *stream) {
    return aimet_b200_histogram_merge_ex(new_min, new_max, cur_min, cur_max, cur_edges, cur_hist, range_limit, num_hist,
                                         num_bins, out_min, out_max, out_carry, out_edges, nullptr, nullptr, AB_F32, stream);
}

extern "C" int aimet_b200_histogram_combine(const int64_t *counts, const int64_t *redo, const float *carry,
                                            const int32_t *moved, int32_t num_hist, int32_t num_bins, float *hist_out,
                                            void *stream) {
    if (num_hist <= 0 || num_bins <= 0) return ab::fail(AB_ERR_INVALID, "num_hist and num_bins must be positive");
    if (num_hist > 65535) return ab::fail(AB_ERR_UNSUPPORTED, "at most 65535 histograms per call");
    if (!counts || !redo || !carry || !moved || !hist_out) return ab::fail(AB_ERR_INVALID, "NULL pointer argument");
    dim3 grid((unsigned)((num_bins + ab::kThreads - 1) / ab::kThreads), (unsigned)num_hist);
    ab::launch_pdl(ab::k_hist_combine, grid, ab::kThreads, 0, static_cast<cudaStream_t>(stream),
                   reinterpret_cast<const long long *>(counts), reinterpret_cast<const long long *>(redo), carry, moved,
                   hist_out, num_bins);
    AB_LAUNCH_OK();
    return AB_OK;
}
