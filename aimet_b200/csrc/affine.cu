// Affine quantize / dequantize / quantize-dequantize: one fused elementwise
// pass forward, one fused pass backward (input gradient + deterministic
// reduction of the scale / offset gradients).
//
// Arithmetic follows QuantizeFunc / DequantizeFunc / QuantDequantFunc of the
// reference (quantization/affine/backends/torch_builtins.py:588-831) step by
// step, including the re-rounding to the internal dtype after every step when
// that dtype is float16 / bfloat16.
#include <mutex>

#include "affine_math.cuh"
#include "common.cuh"

namespace ab {
namespace {

// ---------------------------------------------------------------------------
// forward kernels
// ---------------------------------------------------------------------------
struct FwdArgs {
    const void *x;
    void *y;
    ParamPtr scale, offset;
    int64_t numel;
    ChanMap cm;
    double qmin, qmax, zps;
    int exact_edges;
};

template <int IO, int CT, int OP, bool VECT>
__global__ void __launch_bounds__(kThreads) k_fwd_oci(FwdArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
    const int64_t nvec = a.numel / VEC;
    const bool uniform = (a.cm.I % VEC) == 0;
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    E *__restrict__ yp = static_cast<E *>(a.y);

    const int64_t base = (int64_t)blockIdx.x * (kThreads * kFwdUnroll) + threadIdx.x;
    if constexpr (VECT) {
        Vec16<E> xv[kFwdUnroll];
#pragma unroll
        for (int u = 0; u < kFwdUnroll; ++u) {
            int64_t v = base + (int64_t)u * kThreads;
            if (v < nvec) xv[u] = reinterpret_cast<const Vec16<E> *>(xp)[v];
        }
#pragma unroll
        for (int u = 0; u < kFwdUnroll; ++u) {
            int64_t v = base + (int64_t)u * kThreads;
            if (v >= nvec) continue;
            Vec16<E> yv;
            if (uniform) {
                const Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v * VEC), g);
                constexpr int NV = 16 / (int)sizeof(E);
                T f[NV];
                VecCvt<T, E>::unpack(xv[u], f);
                bool done = false;
                if constexpr (CT != AB_F64 && NV >= 2 && (OP == OP_QDQ || OP == OP_Q)) {
                    if (vec_fast_ok<CT>(e, g)) {
                        fwd_vec_fast<CT, OP, NV, true>(f, e);
                        done = true;
                    }
                }
                if (!done) {
#pragma unroll
                    for (int i = 0; i + 1 < NV; i += 2) fwd_pair<CT, OP>(f[i], f[i + 1], e, g);
                }
                VecCvt<T, E>::pack(f, yv);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v * VEC + i), g);
                    yv.v[i] = C::store(fwd_elem<CT, OP>(C::load(xv[u].v[i]), e, g));
                }
            }
            reinterpret_cast<Vec16<E> *>(yp)[v] = yv;
        }
    } else {
#pragma unroll
        for (int u = 0; u < kFwdUnroll; ++u) {
            int64_t v = base + (int64_t)u * kThreads;
            if (v >= nvec) continue;
            Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v), g);
            yp[v] = C::store(fwd_elem<CT, OP>(C::load(xp[v]), e, g));
        }
    }
}

// ---------------------------------------------------------------------------
// Segment kernels: a group of threads (a power of two) per contiguous run of elements that share
// a parameter ("pseudo-segment"; long runs are cut into several).  A thread sets up its parameter
// pair once, picks one of the loop bodies below and streams 16-byte vectors of its run.
// ---------------------------------------------------------------------------
struct SegPos {
    int64_t s;      // pseudo-segment index
    int64_t v0;     // first 16-byte vector of the run
    int64_t param;  // parameter index
    int nv;         // vectors in the run
    int lane;       // position in the group
    bool valid;
};

template <int VEC>
__device__ __forceinline__ SegPos seg_pos(const ChanMap &cm, int64_t seg_len, int64_t nseg, int64_t nchunk, int group) {
    SegPos p;
    const int glog = 31 - __clz(group);
    const unsigned gi = threadIdx.x >> glog;
    p.lane = (int)(threadIdx.x & (unsigned)(group - 1));
    const unsigned gpc = (unsigned)kThreads >> glog;
    if (cm.narrow) {  // everything fits 32 bits
        const uint32_t s = blockIdx.x * gpc + gi;
        p.s = s;
        p.valid = s < (uint32_t)nseg;
        uint32_t ts = s, k = 0;
        if (nchunk > 1) {
            ts = s / (uint32_t)nchunk;
            k = s - ts * (uint32_t)nchunk;
        }
        const uint32_t I = (uint32_t)cm.I, sl = (uint32_t)seg_len;
        const uint32_t start = ts * I + k * sl;
        uint32_t len = I - k * sl;
        if (len > sl) len = sl;
        p.param = cm.C == 1 ? 0 : (!cm.wrap ? ts : ts % (uint32_t)cm.C);
        p.v0 = start / VEC;
        p.nv = (int)(len / VEC);
    } else {
        const int64_t s = (int64_t)blockIdx.x * gpc + gi;
        p.s = s;
        p.valid = s < nseg;
        int64_t ts = s, k = 0;
        if (nchunk > 1) {
            ts = s / nchunk;
            k = s - ts * nchunk;
        }
        const int64_t start = ts * cm.I + k * seg_len;
        int64_t len = cm.I - k * seg_len;
        if (len > seg_len) len = seg_len;
        p.param = cm.C == 1 ? 0 : (!cm.wrap ? ts : ts % cm.C);
        p.v0 = start / VEC;
        p.nv = (int)(len / VEC);
    }
    return p;
}


struct FwdSegArgs {
    const void *x;
    void *y;
    ParamPtr scale, offset;
    ChanMap cm;
    int64_t seg_len, nseg, nchunk;
    int group;
    double qmin, qmax, zps;
    int exact_edges;
};

// ---------------------------------------------------------------------------
// Per-thread ring of 16-byte slots in shared memory, filled by asynchronous copies
// (global -> shared without passing through registers).  Slot j of thread t lives at
// base + (j * kThreads + t) * 16, so a warp's slots are contiguous.  A thread only ever reads
// what it copied itself, so cp.async.wait_group is all the synchronisation there is.  The ring
// lets a thread keep several iterations' worth of loads in flight, and the first ones can be
// issued before the thread has even looked at its parameters.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t smem, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
template <typename E> __device__ __forceinline__ Vec16<E> ring_read(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return *reinterpret_cast<const Vec16<E> *>(&v);
}
constexpr uint32_t kSlotStride = kThreads * 16;

constexpr int kFwdU = 4;  // 16-byte vectors per forward iteration

// The vectors of a thread's first forward iteration, requested into its ring slots (one commit
// group) before the thread loads its parameters, so that the two memory latencies overlap.
template <typename E>
__device__ __forceinline__ void fwd_first_issue(uint32_t ring, const Vec16<E> *px, int lane, int nv, int G) {
#pragma unroll
    for (int u = 0; u < kFwdU; ++u)
        if (lane + u * G < nv) cp_async16(ring + u * kSlotStride, px + u * G);
    cp_async_commit();
}

template <int IO, int CT, int OP, int PATH, bool PRE>
__device__ __forceinline__ void fwd_seg_loop(uint32_t ring, const Vec16<typename Elem<IO>::type> *__restrict__ px,
                                             Vec16<typename Elem<IO>::type> *__restrict__ py, int lane, int nv, int G,
                                             const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2,
                                             bool ringed) {
    using E = typename Elem<IO>::type;
    constexpr int U = kFwdU;
    int v = lane;
    const int step = U * G;
    // first iteration: from the ring (see fwd_first_issue) when the caller requested it there
    if (ringed) cp_async_wait<0>();
    if (!ringed) {
        // nothing requested: the loops below start at the thread's first vector
    } else if (v + (U - 1) * G < nv) {
        Vec16<E> xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) xv[u] = ring_read<E>(ring + u * kSlotStride);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            Vec16<E> yv;
            fwd_vec<IO, CT, OP, PATH, PRE>(xv[u], yv, e, g, big2);
            py[u * G] = yv;
        }
    } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (v + u * G < nv) {
                Vec16<E> yv;
                fwd_vec<IO, CT, OP, PATH, PRE>(ring_read<E>(ring + u * kSlotStride), yv, e, g, big2);
                py[u * G] = yv;
            }
        }
        return;
    }
    if (ringed) {
        v += step;
        px += step;
        py += step;
    }
    for (; v + (U - 1) * G < nv; v += step, px += step, py += step) {
        Vec16<E> xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) xv[u] = px[u * G];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            Vec16<E> yv;
            fwd_vec<IO, CT, OP, PATH, PRE>(xv[u], yv, e, g, big2);
            py[u * G] = yv;
        }
    }
    if (v < nv) {  // the last, partial iteration: all its loads first, like the full ones
        Vec16<E> xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v + u * G < nv) xv[u] = px[u * G];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (v + u * G < nv) {
                Vec16<E> yv;
                fwd_vec<IO, CT, OP, PATH, PRE>(xv[u], yv, e, g, big2);
                py[u * G] = yv;
            }
        }
    }
}

// A thread whose whole share is one iteration (short runs: a block of 64 elements is eight vectors
// for two threads): its vectors were loaded into registers before its parameters, so the two memory
// latencies overlap.
template <int IO, int CT, int OP, int PATH, bool PRE>
__device__ __forceinline__ void fwd_seg_single(const Vec16<typename Elem<IO>::type> (&xv)[kFwdU],
                                               Vec16<typename Elem<IO>::type> *__restrict__ py, int lane, int nv, int G,
                                               const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2) {
    using E = typename Elem<IO>::type;
#pragma unroll
    for (int u = 0; u < kFwdU; ++u) {
        if (lane + u * G < nv) {
            Vec16<E> yv;
            fwd_vec<IO, CT, OP, PATH, PRE>(xv[u], yv, e, g, big2);
            py[u * G] = yv;
        }
    }
}

template <int IO, int CT, int OP>
__global__ void __launch_bounds__(kThreads, 5) k_fwd_seg(FwdSegArgs a) {
    pdl_launch_dependents();
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    constexpr int NV = 16 / (int)sizeof(E);
    constexpr bool kIo16 = IO == AB_BF16 || IO == AB_F16;
    constexpr bool kQuant = OP == OP_QDQ || OP == OP_Q;
    // index arithmetic needs no memory: it runs while the preceding kernel drains
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
    const SegPos p = seg_pos<NV>(a.cm, a.seg_len, a.nseg, a.nchunk, a.group);
    pdl_wait();
    if (!p.valid) return;
    const Vec16<E> *px = static_cast<const Vec16<E> *>(a.x) + p.v0 + p.lane;
    Vec16<E> *py = static_cast<Vec16<E> *>(a.y) + p.v0 + p.lane;
    __shared__ __align__(16) unsigned char ring_mem[kFwdU * kSlotStride];
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_mem) + threadIdx.x * 16u;
    // worth it when the thread has further iterations; a single-iteration thread (short runs) is
    // better off with plain loads
    const bool ringed = p.nv > kFwdU * a.group;
    Vec16<E> xv[kFwdU];
    if (ringed) {
        fwd_first_issue<E>(ring, px, p.lane, p.nv, a.group);
    } else {
#pragma unroll
        for (int u = 0; u < kFwdU; ++u)
            if (p.lane + u * a.group < p.nv) xv[u] = px[u * a.group];
    }
    const Enc<CT> e = load_enc<CT>(a.scale, a.offset, p.param, g);
#define AB_FWD_RUN(PATH, PRE, BIG)                                                                       \
    do {                                                                                                 \
        if (ringed)                                                                                      \
            fwd_seg_loop<IO, CT, OP, PATH, PRE>(ring, px, py, p.lane, p.nv, a.group, e, g, BIG, true);   \
        else                                                                                             \
            fwd_seg_single<IO, CT, OP, PATH, PRE>(xv, py, p.lane, p.nv, a.group, e, g, BIG);             \
        return;                                                                                          \
    } while (0)
    if constexpr (kQuant && kIo16) {
        uint32_t big2;
        if (abs_bound16<IO, CT>(e, big2)) {
            if constexpr (CT == IO) {
                if (vec_packed_ok<CT>(e, g)) AB_FWD_RUN(PATH_PACKED, true, big2);
            }
            if (vec_fast_ok<CT>(e, g)) AB_FWD_RUN(PATH_FAST, true, big2);
        }
    } else if constexpr (kQuant && CT != AB_F64) {
        if (vec_fast_ok<CT>(e, g)) AB_FWD_RUN(PATH_FAST, false, 0u);
    }
    AB_FWD_RUN(PATH_GENERIC, false, 0u);
#undef AB_FWD_RUN
}

struct FwdGenArgs {
    const void *x;
    void *y;
    ParamPtr scale, offset;
    int64_t numel;
    GenMap gm;
    double qmin, qmax, zps;
    int exact_edges;
};

template <int IO, int CT, int OP>
__global__ void __launch_bounds__(kThreads) k_fwd_gen(FwdGenArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    E *__restrict__ yp = static_cast<E *>(a.y);
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < a.numel; i += stride) {
        Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.gm.of(i), g);
        yp[i] = C::store(fwd_elem<CT, OP>(C::load(xp[i]), e, g));
    }
}

// ---------------------------------------------------------------------------
// backward kernels
// ---------------------------------------------------------------------------
struct BwdArgs {
    const void *x, *gy;
    void *gx;  // may be NULL
    ParamPtr scale, offset;
    ParamOut gs, go;    // direct outputs (may hold NULL pointers)
    double *partial;    // [npartial][2]
    int64_t numel;
    ChanMap cm;
    // segment mode
    int64_t seg_len;    // elements per pseudo-segment (a multiple of the vector width)
    int64_t nseg;       // number of pseudo-segments
    int64_t nchunk;     // pseudo-segments per true segment
    int group;          // threads per pseudo-segment, power of two <= kThreads
    int direct;         // write gs / go straight from the kernel (O == 1, nchunk == 1)
    // column mode
    int64_t rows, row_len, rows_per_tile;
    double qmin, qmax, zps;
    int exact_edges;
    double pgs_thr, pgs_mult;  // pgs_mult == 1: off
};

// the launch's grid of the backward kernels, with the rounding-error threshold in the internal dtype
template <int CT, typename Args> __device__ __forceinline__ Grid<typename Arith<CT>::T> bwd_grid(const Args &a) {
    using T = typename Arith<CT>::T;
    Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
    if (a.pgs_mult != 1.0) {
        g.has_pgs = 1;
        g.pgs_thr = Arith<CT>::rnd((T)a.pgs_thr);
        g.pgs_mult = (T)a.pgs_mult;
    }
    return g;
}

template <int CT> __device__ __forceinline__ double finalize(double v) {
    using A = Arith<CT>;
    using T = typename A::T;
    return (double)A::rnd((T)v);
}

constexpr int kBwdDepth = 3;                               // iterations in flight, backward
constexpr int kBwdSlots = 4;                               // x, gy of two vectors per iteration
constexpr size_t kBwdRingBytes = (size_t)kBwdDepth * kBwdSlots * kSlotStride;

// Requests the vectors of backward iteration k (vectors v and v + G of x and of the upstream
// gradient, v = lane + 2 G k) into the slots of ring position `pos`.
template <typename E>
__device__ __forceinline__ void bwd_ring_issue(uint32_t ring, int pos, const Vec16<E> *px, const Vec16<E> *pg, int v,
                                               int nv, int G) {
    const uint32_t s0 = ring + (uint32_t)(pos * kBwdSlots) * kSlotStride;
    if (v < nv) {
        cp_async16(s0, px);
        cp_async16(s0 + kSlotStride, pg);
        if (v + G < nv) {
            cp_async16(s0 + 2 * kSlotStride, px + G);
            cp_async16(s0 + 3 * kSlotStride, pg + G);
        }
    }
}

// The first kBwdDepth iterations were requested by the caller (before it loaded its parameters).
template <int IO, int CT, int OP, bool WANT_O, int PATH, bool PRE>
__device__ __forceinline__ void bwd_seg_loop(uint32_t ring, const Vec16<typename Elem<IO>::type> *__restrict__ px,
                                             const Vec16<typename Elem<IO>::type> *__restrict__ pg,
                                             Vec16<typename Elem<IO>::type> *__restrict__ pd, int lane, int nv, int G,
                                             const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2,
                                             typename Arith<CT>::T &acc_s, typename Arith<CT>::T &acc_o) {
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    // the generic body also serves callers that want no input gradient; the others always store
    constexpr bool kMayskip = PATH == PATH_GENERIC;
    T acc_s2 = 0;
    const int step = 2 * G;
    int pos = 0;
    for (int v = lane; v < nv; v += step) {
        cp_async_wait<kBwdDepth - 1>();
        const uint32_t s0 = ring + (uint32_t)(pos * kBwdSlots) * kSlotStride;
        const bool two = v + G < nv;
        const Vec16<E> xa = ring_read<E>(s0), ga = ring_read<E>(s0 + kSlotStride);
        Vec16<E> xb, gb;
        if (two) {
            xb = ring_read<E>(s0 + 2 * kSlotStride);
            gb = ring_read<E>(s0 + 3 * kSlotStride);
        }
        // refill this ring position with the iteration kBwdDepth ahead
        bwd_ring_issue<E>(ring, pos, px + kBwdDepth * step, pg + kBwdDepth * step, v + kBwdDepth * step, nv, G);
        cp_async_commit();
        Vec16<E> da, db;
        bwd_vec<IO, CT, OP, WANT_O, PATH, PRE>(xa, ga, da, e, g, big2, acc_s, acc_s2, acc_o);
        if (!kMayskip || pd) pd[0] = da;
        if (two) {
            bwd_vec<IO, CT, OP, WANT_O, PATH, PRE>(xb, gb, db, e, g, big2, acc_s, acc_s2, acc_o);
            if (!kMayskip || pd) pd[G] = db;
        }
        if (!kMayskip || pd) pd += step;
        px += step;
        pg += step;
        pos = pos + 1 == kBwdDepth ? 0 : pos + 1;
    }
    acc_s += acc_s2;
}

// One group of `group` threads per pseudo-segment; a pseudo-segment is a
// contiguous run of elements that share one parameter.
template <int IO, int CT, int OP, bool VECT, bool WANT_O>
__global__ void __launch_bounds__(kThreads, 4) k_bwd_seg(BwdArgs a) {
    pdl_launch_dependents();
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    constexpr bool kIo16 = IO == AB_BF16 || IO == AB_F16;
    const Grid<T> g = bwd_grid<CT>(a);

    const int G = a.group;
    // index arithmetic needs no memory: it runs while the preceding kernel drains
    const SegPos p = seg_pos<VEC>(a.cm, a.seg_len, a.nseg, a.nchunk, G);
    pdl_wait();
    const int lane = p.lane;
    const bool valid = p.valid;
    const int64_t s = p.s, param = p.param;

    T acc_s = 0, acc_o = 0;
    if (valid) {
        [[maybe_unused]] uint32_t ring = 0;
        if constexpr (VECT) {
            // the first iterations' vectors are requested before the parameters are even loaded
            extern __shared__ __align__(16) unsigned char ring_mem[];
            ring = (uint32_t)__cvta_generic_to_shared(ring_mem) + threadIdx.x * 16u;
            const Vec16<E> *px = static_cast<const Vec16<E> *>(a.x) + p.v0 + lane;
            const Vec16<E> *pg = static_cast<const Vec16<E> *>(a.gy) + p.v0 + lane;
#pragma unroll
            for (int k = 0; k < kBwdDepth; ++k) {
                bwd_ring_issue<E>(ring, k, px + k * 2 * G, pg + k * 2 * G, lane + k * 2 * G, p.nv, G);
                cp_async_commit();
            }
        }
        const Enc<CT> e = load_enc<CT>(a.scale, a.offset, param, g);
        if constexpr (VECT) {
            const Vec16<E> *px = static_cast<const Vec16<E> *>(a.x) + p.v0 + lane;
            const Vec16<E> *pg = static_cast<const Vec16<E> *>(a.gy) + p.v0 + lane;
            Vec16<E> *pd = a.gx ? static_cast<Vec16<E> *>(a.gx) + p.v0 + lane : nullptr;
            // the specialised bodies always write the input gradient; a caller that wants none
            // takes the generic one
            bool done = false;
            if constexpr (OP == OP_QDQ && kIo16) {
                uint32_t big2;
                if (pd && abs_bound16<IO, CT>(e, big2)) {
                    if constexpr (CT == IO) {
                        if (vec_packed_ok<CT>(e, g)) {
                            bwd_seg_loop<IO, CT, OP, WANT_O, PATH_PACKED, true>(ring, px, pg, pd, lane, p.nv, G, e, g, big2, acc_s, acc_o);
                            done = true;
                        }
                    }
                    if (!done && vec_fast_ok<CT>(e, g)) {
                        bwd_seg_loop<IO, CT, OP, WANT_O, PATH_FAST, true>(ring, px, pg, pd, lane, p.nv, G, e, g, big2, acc_s, acc_o);
                        done = true;
                    }
                }
            } else if constexpr (OP == OP_QDQ && CT != AB_F64) {
                if (pd && vec_fast_ok<CT>(e, g)) {
                    bwd_seg_loop<IO, CT, OP, WANT_O, PATH_FAST, false>(ring, px, pg, pd, lane, p.nv, G, e, g, 0u, acc_s, acc_o);
                    done = true;
                }
            }
            if (!done) bwd_seg_loop<IO, CT, OP, WANT_O, PATH_GENERIC, false>(ring, px, pg, pd, lane, p.nv, G, e, g, 0u, acc_s, acc_o);
        } else {
            const E *__restrict__ xp = static_cast<const E *>(a.x) + p.v0;
            const E *__restrict__ gp = static_cast<const E *>(a.gy) + p.v0;
            E *__restrict__ dxp = a.gx ? static_cast<E *>(a.gx) + p.v0 : nullptr;
            for (int v = lane; v < p.nv; v += G) {
                T ds, dofs;
                const T dx = bwd_elem<CT, OP, WANT_O>(C::load(xp[v]), C::load(gp[v]), e, g, ds, dofs);
                acc_s += ds;
                acc_o += dofs;
                if (dxp) dxp[v] = C::store(dx);
            }
        }
    }

    // fixed-order reduction over the group, in the register type (the partials are summed in
    // float64 by the finishing kernel)
    T rs = acc_s, ro = acc_o;
    const int span = G < 32 ? G : 32;
    for (int o = span >> 1; o > 0; o >>= 1) {
        rs += __shfl_xor_sync(0xffffffffu, rs, o);
        if (WANT_O) ro += __shfl_xor_sync(0xffffffffu, ro, o);
    }
    if (G > 32) {
        __shared__ T sh[2][kThreads / 32];
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) {
            sh[0][warp] = rs;
            sh[1][warp] = ro;
        }
        __syncthreads();
        if (lane == 0) {
            const int w0 = (threadIdx.x / G) * (G / 32);
            rs = 0;
            ro = 0;
            for (int w = 0; w < G / 32; ++w) {
                rs += sh[0][w0 + w];
                ro += sh[1][w0 + w];
            }
        }
    }
    if (valid && lane == 0) {
        if (a.direct) {
            if (a.gs.p) a.gs.put(param, finalize<CT>((double)rs));
            if (a.go.p) a.go.put(param, finalize<CT>((double)ro));
        } else {
            a.partial[2 * s] = (double)rs;
            a.partial[2 * s + 1] = (double)ro;
        }
    }
}

// Column mode for small inner extents under a large outer dim: the tensor is a
// (rows, row_len) matrix whose columns each belong to one parameter; a thread
// owns one 16-byte column group and walks down a tile of rows.
template <int IO, int CT, int OP, bool VECT, bool WANT_O>
__global__ void __launch_bounds__(kThreads) k_bwd_col(BwdArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g = bwd_grid<CT>(a);
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    const E *__restrict__ gp = static_cast<const E *>(a.gy);
    E *__restrict__ dxp = static_cast<E *>(a.gx);

    const int64_t cv = (int64_t)blockIdx.x * kThreads + threadIdx.x;  // column group
    const int64_t ncv = a.row_len / VEC;
    if (cv >= ncv) return;
    const int64_t r0 = (int64_t)blockIdx.y * a.rows_per_tile;
    int64_t r1 = r0 + a.rows_per_tile;
    if (r1 > a.rows) r1 = a.rows;

    Enc<CT> e[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        int64_t col = cv * VEC + i;
        int64_t p = a.cm.C == 1 ? 0 : (a.cm.shift >= 0 ? (col >> a.cm.shift) : col / a.cm.I);
        e[i] = load_enc<CT>(a.scale, a.offset, p, g);
    }
    T acc_s[VEC], acc_o[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc_s[i] = acc_o[i] = 0;

    for (int64_t r = r0; r < r1; r += 2) {
        const int64_t ia = r * ncv + cv, ib = ia + ncv;
        const bool hb = r + 1 < r1;
        Vec16<E> xa, ga, xb, gb, da, db;
        if (VECT) {
            xa = reinterpret_cast<const Vec16<E> *>(xp)[ia];
            ga = reinterpret_cast<const Vec16<E> *>(gp)[ia];
            if (hb) {
                xb = reinterpret_cast<const Vec16<E> *>(xp)[ib];
                gb = reinterpret_cast<const Vec16<E> *>(gp)[ib];
            }
        } else {
            xa.v[0] = xp[ia];
            ga.v[0] = gp[ia];
            if (hb) {
                xb.v[0] = xp[ib];
                gb.v[0] = gp[ib];
            }
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            T ds, dofs;
            da.v[i] = C::store(bwd_elem<CT, OP, WANT_O>(C::load(xa.v[i]), C::load(ga.v[i]), e[i], g, ds, dofs));
            acc_s[i] += ds;
            acc_o[i] += dofs;
        }
        if (hb) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                T ds, dofs;
                db.v[i] = C::store(bwd_elem<CT, OP, WANT_O>(C::load(xb.v[i]), C::load(gb.v[i]), e[i], g, ds, dofs));
                acc_s[i] += ds;
                acc_o[i] += dofs;
            }
        }
        if (dxp) {
            if (VECT) {
                reinterpret_cast<Vec16<E> *>(dxp)[ia] = da;
                if (hb) reinterpret_cast<Vec16<E> *>(dxp)[ib] = db;
            } else {
                dxp[ia] = da.v[0];
                if (hb) dxp[ib] = db.v[0];
            }
        }
    }
    if (!a.partial) return;
    double *out = a.partial + 2 * ((int64_t)blockIdx.y * a.row_len + cv * VEC);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        out[2 * i] = (double)acc_s[i];
        out[2 * i + 1] = (double)acc_o[i];
    }
}

// grad[c] = sum_{a<na} sum_{b<nb} partial[a*sa + c*sc + b]; one warp per c,
// lanes stride over the (a, b) pairs in a fixed order.
struct FinishArgs {
    const double *partial;
    ParamOut gs, go;
    int64_t nparam, na, sa, sc, nb;
};

template <int CT, bool PER_CTA> __global__ void __launch_bounds__(kThreads) k_bwd_finish(FinishArgs a) {
    pdl_prologue();
    // PER_CTA: one CTA per parameter (many partials each); else one warp per parameter
    const int64_t c = PER_CTA ? (int64_t)blockIdx.x : (((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (c >= a.nparam) return;
    double rs = 0, ro = 0;
    const int64_t n = a.na * a.nb;
    const int step = PER_CTA ? kThreads : 32;
    for (int64_t t = PER_CTA ? threadIdx.x : lane; t < n; t += step) {
        const int64_t ia = t / a.nb, ib = t - ia * a.nb;
        const double *p = a.partial + 2 * (ia * a.sa + c * a.sc + ib);
        rs += p[0];
        ro += p[1];
    }
    rs = warp_sum(rs);
    ro = warp_sum(ro);
    if (PER_CTA) {
        __shared__ double sh[2][kThreads / 32];
        if (lane == 0) {
            sh[0][threadIdx.x >> 5] = rs;
            sh[1][threadIdx.x >> 5] = ro;
        }
        __syncthreads();
        if (threadIdx.x != 0) return;
        rs = ro = 0;
        for (int w = 0; w < kThreads / 32; ++w) {
            rs += sh[0][w];
            ro += sh[1][w];
        }
    }
    if (lane == 0) {
        if (a.gs.p) a.gs.put(c, finalize<CT>(rs));
        if (a.go.p) a.go.put(c, finalize<CT>(ro));
    }
}

// General layouts (e.g. blocks along two dims): one warp per parameter walks
// the box of elements that share it.
struct BwdGenArgs {
    const void *x, *gy;
    void *gx;
    ParamPtr scale, offset;
    ParamOut gs, go;
    int64_t nparam;
    int nd;
    int64_t nblk[AB_MAX_DIMS];     // parameters along dim k
    int64_t block[AB_MAX_DIMS];
    int64_t estride[AB_MAX_DIMS];  // element stride of dim k
    int64_t box;                   // elements per parameter
    double qmin, qmax, zps;
    int exact_edges;
    double pgs_thr, pgs_mult;
};

template <int IO, int CT, int OP, bool WANT_O>
__global__ void __launch_bounds__(kThreads) k_bwd_gen(BwdGenArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    const Grid<T> g = bwd_grid<CT>(a);
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    const E *__restrict__ gp = static_cast<const E *>(a.gy);
    E *__restrict__ dxp = static_cast<E *>(a.gx);
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
    for (int64_t p = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5; p < a.nparam; p += nwarps) {
        int64_t base = 0, rem = p;
        for (int k = a.nd - 1; k >= 0; --k) {
            int64_t pc = rem % a.nblk[k];
            rem /= a.nblk[k];
            base += pc * a.block[k] * a.estride[k];
        }
        const Enc<CT> e = load_enc<CT>(a.scale, a.offset, p, g);
        T acc_s = 0, acc_o = 0;
        for (int64_t t = lane; t < a.box; t += 32) {
            int64_t off = base, r = t;
            for (int k = a.nd - 1; k >= 0; --k) {
                int64_t c = r % a.block[k];
                r /= a.block[k];
                off += c * a.estride[k];
            }
            T ds, dofs;
            T dx = bwd_elem<CT, OP, WANT_O>(C::load(xp[off]), C::load(gp[off]), e, g, ds, dofs);
            acc_s += ds;
            acc_o += dofs;
            if (dxp) dxp[off] = C::store(dx);
        }
        double rs = warp_sum((double)acc_s), ro = warp_sum((double)acc_o);
        if (lane == 0) {
            if (a.gs.p) a.gs.put(p, finalize<CT>(rs));
            if (a.go.p) a.go.put(p, finalize<CT>(ro));
        }
    }
}

// ---------------------------------------------------------------------------
// host-side planning and dispatch
// ---------------------------------------------------------------------------
using BwdPlan = ReducePlan;
// long runs are cut into chunks of 32 vectors per thread
inline BwdPlan plan_backward(const Canon &c, int io_dtype, bool ptr_aligned) { return plan_reduce(c, io_dtype, ptr_aligned, 4, 4); }

// qmin-1 and qmax+1 are exactly representable in the 16-bit internal dtype
bool fits_significand(int64_t v, int bits) {
    if (v < 0) v = -v;
    if (v == 0) return true;
    while ((v & 1) == 0) v >>= 1;
    return v < ((int64_t)1 << bits);
}
int exact_edges(int ct, int64_t qmin, int64_t qmax) {
    const int bits = ct == AB_BF16 ? 8 : (ct == AB_F16 ? 11 : 0);
    if (bits == 0) return 0;
    if (qmax > 60000 || qmin < -60000) return 0;
    return fits_significand(qmin - 1, bits) && fits_significand(qmax + 1, bits);
}

struct Call {
    int op;
    const void *x, *gy, *scale, *offset;
    void *y;  // forward output
    void *gx, *gs, *go;
    const ab_layout *layout;
    int io, ct, pt;
    int64_t qmin, qmax;
    double zps;
    void *scratch;
    int64_t scratch_bytes;
    cudaStream_t stream;
    double pgs_thr = 0.0, pgs_mult = 1.0;  // backward of quantize-dequantize only
};

int check_common(const Call &c, Canon *canon) {
    int rc = canonicalize(c.layout, canon);
    if (rc != AB_OK) return rc;
    if (c.pt != AB_F32 && c.pt != AB_F64) return fail(AB_ERR_INVALID, "param_dtype must be AB_F32 or AB_F64");
    if (c.op != OP_DQ && c.qmin > c.qmax)
        return fail(AB_ERR_INVALID, "qmin (%lld) must be smaller than or equal to qmax (%lld)",
                    (long long)c.qmin, (long long)c.qmax);
    if (canon->numel > 0 && (!c.x || !c.scale || !c.offset))
        return fail(AB_ERR_INVALID, "x, scale and offset must not be NULL");
    return AB_OK;
}

template <int IO, int CT, int OP> int launch_forward(const Call &c, const Canon &canon) {
    if (canon.numel == 0) return AB_OK;
    const int vecw = 16 / dtype_size(IO);
    if (canon.oci) {
        FwdArgs a;
        a.x = c.x;
        a.y = c.y;
        a.scale = ParamPtr{c.scale, c.pt == AB_F64};
        a.offset = ParamPtr{c.offset, c.pt == AB_F64};
        a.numel = canon.numel;
        a.cm = make_chan_map(canon);
        a.qmin = (double)c.qmin;
        a.qmax = (double)c.qmax;
        a.zps = c.zps;
        a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
        const bool vect = aligned16(c.x) && aligned16(c.y) && (canon.numel % vecw == 0);
        const ReducePlan sp = plan_reduce(canon, IO, vect);
        if (vect && vecw >= 2 && sp.mode == ReducePlan::SEG && sp.vect) {
            FwdSegArgs f;
            f.x = c.x;
            f.y = c.y;
            f.scale = a.scale;
            f.offset = a.offset;
            f.cm = a.cm;
            f.seg_len = sp.seg_len;
            f.nseg = sp.nseg;
            f.nchunk = sp.nchunk;
            f.group = sp.group;
            f.qmin = a.qmin;
            f.qmax = a.qmax;
            f.zps = a.zps;
            f.exact_edges = a.exact_edges;
            const int gpc = kThreads / sp.group;
            const int64_t sgrid = (sp.nseg + gpc - 1) / gpc;
            if (sgrid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
            launch_pdl(k_fwd_seg<IO, CT, OP>, (unsigned)sgrid, kThreads, 0, c.stream, f);
            AB_LAUNCH_OK();
            return AB_OK;
        }
        const int64_t nvec = vect ? canon.numel / vecw : canon.numel;
        const int64_t per_cta = (int64_t)kThreads * kFwdUnroll;
        const int64_t grid = (nvec + per_cta - 1) / per_cta;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (vect)
            launch_pdl(k_fwd_oci<IO, CT, OP, true>, (unsigned)grid, kThreads, 0, c.stream, a);
        else
            launch_pdl(k_fwd_oci<IO, CT, OP, false>, (unsigned)grid, kThreads, 0, c.stream, a);
    } else {
        FwdGenArgs a;
        a.x = c.x;
        a.y = c.y;
        a.scale = ParamPtr{c.scale, c.pt == AB_F64};
        a.offset = ParamPtr{c.offset, c.pt == AB_F64};
        a.numel = canon.numel;
        a.gm = make_gen_map(canon);
        a.qmin = (double)c.qmin;
        a.qmax = (double)c.qmax;
        a.zps = c.zps;
        a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
        int64_t grid = (canon.numel + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (grid > cap) grid = cap;
        launch_pdl(k_fwd_gen<IO, CT, OP>, (unsigned)grid, kThreads, 0, c.stream, a);
    }
    AB_LAUNCH_OK();
    return AB_OK;
}

template <int IO, int CT, int OP> int launch_backward(const Call &c, const Canon &canon) {
    if (canon.numel == 0) return AB_OK;
    const bool al = aligned16(c.x) && aligned16(c.gy) && (!c.gx || aligned16(c.gx));
    const ParamOut gs{c.gs, c.pt == AB_F64}, go{c.go, c.pt == AB_F64};
    const BwdPlan p = plan_backward(canon, IO, al);
    if (p.mode == BwdPlan::GEN) {
        BwdGenArgs a;
        a.x = c.x;
        a.gy = c.gy;
        a.gx = c.gx;
        a.scale = ParamPtr{c.scale, c.pt == AB_F64};
        a.offset = ParamPtr{c.offset, c.pt == AB_F64};
        a.gs = gs;
        a.go = go;
        a.nparam = canon.nparam;
        a.nd = canon.nd;
        int64_t es = 1, box = 1;
        for (int k = AB_MAX_DIMS - 1; k >= 0; --k) {
            if (k < canon.nd) {
                a.nblk[k] = canon.size[k] / canon.block[k];
                a.block[k] = canon.block[k];
                a.estride[k] = es;
                es *= canon.size[k];
                box *= canon.block[k];
            } else {
                a.nblk[k] = 1;
                a.block[k] = 1;
                a.estride[k] = 0;
            }
        }
        a.box = box;
        a.qmin = (double)c.qmin;
        a.qmax = (double)c.qmax;
        a.zps = c.zps;
        a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
        a.pgs_thr = c.pgs_thr;
        a.pgs_mult = c.pgs_mult;
        int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (grid > cap) grid = cap;
        if (c.go)
            launch_pdl(k_bwd_gen<IO, CT, OP, true>, (unsigned)grid, kThreads, 0, c.stream, a);
        else
            launch_pdl(k_bwd_gen<IO, CT, OP, false>, (unsigned)grid, kThreads, 0, c.stream, a);
        AB_LAUNCH_OK();
        return AB_OK;
    }

    const bool want_param_grads = c.gs || c.go;
    const int64_t need = want_param_grads ? p.npartial * 2 * (int64_t)sizeof(double) : 0;
    if (need > 0 && (!c.scratch || c.scratch_bytes < need))
        return fail(AB_ERR_SCRATCH, "backward needs %lld bytes of scratch, got %lld", (long long)need,
                    (long long)c.scratch_bytes);
    if (need > 0 && !aligned16(c.scratch)) return fail(AB_ERR_INVALID, "scratch must be 16-byte aligned");

    BwdArgs a;
    a.x = c.x;
    a.gy = c.gy;
    a.gx = c.gx;
    a.scale = ParamPtr{c.scale, c.pt == AB_F64};
    a.offset = ParamPtr{c.offset, c.pt == AB_F64};
    a.gs = gs;
    a.go = go;
    a.partial = need > 0 ? static_cast<double *>(c.scratch) : nullptr;
    a.numel = canon.numel;
    a.cm = make_chan_map(canon);
    a.seg_len = p.seg_len;
    a.nseg = p.nseg;
    a.nchunk = p.nchunk;
    a.group = p.group;
    a.direct = (p.direct || !want_param_grads) ? 1 : 0;
    a.rows = canon.O;
    a.row_len = canon.C * canon.I;
    a.rows_per_tile = p.rows_per_tile;
    a.qmin = (double)c.qmin;
    a.qmax = (double)c.qmax;
    a.zps = c.zps;
    a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
    a.pgs_thr = c.pgs_thr;
    a.pgs_mult = c.pgs_mult;

    if (p.mode == BwdPlan::SEG) {
        const int gpc = kThreads / p.group;
        const int64_t grid = (p.nseg + gpc - 1) / gpc;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (p.vect && c.go)
            {
                int rc = opt_in_smem<k_bwd_seg<IO, CT, OP, true, true>>(kBwdRingBytes);
                if (rc != AB_OK) return rc;
                launch_pdl(k_bwd_seg<IO, CT, OP, true, true>, (unsigned)grid, kThreads, kBwdRingBytes, c.stream, a);
            }
        else if (p.vect)
            {
                int rc = opt_in_smem<k_bwd_seg<IO, CT, OP, true, false>>(kBwdRingBytes);
                if (rc != AB_OK) return rc;
                launch_pdl(k_bwd_seg<IO, CT, OP, true, false>, (unsigned)grid, kThreads, kBwdRingBytes, c.stream, a);
            }
        else if (c.go)
            launch_pdl(k_bwd_seg<IO, CT, OP, false, true>, (unsigned)grid, kThreads, 0, c.stream, a);
        else
            launch_pdl(k_bwd_seg<IO, CT, OP, false, false>, (unsigned)grid, kThreads, 0, c.stream, a);
    } else {
        const int v = p.vect ? 16 / dtype_size(IO) : 1;
        const int64_t gx = (a.row_len / v + kThreads - 1) / kThreads;
        if (gx > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        dim3 grid((unsigned)gx, (unsigned)p.row_tiles);
        if (p.vect && c.go)
            launch_pdl(k_bwd_col<IO, CT, OP, true, true>, grid, kThreads, 0, c.stream, a);
        else if (p.vect)
            launch_pdl(k_bwd_col<IO, CT, OP, true, false>, grid, kThreads, 0, c.stream, a);
        else if (c.go)
            launch_pdl(k_bwd_col<IO, CT, OP, false, true>, grid, kThreads, 0, c.stream, a);
        else
            launch_pdl(k_bwd_col<IO, CT, OP, false, false>, grid, kThreads, 0, c.stream, a);
    }
    AB_LAUNCH_OK();
    if (need > 0) {
        FinishArgs f;
        f.partial = a.partial;
        f.gs = gs;
        f.go = go;
        f.nparam = canon.nparam;
        f.na = p.na;
        f.sa = p.sa;
        f.sc = p.sc;
        f.nb = p.nb;
        if (p.na * p.nb > 256) {
            launch_pdl(k_bwd_finish<CT, true>, (unsigned)canon.nparam, kThreads, 0, c.stream, f);
        } else {
            const int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
            launch_pdl(k_bwd_finish<CT, false>, (unsigned)grid, kThreads, 0, c.stream, f);
        }
        AB_LAUNCH_OK();
    }
    return AB_OK;
}

template <int IO, int CT> int dispatch_op(const Call &c, const Canon &canon, bool backward) {
    switch (c.op) {
        case OP_Q: return backward ? launch_backward<IO, CT, OP_Q>(c, canon) : launch_forward<IO, CT, OP_Q>(c, canon);
        case OP_DQ: return backward ? launch_backward<IO, CT, OP_DQ>(c, canon) : launch_forward<IO, CT, OP_DQ>(c, canon);
        case OP_QDQ: return backward ? launch_backward<IO, CT, OP_QDQ>(c, canon) : launch_forward<IO, CT, OP_QDQ>(c, canon);
        case OP_FQ:
            if constexpr (CT == AB_F32 && IO != AB_F64) {
                if (backward && (c.gs || c.go))
                    return fail(AB_ERR_INVALID, "fake_quantize has no scale / offset gradient");
                return backward ? launch_backward<IO, CT, OP_FQ>(c, canon) : launch_forward<IO, CT, OP_FQ>(c, canon);
            } else {
                return fail(AB_ERR_UNSUPPORTED, "fake_quantize arithmetic is float32 on float32 / float16 / bfloat16 tensors");
            }
    }
    return fail(AB_ERR_INVALID, "unknown op %d", c.op);
}

int dispatch(const Call &c, bool backward) {
    Canon canon;
    int rc = check_common(c, &canon);
    if (rc != AB_OK) return rc;
    if (canon.numel > 0) {
        if (!backward && !c.y) return fail(AB_ERR_INVALID, "output pointer is NULL");
        if (backward && !c.gy) return fail(AB_ERR_INVALID, "grad_y is NULL");
    }
#define AB_COMBO(IO_, CT_) \
    if (c.io == IO_ && c.ct == CT_) return dispatch_op<IO_, CT_>(c, canon, backward);
    AB_COMBO(AB_F32, AB_F32)
    AB_COMBO(AB_F32, AB_F64)
    AB_COMBO(AB_BF16, AB_BF16)
    AB_COMBO(AB_BF16, AB_F32)
    AB_COMBO(AB_F16, AB_F16)
    AB_COMBO(AB_F16, AB_F32)
    AB_COMBO(AB_F64, AB_F64)
#undef AB_COMBO
    return fail(AB_ERR_UNSUPPORTED, "unsupported (io_dtype=%d, compute_dtype=%d) combination", c.io, c.ct);
}

}  // namespace
}  // namespace ab

using ab::Call;

extern "C" int aimet_b200_quantize(const void *x, void *y, const void *scale, const void *offset,
                                   const ab_layout *layout, int io_dtype, int compute_dtype,
                                   int param_dtype, int64_t qmin, int64_t qmax, void *stream) {
    Call c{};
    c.op = ab::OP_Q;
    c.x = x; c.y = y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = 0.0;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, false);
}

extern "C" int aimet_b200_dequantize(const void *x, void *y, const void *scale, const void *offset,
                                     const ab_layout *layout, int io_dtype, int compute_dtype,
                                     int param_dtype, void *stream) {
    Call c{};
    c.op = ab::OP_DQ;
    c.x = x; c.y = y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, false);
}

extern "C" int aimet_b200_quantize_dequantize(const void *x, void *y, const void *scale,
                                              const void *offset, const ab_layout *layout,
                                              int io_dtype, int compute_dtype, int param_dtype,
                                              int64_t qmin, int64_t qmax, double zero_point_shift,
                                              void *stream) {
    Call c{};
    c.op = ab::OP_QDQ;
    c.x = x; c.y = y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = zero_point_shift;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, false);
}

extern "C" int64_t aimet_b200_backward_scratch_bytes(const ab_layout *layout, int io_dtype) {
    ab::Canon canon;
    int rc = ab::canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (ab::dtype_size(io_dtype) == 0) return ab::fail(AB_ERR_INVALID, "unknown io_dtype %d", io_dtype);
    if (canon.numel == 0) return 0;
    // the aligned plan is an upper bound for the scalar one except for the
    // segment mode, where shorter chunks mean more partials: take the maximum
    const ab::BwdPlan pa = ab::plan_backward(canon, io_dtype, true);
    const ab::BwdPlan pb = ab::plan_backward(canon, io_dtype, false);
    const int64_t n = pa.npartial > pb.npartial ? pa.npartial : pb.npartial;
    return n * 2 * (int64_t)sizeof(double);
}

extern "C" int aimet_b200_quantize_dequantize_backward(
    const void *x, const void *grad_y, const void *scale, const void *offset, const ab_layout *layout,
    int io_dtype, int compute_dtype, int param_dtype, int64_t qmin, int64_t qmax,
    double zero_point_shift, void *grad_x, void *grad_scale, void *grad_offset, void *scratch,
    int64_t scratch_bytes, void *stream) {
    Call c{};
    c.op = ab::OP_QDQ;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = zero_point_shift;
    c.gx = grad_x; c.gs = grad_scale; c.go = grad_offset;
    c.scratch = scratch; c.scratch_bytes = scratch_bytes;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, true);
}

extern "C" int aimet_b200_quantize_dequantize_backward_ex(
    const void *x, const void *grad_y, const void *scale, const void *offset, const ab_layout *layout,
    int io_dtype, int compute_dtype, int param_dtype, int64_t qmin, int64_t qmax,
    double zero_point_shift, double pgs_eps, double pgs_multiplier, void *grad_x, void *grad_scale,
    void *grad_offset, void *scratch, int64_t scratch_bytes, void *stream) {
    if (!(pgs_eps >= 0.0 && pgs_eps <= 1.0))
        return ab::fail(AB_ERR_INVALID, "pgs_eps must be in [0, 1], got %g", pgs_eps);
    Call c{};
    c.op = ab::OP_QDQ;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = zero_point_shift;
    c.gx = grad_x; c.gs = grad_scale; c.go = grad_offset;
    c.scratch = scratch; c.scratch_bytes = scratch_bytes;
    c.stream = static_cast<cudaStream_t>(stream);
    if (pgs_eps > 0.0 && pgs_multiplier != 1.0 && grad_x) {
        c.pgs_thr = (1.0 - pgs_eps) / 2.0;
        c.pgs_mult = pgs_multiplier;
    }
    return ab::dispatch(c, true);
}

extern "C" int aimet_b200_quantize_backward(const void *x, const void *grad_y, const void *scale,
                                            const void *offset, const ab_layout *layout,
                                            int io_dtype, int compute_dtype, int param_dtype,
                                            int64_t qmin, int64_t qmax, void *grad_x,
                                            void *grad_scale, void *grad_offset, void *scratch,
                                            int64_t scratch_bytes, void *stream) {
    Call c{};
    c.op = ab::OP_Q;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = 0.0;
    c.gx = grad_x; c.gs = grad_scale; c.go = grad_offset;
    c.scratch = scratch; c.scratch_bytes = scratch_bytes;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, true);
}

extern "C" int aimet_b200_dequantize_backward(const void *x, const void *grad_y, const void *scale,
                                              const void *offset, const ab_layout *layout,
                                              int io_dtype, int compute_dtype, int param_dtype,
                                              void *grad_x, void *grad_scale, void *grad_offset,
                                              void *scratch, int64_t scratch_bytes, void *stream) {
    Call c{};
    c.op = ab::OP_DQ;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.gx = grad_x; c.gs = grad_scale; c.go = grad_offset;
    c.scratch = scratch; c.scratch_bytes = scratch_bytes;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, true);
}

extern "C" int aimet_b200_fake_quantize(const void *x, void *y, const void *scale, const void *offset,
                                        const ab_layout *layout, int io_dtype, int64_t qmin, int64_t qmax,
                                        void *stream) {
    Call c{};
    c.op = ab::OP_FQ;
    c.x = x; c.y = y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = AB_F32; c.pt = AB_F32;
    c.qmin = qmin; c.qmax = qmax; c.zps = 0.0;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, false);
}

extern "C" int aimet_b200_fake_quantize_backward(const void *x, const void *grad_y, const void *scale,
                                                 const void *offset, const ab_layout *layout, int io_dtype,
                                                 int64_t qmin, int64_t qmax, void *grad_x, void *stream) {
    Call c{};
    c.op = ab::OP_FQ;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = AB_F32; c.pt = AB_F32;
    c.qmin = qmin; c.qmax = qmax; c.zps = 0.0;
    c.gx = grad_x;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, true);
}

// ---------------------------------------------------------------------------
// Quantize-dequantize backward for hosts that may not allocate device memory.
//
// The partial sums of the scale / offset gradients normally live in a scratch
// buffer the caller allocates.  A caller that runs inside someone else's memory
// budget -- an operator plugged into a serving runtime whose execute hook must
// not touch the allocator, a worker that has handed all of its memory to a
// pool it does not own -- cannot provide one.  For them the partial sums go to
// the fixed array below, which every GPU that loads this library holds until
// the process exits.
//
// The array is shared by all calls on a device and keeps whatever the last call
// left in it.  Nothing in it has to start at zero: every slot the finishing
// kernel reads was written by the pass before it in the same call.  Two calls
// whose kernels overlap on the GPU (different streams) would write the same
// slots and race; issue them on one stream or order them yourself.
// ---------------------------------------------------------------------------
namespace ab {
namespace {

constexpr int64_t kFixedScratchBytes = 1 << 20;  // 65536 partial (scale, offset) pairs
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

// Device address of g_fixed_scratch for the current device.  In host code the array's name is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress, looked up once per
// device with that device current.
int fixed_scratch_ptr(void **out) {
    static void *ptrs[64] = {};
    static std::mutex lock;
    int dev = 0;
    AB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(AB_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> guard(lock);
    if (!ptrs[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_fixed_scratch);
        if (e != cudaSuccess || !p)
            return fail(AB_ERR_CUDA, "cudaGetSymbolAddress(fixed scratch) failed on device %d: %s", dev,
                        cudaGetErrorString(e));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return AB_OK;
}

}  // namespace
}  // namespace ab

extern "C" int64_t aimet_b200_fixed_scratch_capacity(void) { return ab::kFixedScratchBytes; }

extern "C" int aimet_b200_quantize_dequantize_backward_fixed_scratch(
    const void *x, const void *grad_y, const void *scale, const void *offset, const ab_layout *layout,
    int io_dtype, int compute_dtype, int param_dtype, int64_t qmin, int64_t qmax, double zero_point_shift,
    void *grad_x, void *grad_scale, void *grad_offset, void *stream) {
    const int64_t need = aimet_b200_backward_scratch_bytes(layout, io_dtype);
    if (need < 0) return (int)need;
    if (need > ab::kFixedScratchBytes)
        return ab::fail(AB_ERR_SCRATCH,
                        "this layout needs %lld bytes of reduction scratch but the built-in buffer holds %lld; "
                        "use aimet_b200_quantize_dequantize_backward with a caller-provided buffer",
                        (long long)need, (long long)ab::kFixedScratchBytes);
    void *scratch = nullptr;
    int rc = ab::fixed_scratch_ptr(&scratch);
    if (rc != AB_OK) return rc;
    Call c{};
    c.op = ab::OP_QDQ;
    c.x = x; c.gy = grad_y; c.scale = scale; c.offset = offset; c.layout = layout;
    c.io = io_dtype; c.ct = compute_dtype; c.pt = param_dtype;
    c.qmin = qmin; c.qmax = qmax; c.zps = zero_point_shift;
    c.gx = grad_x; c.gs = grad_scale; c.go = grad_offset;
    c.scratch = scratch; c.scratch_bytes = ab::kFixedScratchBytes;
    c.stream = static_cast<cudaStream_t>(stream);
    return ab::dispatch(c, true);
}
