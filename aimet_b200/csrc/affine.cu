// Affine quantize / dequantize / quantize-dequantize: one fused elementwise
// pass forward, one fused pass backward (input gradient + deterministic
// reduction of the scale / offset gradients).
//
// Arithmetic follows QuantizeFunc / DequantizeFunc / QuantDequantFunc of the
// reference (quantization/affine/backends/torch_builtins.py:588-831) step by
// step, including the re-rounding to the internal dtype after every step when
// that dtype is float16 / bfloat16.
#include "common.cuh"

namespace ab {
namespace {

enum { OP_Q = 0, OP_DQ = 1, OP_QDQ = 2 };

constexpr int kFwdUnroll = 4;       // 16-byte vectors in flight per thread, forward

// ---------------------------------------------------------------------------
// per-parameter values, rounded to the internal dtype once
// ---------------------------------------------------------------------------
template <int CT> struct Enc {
    using T = typename Arith<CT>::T;
    T s, o;
};

template <int CT>
__device__ __forceinline__ Enc<CT> load_enc(const ParamPtr &scale, const ParamPtr &offset, int64_t p) {
    using A = Arith<CT>;
    using T = typename A::T;
    Enc<CT> e;
    if (scale.f64) {
        e.s = A::rnd((T) static_cast<const double *>(scale.p)[p]);
        e.o = A::rnd((T) static_cast<const double *>(offset.p)[p]);
    } else {
        e.s = A::rnd((T)__ldg(static_cast<const float *>(scale.p) + p));
        e.o = A::rnd((T)__ldg(static_cast<const float *>(offset.p) + p));
    }
    return e;
}

template <typename T> struct Grid {  // quantization grid, in the register type
    T qmin, qmax, zps;
    int has_zps;
};

// ---------------------------------------------------------------------------
// forward element functions
// ---------------------------------------------------------------------------
template <int CT, int OP>
__device__ __forceinline__ typename Arith<CT>::T fwd_elem(typename Arith<CT>::T x, const Enc<CT> &e,
                                                          const Grid<typename Arith<CT>::T> &g) {
    using A = Arith<CT>;
    using T = typename A::T;
    if (OP == OP_DQ) {
        T t = A::rnd(op_add(x, e.o));
        return A::rnd(op_mul(t, e.s));
    }
    T t = A::rnd(op_div(x, e.s));
    if (OP == OP_QDQ && g.has_zps) t = A::rnd(op_sub(t, g.zps));
    t = op_rint(t);
    t = A::rnd(op_sub(t, e.o));
    t = clamp_nan(t, g.qmin, g.qmax);
    if (OP == OP_Q) return t;
    T back = g.has_zps ? A::rnd(op_add(e.o, g.zps)) : e.o;
    t = A::rnd(op_add(t, back));
    return A::rnd(op_mul(t, e.s));
}

// ---------------------------------------------------------------------------
// backward element functions: returns input gradient, adds this element's
// contribution to the scale / offset gradient accumulators
// ---------------------------------------------------------------------------
template <int CT, int OP>
__device__ __forceinline__ typename Arith<CT>::T bwd_elem(typename Arith<CT>::T x,
                                                          typename Arith<CT>::T gy, const Enc<CT> &e,
                                                          const Grid<typename Arith<CT>::T> &g,
                                                          typename Arith<CT>::T &ds,
                                                          typename Arith<CT>::T &dofs) {
    using A = Arith<CT>;
    using T = typename A::T;
    if (OP == OP_DQ) {
        T dx = A::rnd(op_mul(gy, e.s));
        ds = A::rnd(op_mul(gy, A::rnd(op_add(x, e.o))));
        dofs = dx;
        return dx;
    }
    if (OP == OP_Q) {
        T xs = A::rnd(op_div(x, e.s));
        T t = A::rnd(op_sub(op_rint(xs), e.o));
        bool in = (t >= g.qmin) && (t <= g.qmax);
        T mg = op_mul(gy, in ? (T)1 : (T)0);
        T dx = A::rnd(op_div(mg, e.s));
        ds = A::rnd(op_mul(-dx, xs));
        dofs = -mg;
        return dx;
    }
    // OP_QDQ
    T xs = A::rnd(op_div(x, e.s));
    if (g.has_zps) xs = A::rnd(op_sub(xs, g.zps));
    T xr = op_rint(xs);
    T t = A::rnd(op_sub(xr, e.o));
    bool in = (g.qmin <= t) && (t <= g.qmax);
    T err = A::rnd(op_sub(xr, xs));
    T lo = A::rnd(op_add(e.o, g.qmin));
    T hi = A::rnd(op_add(e.o, g.qmax));
    T xc = clamp_nan(xr, lo, hi);
    if (g.has_zps) xc = A::rnd(op_add(xc, g.zps));
    ds = A::rnd(op_mul(gy, in ? err : xc));
    dofs = in ? (T)0 : A::rnd(op_mul(gy, e.s));
    return in ? gy : (T)0;
}

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
};

template <int IO, int CT, int OP, bool VECT>
__global__ void __launch_bounds__(kThreads) k_fwd_oci(FwdArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0};
    const int64_t nvec = a.numel / VEC;
    const bool uniform = (a.cm.I % VEC) == 0;
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    E *__restrict__ yp = static_cast<E *>(a.y);

    const int64_t base = (int64_t)blockIdx.x * (kThreads * kFwdUnroll) + threadIdx.x;
    if (VECT) {
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
                Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v * VEC));
#pragma unroll
                for (int i = 0; i < VEC; ++i) yv.v[i] = C::store(fwd_elem<CT, OP>(C::load(xv[u].v[i]), e, g));
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v * VEC + i));
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
            Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.cm.of(v));
            yp[v] = C::store(fwd_elem<CT, OP>(C::load(xp[v]), e, g));
        }
    }
}

struct FwdGenArgs {
    const void *x;
    void *y;
    ParamPtr scale, offset;
    int64_t numel;
    GenMap gm;
    double qmin, qmax, zps;
};

template <int IO, int CT, int OP>
__global__ void __launch_bounds__(kThreads) k_fwd_gen(FwdGenArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0};
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    E *__restrict__ yp = static_cast<E *>(a.y);
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < a.numel; i += stride) {
        Enc<CT> e = load_enc<CT>(a.scale, a.offset, a.gm.of(i));
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
};

template <int CT> __device__ __forceinline__ double finalize(double v) {
    using A = Arith<CT>;
    using T = typename A::T;
    return (double)A::rnd((T)v);
}

// One group of `group` threads per pseudo-segment; a pseudo-segment is a
// contiguous run of elements that share one parameter.
template <int IO, int CT, int OP, bool VECT>
__global__ void __launch_bounds__(kThreads) k_bwd_seg(BwdArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0};
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    const E *__restrict__ gp = static_cast<const E *>(a.gy);
    E *__restrict__ dxp = static_cast<E *>(a.gx);

    const int G = a.group;
    const int groups_per_cta = kThreads / G;
    const int64_t s = (int64_t)blockIdx.x * groups_per_cta + threadIdx.x / G;
    const int lane = threadIdx.x % G;
    const bool valid = s < a.nseg;

    T acc_s = 0, acc_o = 0;
    int64_t param = 0;
    if (valid) {
        const int64_t ts = s / a.nchunk;
        const int64_t k = s - ts * a.nchunk;
        const int64_t start = ts * a.cm.I + k * a.seg_len;
        int64_t len = a.cm.I - k * a.seg_len;
        if (len > a.seg_len) len = a.seg_len;
        param = a.cm.wrap ? ts % a.cm.C : ts;
        if (a.cm.C == 1) param = 0;
        const Enc<CT> e = load_enc<CT>(a.scale, a.offset, param);
        const int64_t nv = len / VEC;
        const int64_t v0 = start / VEC;
        for (int64_t v = lane; v < nv; v += 2 * (int64_t)G) {
            const int64_t va = v0 + v, vb = va + G;
            const bool hb = v + G < nv;
            if (VECT) {
                Vec16<E> xa, ga, xb, gb, da, db;
                xa = reinterpret_cast<const Vec16<E> *>(xp)[va];
                ga = reinterpret_cast<const Vec16<E> *>(gp)[va];
                if (hb) {
                    xb = reinterpret_cast<const Vec16<E> *>(xp)[vb];
                    gb = reinterpret_cast<const Vec16<E> *>(gp)[vb];
                }
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    T ds, dofs;
                    da.v[i] = C::store(bwd_elem<CT, OP>(C::load(xa.v[i]), C::load(ga.v[i]), e, g, ds, dofs));
                    acc_s += ds;
                    acc_o += dofs;
                }
                if (dxp) reinterpret_cast<Vec16<E> *>(dxp)[va] = da;
                if (hb) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        T ds, dofs;
                        db.v[i] = C::store(bwd_elem<CT, OP>(C::load(xb.v[i]), C::load(gb.v[i]), e, g, ds, dofs));
                        acc_s += ds;
                        acc_o += dofs;
                    }
                    if (dxp) reinterpret_cast<Vec16<E> *>(dxp)[vb] = db;
                }
            } else {
                T ds, dofs;
                T dx = bwd_elem<CT, OP>(C::load(xp[va]), C::load(gp[va]), e, g, ds, dofs);
                acc_s += ds;
                acc_o += dofs;
                if (dxp) dxp[va] = C::store(dx);
                if (hb) {
                    dx = bwd_elem<CT, OP>(C::load(xp[vb]), C::load(gp[vb]), e, g, ds, dofs);
                    acc_s += ds;
                    acc_o += dofs;
                    if (dxp) dxp[vb] = C::store(dx);
                }
            }
        }
    }

    // fixed-order reduction over the group
    double rs = (double)acc_s, ro = (double)acc_o;
    const int span = G < 32 ? G : 32;
    for (int o = span >> 1; o > 0; o >>= 1) {
        rs += __shfl_xor_sync(0xffffffffu, rs, o);
        ro += __shfl_xor_sync(0xffffffffu, ro, o);
    }
    if (G > 32) {
        __shared__ double sh[2][kThreads / 32];
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
            if (a.gs.p) a.gs.put(param, finalize<CT>(rs));
            if (a.go.p) a.go.put(param, finalize<CT>(ro));
        } else {
            a.partial[2 * s] = rs;
            a.partial[2 * s + 1] = ro;
        }
    }
}

// Column mode for small inner extents under a large outer dim: the tensor is a
// (rows, row_len) matrix whose columns each belong to one parameter; a thread
// owns one 16-byte column group and walks down a tile of rows.
template <int IO, int CT, int OP, bool VECT>
__global__ void __launch_bounds__(kThreads) k_bwd_col(BwdArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0};
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
        e[i] = load_enc<CT>(a.scale, a.offset, p);
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
            da.v[i] = C::store(bwd_elem<CT, OP>(C::load(xa.v[i]), C::load(ga.v[i]), e[i], g, ds, dofs));
            acc_s[i] += ds;
            acc_o[i] += dofs;
        }
        if (hb) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                T ds, dofs;
                db.v[i] = C::store(bwd_elem<CT, OP>(C::load(xb.v[i]), C::load(gb.v[i]), e[i], g, ds, dofs));
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

template <int CT> __global__ void __launch_bounds__(kThreads) k_bwd_finish(FinishArgs a) {
    const int64_t c = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (c >= a.nparam) return;
    double rs = 0, ro = 0;
    const int64_t n = a.na * a.nb;
    for (int64_t t = lane; t < n; t += 32) {
        const int64_t ia = t / a.nb, ib = t - ia * a.nb;
        const double *p = a.partial + 2 * (ia * a.sa + c * a.sc + ib);
        rs += p[0];
        ro += p[1];
    }
    rs = warp_sum(rs);
    ro = warp_sum(ro);
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
};

template <int IO, int CT, int OP>
__global__ void __launch_bounds__(kThreads) k_bwd_gen(BwdGenArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0};
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
        const Enc<CT> e = load_enc<CT>(a.scale, a.offset, p);
        T acc_s = 0, acc_o = 0;
        for (int64_t t = lane; t < a.box; t += 32) {
            int64_t off = base, r = t;
            for (int k = a.nd - 1; k >= 0; --k) {
                int64_t c = r % a.block[k];
                r /= a.block[k];
                off += c * a.estride[k];
            }
            T ds, dofs;
            T dx = bwd_elem<CT, OP>(C::load(xp[off]), C::load(gp[off]), e, g, ds, dofs);
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
inline BwdPlan plan_backward(const Canon &c, int io_dtype, bool ptr_aligned) { return plan_reduce(c, io_dtype, ptr_aligned); }

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
        const bool vect = aligned16(c.x) && aligned16(c.y) && (canon.numel % vecw == 0);
        const int64_t nvec = vect ? canon.numel / vecw : canon.numel;
        const int64_t per_cta = (int64_t)kThreads * kFwdUnroll;
        const int64_t grid = (nvec + per_cta - 1) / per_cta;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (vect)
            k_fwd_oci<IO, CT, OP, true><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else
            k_fwd_oci<IO, CT, OP, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
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
        int64_t grid = (canon.numel + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (grid > cap) grid = cap;
        k_fwd_gen<IO, CT, OP><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
    }
    AB_LAUNCH_OK();
    return AB_OK;
}

template <int IO, int CT, int OP> int launch_backward(const Call &c, const Canon &canon) {
    if (canon.numel == 0) return AB_OK;
    const bool al = aligned16(c.x) && aligned16(c.gy) && (!c.gx || aligned16(c.gx));
    const BwdPlan p = plan_backward(canon, IO, al);
    const ParamOut gs{c.gs, c.pt == AB_F64}, go{c.go, c.pt == AB_F64};
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
        int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (grid > cap) grid = cap;
        k_bwd_gen<IO, CT, OP><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
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

    if (p.mode == BwdPlan::SEG) {
        const int gpc = kThreads / p.group;
        const int64_t grid = (p.nseg + gpc - 1) / gpc;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (p.vect)
            k_bwd_seg<IO, CT, OP, true><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else
            k_bwd_seg<IO, CT, OP, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
    } else {
        const int v = p.vect ? 16 / dtype_size(IO) : 1;
        const int64_t gx = (a.row_len / v + kThreads - 1) / kThreads;
        if (gx > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        dim3 grid((unsigned)gx, (unsigned)p.row_tiles);
        if (p.vect)
            k_bwd_col<IO, CT, OP, true><<<grid, kThreads, 0, c.stream>>>(a);
        else
            k_bwd_col<IO, CT, OP, false><<<grid, kThreads, 0, c.stream>>>(a);
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
        const int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
        k_bwd_finish<CT><<<(unsigned)grid, kThreads, 0, c.stream>>>(f);
        AB_LAUNCH_OK();
    }
    return AB_OK;
}

template <int IO, int CT> int dispatch_op(const Call &c, const Canon &canon, bool backward) {
    switch (c.op) {
        case OP_Q: return backward ? launch_backward<IO, CT, OP_Q>(c, canon) : launch_forward<IO, CT, OP_Q>(c, canon);
        case OP_DQ: return backward ? launch_backward<IO, CT, OP_DQ>(c, canon) : launch_forward<IO, CT, OP_DQ>(c, canon);
        case OP_QDQ: return backward ? launch_backward<IO, CT, OP_QDQ>(c, canon) : launch_forward<IO, CT, OP_QDQ>(c, canon);
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
