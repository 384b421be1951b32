// Device-side arithmetic of the affine quantizers, used by the kernels in affine.cu: the
// per-parameter set-up (Enc), the element functions that follow the reference op by op, and the
// straight-line fast paths over one 16-byte vector.
//
// Arithmetic follows QuantizeFunc / DequantizeFunc / QuantDequantFunc of the reference
// (quantization/affine/backends/torch_builtins.py:588-831) step by step, including the
// re-rounding to the internal dtype after every step when that dtype is float16 / bfloat16.
#pragma once

#include "common.cuh"

namespace ab {
namespace {

// OP_FQ: the arithmetic of torch.fake_quantize_per_{tensor,channel}_affine, which the reference
// calls instead of QuantDequantFunc whenever no scale / offset gradient is needed
// (torch_builtins.py:243-266, 335-431): out = (clamp(rint(x * (1/s)) + zp, qmin, qmax) - zp) * s
// in float32 with the integer zero point zp = -(int)offset.
enum { OP_Q = 0, OP_DQ = 1, OP_QDQ = 2, OP_FQ = 3 };

constexpr int kFwdUnroll = 4;       // 16-byte vectors in flight per thread, forward

// ---------------------------------------------------------------------------
// The quantization grid in the register type, plus facts about it that hold for
// the whole launch.
// ---------------------------------------------------------------------------
template <typename T> struct Grid {
    T qmin, qmax, zps;
    int has_zps;
    // 16-bit internal dtypes only: qmin-1 and qmax+1 are exact in that dtype, so
    // re-rounding an integer difference cannot move it across a grid boundary
    int exact_edges;
    // backward only: the input gradient of an element whose rounding error exceeds pgs_thr is
    // multiplied by pgs_mult (QuantDequantFunc.backward with the experimental "pivot gradient
    // spiking" switched on, torch_builtins.py:779-831); off unless has_pgs
    int has_pgs = 0;
    T pgs_thr = (T)0, pgs_mult = (T)1;
};

// ---------------------------------------------------------------------------
// Per-parameter values, rounded to the internal dtype once per 16-byte vector
// (or per element where neighbouring elements use different parameters).
// ---------------------------------------------------------------------------
template <int CT> struct Enc {
    using T = typename Arith<CT>::T;
    T s, o;
    T r;     // correctly rounded 1 / s (float arithmetic only)
    T back;  // what is added back after clamping: o, or o + zero_point_shift
    T lo, hi;  // o + qmin, o + qmax in the internal dtype (backward clamp bounds)
    T zp;      // -(int)o, the integer zero point of the fake-quantize arithmetic
    // float arithmetic: s is a normal number of moderate magnitude and the clamp
    // bounds are small integers, so x / s can be formed from r with an exact
    // remainder correction and rounding can use the 2^23 trick
    bool fast;
    // 16-bit internal dtype: integer sums around this offset are exact
    bool exact_int;
};

// The raw (scale, offset) pair of parameter p, converted to the register type but not yet
// rounded; split from make_enc so that a kernel can request the pair well before it needs it.
template <int CT>
__device__ __forceinline__ void load_param(const ParamPtr &scale, const ParamPtr &offset, int64_t p,
                                           typename Arith<CT>::T &s, typename Arith<CT>::T &o) {
    using T = typename Arith<CT>::T;
    if (scale.f64) {
        s = (T) static_cast<const double *>(scale.p)[p];
        o = (T) static_cast<const double *>(offset.p)[p];
    } else {
        s = (T)__ldg(static_cast<const float *>(scale.p) + p);
        o = (T)__ldg(static_cast<const float *>(offset.p) + p);
    }
}

template <int CT>
__device__ __forceinline__ Enc<CT> make_enc(typename Arith<CT>::T s_raw, typename Arith<CT>::T o_raw,
                                            const Grid<typename Arith<CT>::T> &g) {
    using A = Arith<CT>;
    using T = typename A::T;
    Enc<CT> e;
    e.s = A::rnd(s_raw);
    e.o = A::rnd(o_raw);
    e.back = g.has_zps ? A::rnd(op_add(e.o, g.zps)) : e.o;
    e.lo = A::rnd(op_add(e.o, g.qmin));
    e.hi = A::rnd(op_add(e.o, g.qmax));
    e.r = (T)0;
    e.zp = (T)0;
    e.fast = false;
    e.exact_int = false;
    if (CT != AB_F64) {
        const float as = fabsf((float)e.s);
        const float bound = fmaxf(fabsf((float)e.lo), fabsf((float)e.hi));
        e.fast = (as > 7.888609e-31f) && (as < 1.2676506e30f) && (bound < 4194304.0f);  // 2^-100, 2^100, 2^22
        e.r = (T)__frcp_rn((float)e.s);
        e.zp = (T)(-(float)__float2int_rz((float)e.o));
        // all integers up to 2^(mantissa+1) are exact: 256 for bfloat16, 2048 for float16
        const float lim = CT == AB_BF16 ? 256.0f : 2048.0f;
        e.exact_int = g.exact_edges && bound <= lim && fabsf((float)e.o) <= lim && (float)e.o == rintf((float)e.o);
    }
    return e;
}

template <int CT>
__device__ __forceinline__ Enc<CT> load_enc(const ParamPtr &scale, const ParamPtr &offset, int64_t p,
                                            const Grid<typename Arith<CT>::T> &g) {
    typename Arith<CT>::T s, o;
    load_param<CT>(scale, offset, p, s, o);
    return make_enc<CT>(s, o, g);
}

// x / s, correctly rounded.  With r = RN(1/s): q0 = RN(x*r) is within one ulp,
// the remainder x - q0*s is exact in an fma, and RN(q0 + rem*r) is the correctly
// rounded quotient (Markstein).  Infinities, NaN and absurd magnitudes take the
// IEEE division instruction.
template <int CT>
__device__ __forceinline__ typename Arith<CT>::T div_scale(typename Arith<CT>::T x, const Enc<CT> &e) {
    return op_div(x, e.s);
}
__device__ __forceinline__ float div_scale_f32(float x, float sc, float r, bool fast) {
    if (!fast) return __fdiv_rn(x, sc);
    const float q0 = __fmul_rn(x, r);
    float rem = __fmaf_rn(-q0, sc, x);
    // +-inf, NaN and quotients beyond 2^100 keep q0 (the remainder would be NaN);
    // such quotients are far outside any grid, so their last bit is immaterial
    rem = fabsf(q0) < 1.2676506e30f ? rem : 0.0f;
    return __fmaf_rn(rem, r, q0);
}
template <> __device__ __forceinline__ float div_scale<AB_F32>(float x, const Enc<AB_F32> &e) { return div_scale_f32(x, e.s, e.r, e.fast); }
template <> __device__ __forceinline__ float div_scale<AB_BF16>(float x, const Enc<AB_BF16> &e) { return div_scale_f32(x, e.s, e.r, e.fast); }
template <> __device__ __forceinline__ float div_scale<AB_F16>(float x, const Enc<AB_F16> &e) { return div_scale_f32(x, e.s, e.r, e.fast); }

// Round half to even.  In float, (|v| + 2^23) - 2^23 is exact rounding for
// |v| < 2^23; larger magnitudes stay far outside any grid whose clamp bounds are
// below 2^22 (Enc::fast), which is all the callers need of them.
template <int CT>
__device__ __forceinline__ typename Arith<CT>::T round_even(typename Arith<CT>::T v, const Enc<CT> &e) {
    return op_rint(v);
}
__device__ __forceinline__ float round_even_f32(float v, bool fast) {
    if (!fast) return rintf(v);
    const float r = __fsub_rn(__fadd_rn(fabsf(v), 8388608.0f), 8388608.0f);
    return copysignf(r, v);
}
template <> __device__ __forceinline__ float round_even<AB_F32>(float v, const Enc<AB_F32> &e) { return round_even_f32(v, e.fast); }
template <> __device__ __forceinline__ float round_even<AB_BF16>(float v, const Enc<AB_BF16> &e) { return round_even_f32(v, e.fast); }
template <> __device__ __forceinline__ float round_even<AB_F16>(float v, const Enc<AB_F16> &e) { return round_even_f32(v, e.fast); }

// torch.clamp semantics (NaN propagates) in two instructions
__device__ __forceinline__ float clamp_prop(float v, float lo, float hi) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "f"(lo));
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(r), "f"(hi));
    return r;
}
__device__ __forceinline__ double clamp_prop(double v, double lo, double hi) { return clamp_nan(v, lo, hi); }

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
    if (OP == OP_FQ) {
        // the int64 cast of the reference kernel is the identity on integer-valued floats and its
        // saturation coincides with the clamp; NaN converts to 0 on the device
        T t = op_add(round_even<CT>(op_mul(x, e.r), e), e.zp);
        t = (t != t) ? (T)0 : t;
        t = t < g.qmin ? g.qmin : (t > g.qmax ? g.qmax : t);
        return op_mul(op_sub(t, e.zp), e.s);
    }
    T t = A::rnd(div_scale<CT>(x, e));
    if (OP == OP_QDQ && g.has_zps) t = A::rnd(op_sub(t, g.zps));
    t = round_even<CT>(t, e);
    t = op_sub(t, e.o);
    if (!e.exact_int) t = A::rnd(t);
    t = clamp_prop(t, g.qmin, g.qmax);
    if (OP == OP_Q) return t;
    t = op_add(t, e.back);
    if (!e.exact_int || g.has_zps) t = A::rnd(t);
    return A::rnd(op_mul(t, e.s));
}

// ---------------------------------------------------------------------------
// backward element functions: returns the input gradient and this element's
// contribution to the scale / offset gradients
// ---------------------------------------------------------------------------
template <int CT, int OP, bool WANT_O>
__device__ __forceinline__ typename Arith<CT>::T bwd_elem(typename Arith<CT>::T x,
                                                          typename Arith<CT>::T gy, const Enc<CT> &e,
                                                          const Grid<typename Arith<CT>::T> &g,
                                                          typename Arith<CT>::T &ds,
                                                          typename Arith<CT>::T &dofs) {
    using A = Arith<CT>;
    using T = typename A::T;
    dofs = (T)0;
    if (OP == OP_FQ) {
        T t = op_add(round_even<CT>(op_mul(x, e.r), e), e.zp);
        t = (t != t) ? (T)0 : t;
        ds = (T)0;
        return ((g.qmin <= t) && (t <= g.qmax)) ? gy : (T)0;
    }
    if (OP == OP_DQ) {
        T dx = A::rnd(op_mul(gy, e.s));
        ds = A::rnd(op_mul(gy, A::rnd(op_add(x, e.o))));
        if (WANT_O) dofs = dx;
        return dx;
    }
    if (OP == OP_Q) {
        T xs = A::rnd(div_scale<CT>(x, e));
        T t = A::rnd(op_sub(round_even<CT>(xs, e), e.o));
        bool in = (t >= g.qmin) && (t <= g.qmax);
        T mg = op_mul(gy, in ? (T)1 : (T)0);
        T dx = A::rnd(op_div(mg, e.s));
        ds = A::rnd(op_mul(-dx, xs));
        if (WANT_O) dofs = -mg;
        return dx;
    }
    // OP_QDQ
    T xs = A::rnd(div_scale<CT>(x, e));
    if (g.has_zps) xs = A::rnd(op_sub(xs, g.zps));
    T xr = round_even<CT>(xs, e);
    T t = op_sub(xr, e.o);
    if (!e.exact_int) t = A::rnd(t);
    bool in = (g.qmin <= t) && (t <= g.qmax);
    // xr - xs needs no re-rounding: its bits are a subset of the fraction bits of xs
    T err = op_sub(xr, xs);
    T xc = clamp_prop(xr, e.lo, e.hi);
    if (g.has_zps) xc = A::rnd(op_add(xc, g.zps));
    ds = A::rnd(op_mul(gy, in ? err : xc));
    if (WANT_O) dofs = in ? (T)0 : A::rnd(op_mul(gy, e.s));
    if (g.has_pgs) {
        // the product is in the gradient's dtype: the store conversion does that rounding
        const T mag = err < (T)0 ? -err : err;
        return in ? (mag > g.pgs_thr ? op_mul(gy, g.pgs_mult) : gy) : (T)0;
    }
    return in ? gy : (T)0;
}

// ---------------------------------------------------------------------------
// Two elements at a time (same parameter): identical arithmetic to fwd_elem /
// bwd_elem with the re-roundings to a 16-bit internal dtype done pairwise.
// ---------------------------------------------------------------------------
template <int CT, int OP>
__device__ __forceinline__ void fwd_pair(typename Arith<CT>::T &a, typename Arith<CT>::T &b, const Enc<CT> &e,
                                         const Grid<typename Arith<CT>::T> &g) {
    using A = Arith<CT>;
    if (OP != OP_QDQ) {
        a = fwd_elem<CT, OP>(a, e, g);
        b = fwd_elem<CT, OP>(b, e, g);
        return;
    }
    a = div_scale<CT>(a, e);
    b = div_scale<CT>(b, e);
    A::rnd2(a, b);
    if (g.has_zps) {
        a = op_sub(a, g.zps);
        b = op_sub(b, g.zps);
        A::rnd2(a, b);
    }
    a = op_sub(round_even<CT>(a, e), e.o);
    b = op_sub(round_even<CT>(b, e), e.o);
    if (!e.exact_int) A::rnd2(a, b);
    a = op_add(clamp_prop(a, g.qmin, g.qmax), e.back);
    b = op_add(clamp_prop(b, g.qmin, g.qmax), e.back);
    if (!e.exact_int || g.has_zps) A::rnd2(a, b);
    // the product is re-rounded by the store conversion when the output dtype is
    // the internal dtype; VecCvt::pack does that rounding
    a = op_mul(a, e.s);
    b = op_mul(b, e.s);
}

template <int CT, int OP, bool WANT_O>
__device__ __forceinline__ void bwd_pair(typename Arith<CT>::T &xa, typename Arith<CT>::T &xb,
                                         typename Arith<CT>::T ga, typename Arith<CT>::T gb, const Enc<CT> &e,
                                         const Grid<typename Arith<CT>::T> &g, typename Arith<CT>::T &acc_s,
                                         typename Arith<CT>::T &acc_o) {
    using A = Arith<CT>;
    using T = typename A::T;
    if (OP != OP_QDQ) {
        T ds, dofs;
        xa = bwd_elem<CT, OP, WANT_O>(xa, ga, e, g, ds, dofs);
        acc_s += ds;
        acc_o += dofs;
        xb = bwd_elem<CT, OP, WANT_O>(xb, gb, e, g, ds, dofs);
        acc_s += ds;
        acc_o += dofs;
        return;
    }
    T sa = div_scale<CT>(xa, e), sb = div_scale<CT>(xb, e);
    A::rnd2(sa, sb);
    if (g.has_zps) {
        sa = op_sub(sa, g.zps);
        sb = op_sub(sb, g.zps);
        A::rnd2(sa, sb);
    }
    const T ra = round_even<CT>(sa, e), rb = round_even<CT>(sb, e);
    T ta = op_sub(ra, e.o), tb = op_sub(rb, e.o);
    if (!e.exact_int) A::rnd2(ta, tb);
    const bool ina = (g.qmin <= ta) && (ta <= g.qmax);
    const bool inb = (g.qmin <= tb) && (tb <= g.qmax);
    T ca = clamp_prop(ra, e.lo, e.hi), cb = clamp_prop(rb, e.lo, e.hi);
    if (g.has_zps) {
        ca = op_add(ca, g.zps);
        cb = op_add(cb, g.zps);
        A::rnd2(ca, cb);
    }
    T da = op_mul(ga, ina ? op_sub(ra, sa) : ca);
    T db = op_mul(gb, inb ? op_sub(rb, sb) : cb);
    A::rnd2(da, db);
    acc_s += da;
    acc_s += db;
    if (WANT_O) {
        T oa = op_mul(ga, e.s), ob = op_mul(gb, e.s);
        A::rnd2(oa, ob);
        acc_o += ina ? (T)0 : oa;
        acc_o += inb ? (T)0 : ob;
    }
    if (g.has_pgs) {
        const T ea = op_sub(ra, sa), eb = op_sub(rb, sb);
        if ((ea < (T)0 ? -ea : ea) > g.pgs_thr) ga = op_mul(ga, g.pgs_mult);
        if ((eb < (T)0 ? -eb : eb) > g.pgs_thr) gb = op_mul(gb, g.pgs_mult);
    }
    xa = ina ? ga : (T)0;
    xb = inb ? gb : (T)0;
}

// ---------------------------------------------------------------------------
// Straight-line fast paths for a whole 16-byte vector sharing one parameter pair.
// Preconditions (checked once per vector by the caller): float arithmetic,
// Enc::fast (moderate scale, clamp bounds below 2^22), no zero-point shift, an
// integer offset, and for a 16-bit internal dtype Enc::exact_int.  Under these
//   * x / s comes from the exact-remainder form (div_scale_f32, no branches);
//   * t = v + 1.5*2^23 is the integer nearest to v (ties to even) plus the magic
//     constant, and t - (1.5*2^23 + o) is round(v) - o in one exact subtraction
//     (both operands are integers below 2^24); values of |v| >= 2^22 come out
//     inexact but still far outside the clamp range, which is all that is
//     observable of them;
//   * integer sums need no re-rounding in the 16-bit internal dtypes.
// ---------------------------------------------------------------------------
constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23

template <int CT> __device__ __forceinline__ bool vec_fast_ok(const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g) {
    if (CT == AB_F64) return false;
    const bool int_offset = (float)e.o == rintf((float)e.o);
    const bool lowp_ok = (CT == AB_F32) || e.exact_int;
    return e.fast && !g.has_zps && !g.has_pgs && int_offset && lowp_ok;
}

// x / s by reciprocal and exact remainder.  GUARD keeps q0 when it is infinite or absurdly large
// (the remainder would be NaN); without it the caller has bounded |x| beforehand (clamp_abs16).
template <bool GUARD> __device__ __forceinline__ float div_fast(float x, float s, float r) {
    const float q0 = __fmul_rn(x, r);
    float rem = __fmaf_rn(-q0, s, x);
    if (GUARD) rem = fabsf(q0) < 1.2676506e30f ? rem : 0.0f;
    return __fmaf_rn(rem, r, q0);
}

// The same for two values at once with the two-wide float instructions (one issue slot for both).
template <bool GUARD> __device__ __forceinline__ float2 div_fast2(float2 x, float s, float r) {
    const float2 q0 = __fmul2_rn(x, make_float2(r, r));
    float2 rem = __ffma2_rn(q0, make_float2(-s, -s), x);  // x - q0 * s, exact
    if (GUARD) {
        rem.x = fabsf(q0.x) < 1.2676506e30f ? rem.x : 0.0f;
        rem.y = fabsf(q0.y) < 1.2676506e30f ? rem.y : 0.0f;
    }
    return __ffma2_rn(rem, make_float2(r, r), q0);
}

// The clamp is applied to round(v) + magic against (o + qmin) + magic and (o + qmax) + magic,
// which is clamp(round(v) - o, qmin, qmax) + o on exact integers; quantize subtracts magic + o
// afterwards, quantize-dequantize subtracts magic and multiplies by the scale.
template <int CT, int OP, int NV, bool GUARD>
__device__ __forceinline__ void fwd_vec_fast(float (&f)[NV], const Enc<CT> &e) {
    using A = Arith<CT>;
    const float s = (float)e.s, r = (float)e.r;
    const float c_lo = __fadd_rn(kMagic, (float)e.lo), c_hi = __fadd_rn(kMagic, (float)e.hi);  // exact: |lo|, |hi| < 2^22
    const float c_back = OP == OP_QDQ ? kMagic : __fadd_rn(kMagic, (float)e.o);
#pragma unroll
    for (int i = 0; i < NV; i += 2) {
        if constexpr (CT == AB_F32) {
            float2 t = __fadd2_rn(div_fast2<GUARD>(make_float2(f[i], f[i + 1]), s, r), make_float2(kMagic, kMagic));
            t.x = clamp_prop(t.x, c_lo, c_hi);
            t.y = clamp_prop(t.y, c_lo, c_hi);
            t = __fadd2_rn(t, make_float2(-c_back, -c_back));
            if (OP == OP_QDQ) t = __fmul2_rn(t, make_float2(s, s));
            f[i] = t.x;
            f[i + 1] = t.y;
        } else {
            float a = div_fast<GUARD>(f[i], s, r), b = div_fast<GUARD>(f[i + 1], s, r);
            A::rnd2(a, b);
            a = __fsub_rn(clamp_prop(__fadd_rn(a, kMagic), c_lo, c_hi), c_back);
            b = __fsub_rn(clamp_prop(__fadd_rn(b, kMagic), c_lo, c_hi), c_back);
            if (OP == OP_QDQ) {
                a = __fmul_rn(a, s);
                b = __fmul_rn(b, s);
            }
            f[i] = a;
            f[i + 1] = b;
        }
    }
}

// Backward of quantize-dequantize: x[] becomes the input gradient, the scale-gradient terms are
// added to acc_s.  An element is inside the grid exactly when clamping round(x / s) to
// [o + qmin, o + qmax] leaves it unchanged (NaN compares unequal, as in the reference's mask).
// The offset-gradient terms are added by the caller, which finds the (rare) masked elements by
// comparing the input gradient with the upstream gradient.
template <int CT, int NV, bool GUARD>
__device__ __forceinline__ void bwd_vec_fast(float (&x)[NV], const float (&gy)[NV], const Enc<CT> &e, float &acc_s,
                                             float &acc_s2) {
    using A = Arith<CT>;
    const float s = (float)e.s, r = (float)e.r;
    const float lo = (float)e.lo, hi = (float)e.hi;
#pragma unroll
    for (int i = 0; i < NV; i += 2) {
        if constexpr (CT == AB_F32) {
            // float32 arithmetic: two elements per instruction, and the product gy * term goes into
            // the running sums (one per element parity) through an fma, i.e. without the
            // intermediate rounding of the product -- the sums differ from any summation order of
            // the rounded products by less than that rounding
            const float2 sa = div_fast2<GUARD>(make_float2(x[i], x[i + 1]), s, r);
            const float2 ra = __fadd2_rn(__fadd2_rn(sa, make_float2(kMagic, kMagic)), make_float2(-kMagic, -kMagic));
            const float2 err = __ffma2_rn(sa, make_float2(-1.0f, -1.0f), ra);  // round(x / s) - x / s
            const float ca = clamp_prop(ra.x, lo, hi), cb = clamp_prop(ra.y, lo, hi);
            const bool ina = ca == ra.x, inb = cb == ra.y;
            const float2 acc = __ffma2_rn(make_float2(gy[i], gy[i + 1]), make_float2(ina ? err.x : ca, inb ? err.y : cb),
                                          make_float2(acc_s, acc_s2));
            acc_s = acc.x;
            acc_s2 = acc.y;
            x[i] = ina ? gy[i] : 0.0f;
            x[i + 1] = inb ? gy[i + 1] : 0.0f;
        } else {
            float sa = div_fast<GUARD>(x[i], s, r), sb = div_fast<GUARD>(x[i + 1], s, r);
            A::rnd2(sa, sb);
            const float ra = __fsub_rn(__fadd_rn(sa, kMagic), kMagic), rb = __fsub_rn(__fadd_rn(sb, kMagic), kMagic);
            const float ca = clamp_prop(ra, lo, hi), cb = clamp_prop(rb, lo, hi);
            const bool ina = ca == ra, inb = cb == rb;
            float da = __fmul_rn(gy[i], ina ? __fsub_rn(ra, sa) : ca);
            float db = __fmul_rn(gy[i + 1], inb ? __fsub_rn(rb, sb) : cb);
            A::rnd2(da, db);
            acc_s += da;
            acc_s2 += db;
            x[i] = ina ? gy[i] : 0.0f;
            x[i + 1] = inb ? gy[i + 1] : 0.0f;
        }
    }
}

// Offset-gradient terms of one vector, given the upstream gradient and the input gradient just
// computed from it: an element was masked exactly when the two differ bitwise (a masked zero
// contributes nothing either way).  Only called for vectors that contain such an element.
template <int CT, int NV>
__device__ __forceinline__ void bwd_offset_terms(const float (&dx)[NV], const float (&gy)[NV], float s, float &acc_o) {
    using A = Arith<CT>;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (__float_as_uint(dx[i]) != __float_as_uint(gy[i])) acc_o += A::rnd(__fmul_rn(gy[i], s));
}

// ---------------------------------------------------------------------------
// Packed 16-bit fast paths: when the internal dtype IS the tensor dtype (bfloat16 for <= 5-bit
// grids, float16 for <= 8-bit grids) every step after the division is a native two-wide
// half-precision instruction.  A native add / sub / mul rounds the exact result once to the
// 16-bit type; the reference computes the same operation in float and rounds to the 16-bit type,
// which is the same value whenever the float result is exact -- true for every operation below
// (products of two 8/11-bit significands, sums of small integers).  Rounding to an integer uses
// the 16-bit magic constant 1.5 * 2^(p-1) (p significant bits): exact for |v| < 2^(p-2); beyond
// that the result stays outside the grid as long as the clamp bounds are below 2^(p-3)
// (vec_packed_ok), which is all that is observable.
// ---------------------------------------------------------------------------
template <int CT> struct Packed;
template <> struct Packed<AB_BF16> {
    using H2 = __nv_bfloat162;
    static constexpr float kMagic16 = 192.0f;   // 1.5 * 2^7
    static constexpr float kLimit = 32.0f;      // 2^5
    static __device__ __forceinline__ H2 dup(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ H2 pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
    static __device__ __forceinline__ float lo(H2 v) { return __uint_as_float(*reinterpret_cast<uint32_t *>(&v) << 16); }
    static __device__ __forceinline__ float hi(H2 v) { return __uint_as_float(*reinterpret_cast<uint32_t *>(&v) & 0xffff0000u); }
};
template <> struct Packed<AB_F16> {
    using H2 = __half2;
    static constexpr float kMagic16 = 1536.0f;  // 1.5 * 2^10
    static constexpr float kLimit = 256.0f;     // 2^8
    static __device__ __forceinline__ H2 dup(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ H2 pack(float a, float b) { return __floats2half2_rn(a, b); }
    static __device__ __forceinline__ float lo(H2 v) { return __low2float(v); }
    static __device__ __forceinline__ float hi(H2 v) { return __high2float(v); }
};

template <int CT> __device__ __forceinline__ bool vec_packed_ok(const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g) {
    if (CT != AB_BF16 && CT != AB_F16) return false;
    const float lim = CT == AB_BF16 ? 32.0f : 256.0f;
    const float o = (float)e.o;
    return e.fast && e.exact_int && !g.has_zps && !g.has_pgs && o == rintf(o) && fabsf(o) <= lim &&
           fabsf((float)e.lo) <= lim && fabsf((float)e.hi) <= lim;
}

template <typename H2> __device__ __forceinline__ H2 bit_select(H2 a, H2 b, unsigned mask) {  // mask ? a : b
    const unsigned ua = *reinterpret_cast<unsigned *>(&a), ub = *reinterpret_cast<unsigned *>(&b);
    const unsigned r = (ua & mask) | (ub & ~mask);
    return *reinterpret_cast<const H2 *>(&r);
}

// Bound on |x| for 16-bit tensors, applied to the packed input before the division so that
// x * (1/s) cannot overflow: (largest clamp bound + 4) * |s| with some slack, as a pair of the
// tensor's own 16-bit type.  Returns false when that bound is not finite in the type.
template <int IO, int CT> __device__ __forceinline__ bool abs_bound16(const Enc<CT> &e, uint32_t &big2) {
    using P = Packed<IO>;
    const float bound = fmaxf(fabsf((float)e.lo), fabsf((float)e.hi));
    const float big = (bound + 4.0f) * fabsf((float)e.s) * 1.0625f;
    const typename P::H2 h = P::dup(big);
    big2 = *reinterpret_cast<const uint32_t *>(&h);
    return e.fast && P::lo(h) < 3.0e38f && P::lo(h) >= big * 0.99f;
}
template <int IO, typename E> __device__ __forceinline__ void clamp_abs16(Vec16<E> &v, uint32_t big2) {
    using H2 = typename Packed<IO>::H2;
    const uint32_t nb = big2 ^ 0x80008000u;
    const H2 pos = *reinterpret_cast<const H2 *>(&big2), neg = *reinterpret_cast<const H2 *>(&nb);
    H2 *w = reinterpret_cast<H2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __hmin2_nan(__hmax2_nan(w[i], neg), pos);
}

// E is the 16-bit tensor element type matching CT
template <int CT, int OP, typename E, bool GUARD>
__device__ __forceinline__ void fwd_vec_packed(const Vec16<E> &in, Vec16<E> &out, const Enc<CT> &e) {
    using P = Packed<CT>;
    using H2 = typename P::H2;
    const float s = (float)e.s, r = (float)e.r;
    const H2 magic = P::dup(P::kMagic16), s2 = P::dup(s);
    const H2 c_lo = P::dup(P::kMagic16 + (float)e.lo), c_hi = P::dup(P::kMagic16 + (float)e.hi);
    const H2 c_back = OP == OP_QDQ ? magic : P::dup(P::kMagic16 + (float)e.o);
    const H2 *ip = reinterpret_cast<const H2 *>(&in);
    H2 *op = reinterpret_cast<H2 *>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 ab = div_fast2<GUARD>(make_float2(P::lo(ip[i]), P::hi(ip[i])), s, r);
        H2 q = __hadd2(P::pack(ab.x, ab.y), magic);
        q = __hsub2(__hmin2_nan(__hmax2_nan(q, c_lo), c_hi), c_back);
        op[i] = OP == OP_QDQ ? __hmul2(q, s2) : q;
    }
}

template <int CT, typename E, bool GUARD>
__device__ __forceinline__ void bwd_vec_packed(const Vec16<E> &x, const Vec16<E> &gy, Vec16<E> &dx, const Enc<CT> &e,
                                               float &acc_s, float &acc_s2) {
    using P = Packed<CT>;
    using H2 = typename P::H2;
    const float s = (float)e.s, r = (float)e.r;
    const H2 magic = P::dup(P::kMagic16);
    const H2 lo2 = P::dup((float)e.lo), hi2 = P::dup((float)e.hi);
    const H2 *xp = reinterpret_cast<const H2 *>(&x);
    const H2 *gp = reinterpret_cast<const H2 *>(&gy);
    unsigned *dp = reinterpret_cast<unsigned *>(&dx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 ab = div_fast2<GUARD>(make_float2(P::lo(xp[i]), P::hi(xp[i])), s, r);
        const H2 v = P::pack(ab.x, ab.y);                    // x / s in the internal dtype
        const H2 rd = __hsub2(__hadd2(v, magic), magic);     // round(x / s)
        const H2 cl = __hmin2_nan(__hmax2_nan(rd, lo2), hi2);
        const unsigned m = __heq2_mask(cl, rd);              // inside the grid (false for NaN)
        const H2 d = __hmul2(gp[i], bit_select(__hsub2(rd, v), cl, m));
        acc_s += P::lo(d);
        acc_s2 += P::hi(d);
        dp[i] = *reinterpret_cast<const unsigned *>(&gp[i]) & m;
    }
}

// Offset-gradient terms of one packed vector (see bwd_offset_terms).
template <int CT, typename E>
__device__ __forceinline__ void bwd_offset_terms_packed(const Vec16<E> &dx, const Vec16<E> &gy, float s, float &acc_o) {
    using P = Packed<CT>;
    using H2 = typename P::H2;
    const H2 s2 = P::dup(s);
    const H2 *gp = reinterpret_cast<const H2 *>(&gy);
    const unsigned *dw = reinterpret_cast<const unsigned *>(&dx);
    const unsigned *gw = reinterpret_cast<const unsigned *>(&gy);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const unsigned diff = dw[i] ^ gw[i];
        const H2 od = __hmul2(gp[i], s2);
        if (diff & 0xffffu) acc_o += P::lo(od);
        if (diff >> 16) acc_o += P::hi(od);
    }
}

template <typename E> __device__ __forceinline__ bool same_bits(const Vec16<E> &a, const Vec16<E> &b) {
    const uint4 u = *reinterpret_cast<const uint4 *>(&a), w = *reinterpret_cast<const uint4 *>(&b);
    return u.x == w.x && u.y == w.y && u.z == w.z && u.w == w.w;
}

// ---------------------------------------------------------------------------
// One 16-byte vector through one of three bodies that give identical results: the generic one
// follows the reference op by op, PATH_FAST / PATH_PACKED are the straight-line forms above.
// PRE: the packed input is bounded first (16-bit tensors), which replaces the overflow guard.
// ---------------------------------------------------------------------------
enum { PATH_GENERIC = 0, PATH_FAST = 1, PATH_PACKED = 2 };

template <int IO, int CT, int OP, int PATH, bool PRE>
__device__ __forceinline__ void fwd_vec(Vec16<typename Elem<IO>::type> xv, Vec16<typename Elem<IO>::type> &yv,
                                        const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2) {
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    constexpr int NV = 16 / (int)sizeof(E);
    if constexpr (PRE) clamp_abs16<IO, E>(xv, big2);
    if constexpr (PATH == PATH_PACKED) {
        fwd_vec_packed<CT, OP, E, !PRE>(xv, yv, e);
    } else {
        T f[NV];
        VecCvt<T, E>::unpack(xv, f);
        if constexpr (PATH == PATH_FAST) {
            fwd_vec_fast<CT, OP, NV, !PRE>(f, e);
        } else {
#pragma unroll
            for (int i = 0; i + 1 < NV; i += 2) fwd_pair<CT, OP>(f[i], f[i + 1], e, g);
        }
        VecCvt<T, E>::pack(f, yv);
    }
}

template <int IO, int CT, int OP, bool WANT_O, int PATH, bool PRE>
__device__ __forceinline__ void bwd_vec(Vec16<typename Elem<IO>::type> xv, const Vec16<typename Elem<IO>::type> &gv,
                                        Vec16<typename Elem<IO>::type> &dv, const Enc<CT> &e,
                                        const Grid<typename Arith<CT>::T> &g, uint32_t big2,
                                        typename Arith<CT>::T &acc_s, typename Arith<CT>::T &acc_s2,
                                        typename Arith<CT>::T &acc_o) {
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    constexpr int NV = 16 / (int)sizeof(E);
    if constexpr (PRE) clamp_abs16<IO, E>(xv, big2);
    if constexpr (PATH == PATH_PACKED) {
        bwd_vec_packed<CT, E, !PRE>(xv, gv, dv, e, acc_s, acc_s2);
        if (WANT_O) {
            if (!same_bits(dv, gv)) bwd_offset_terms_packed<CT, E>(dv, gv, (float)e.s, acc_o);
        }
    } else {
        T fx[NV], fg[NV];
        VecCvt<T, E>::unpack(xv, fx);
        VecCvt<T, E>::unpack(gv, fg);
        if constexpr (PATH == PATH_FAST) {
            bwd_vec_fast<CT, NV, !PRE>(fx, fg, e, acc_s, acc_s2);
            VecCvt<T, E>::pack(fx, dv);
            if (WANT_O) {
                if (!same_bits(dv, gv)) bwd_offset_terms<CT, NV>(fx, fg, (float)e.s, acc_o);
            }
        } else {
#pragma unroll
            for (int i = 0; i + 1 < NV; i += 2)
                bwd_pair<CT, OP, WANT_O>(fx[i], fx[i + 1], fg[i], fg[i + 1], e, g, acc_s, acc_o);
            VecCvt<T, E>::pack(fx, dv);
        }
    }
}

}  // namespace
}  // namespace ab
