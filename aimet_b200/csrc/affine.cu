// Affine quantize / dequantize / quantize-dequantize: one fused elementwise
// pass forward, one fused pass backward (input gradient + deterministic
// reduction of the scale / offset gradients).
//
// Arithmetic follows QuantizeFunc / DequantizeFunc / QuantDequantFunc of the
// reference (quantization/affine/backends/torch_builtins.py:588-831) step by
// step, including the re-rounding to the internal dtype after every step when
// that dtype is float16 / bfloat16.
#include <mutex>

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

template <int CT>
__device__ __forceinline__ Enc<CT> load_enc(const ParamPtr &scale, const ParamPtr &offset, int64_t p,
                                            const Grid<typename Arith<CT>::T> &g) {
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
    return e.fast && !g.has_zps && int_offset && lowp_ok;
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
    return e.fast && e.exact_int && !g.has_zps && o == rintf(o) && fabsf(o) <= lim &&
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

enum { PATH_GENERIC = 0, PATH_FAST = 1, PATH_PACKED = 2 };

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

template <int IO, int CT, int OP, int PATH, bool PRE>
__device__ __forceinline__ void fwd_seg_loop(const Vec16<typename Elem<IO>::type> *__restrict__ px,
                                             Vec16<typename Elem<IO>::type> *__restrict__ py, int lane, int nv, int G,
                                             const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2) {
    using E = typename Elem<IO>::type;
    constexpr int U = 4;
    int v = lane;
    const int step = U * G;
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
    for (; v < nv; v += G, px += G, py += G) {
        Vec16<E> yv;
        fwd_vec<IO, CT, OP, PATH, PRE>(*px, yv, e, g, big2);
        *py = yv;
    }
}

template <int IO, int CT, int OP>
__global__ void __launch_bounds__(kThreads, 5) k_fwd_seg(FwdSegArgs a) {
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    constexpr int NV = 16 / (int)sizeof(E);
    constexpr bool kIo16 = IO == AB_BF16 || IO == AB_F16;
    constexpr bool kQuant = OP == OP_QDQ || OP == OP_Q;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
    const SegPos p = seg_pos<NV>(a.cm, a.seg_len, a.nseg, a.nchunk, a.group);
    if (!p.valid) return;
    const Vec16<E> *px = static_cast<const Vec16<E> *>(a.x) + p.v0 + p.lane;
    Vec16<E> *py = static_cast<Vec16<E> *>(a.y) + p.v0 + p.lane;
    const Enc<CT> e = load_enc<CT>(a.scale, a.offset, p.param, g);
    if constexpr (kQuant && kIo16) {
        uint32_t big2;
        if (abs_bound16<IO, CT>(e, big2)) {
            if constexpr (CT == IO) {
                if (vec_packed_ok<CT>(e, g)) {
                    fwd_seg_loop<IO, CT, OP, PATH_PACKED, true>(px, py, p.lane, p.nv, a.group, e, g, big2);
                    return;
                }
            }
            if (vec_fast_ok<CT>(e, g)) {
                fwd_seg_loop<IO, CT, OP, PATH_FAST, true>(px, py, p.lane, p.nv, a.group, e, g, big2);
                return;
            }
        }
    } else if constexpr (kQuant && CT != AB_F64) {
        if (vec_fast_ok<CT>(e, g)) {
            fwd_seg_loop<IO, CT, OP, PATH_FAST, false>(px, py, p.lane, p.nv, a.group, e, g, 0u);
            return;
        }
    }
    fwd_seg_loop<IO, CT, OP, PATH_GENERIC, false>(px, py, p.lane, p.nv, a.group, e, g, 0u);
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
};

template <int CT> __device__ __forceinline__ double finalize(double v) {
    using A = Arith<CT>;
    using T = typename A::T;
    return (double)A::rnd((T)v);
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

template <int IO, int CT, int OP, bool WANT_O, int PATH, bool PRE>
__device__ __forceinline__ void bwd_seg_loop(const Vec16<typename Elem<IO>::type> *__restrict__ px,
                                             const Vec16<typename Elem<IO>::type> *__restrict__ pg,
                                             Vec16<typename Elem<IO>::type> *__restrict__ pd, int lane, int nv, int G,
                                             const Enc<CT> &e, const Grid<typename Arith<CT>::T> &g, uint32_t big2,
                                             typename Arith<CT>::T &acc_s, typename Arith<CT>::T &acc_o) {
    using E = typename Elem<IO>::type;
    using T = typename Arith<CT>::T;
    // the generic body also serves callers that want no input gradient; the others always store
    constexpr bool kMayskip = PATH == PATH_GENERIC;
    T acc_s2 = 0;
    int v = lane;
    const int step = 2 * G;
    for (; v + G < nv; v += step, px += step, pg += step) {
        const Vec16<E> xa = px[0], ga = pg[0], xb = px[G], gb = pg[G];
        Vec16<E> da, db;
        bwd_vec<IO, CT, OP, WANT_O, PATH, PRE>(xa, ga, da, e, g, big2, acc_s, acc_s2, acc_o);
        if (!kMayskip || pd) pd[0] = da;
        bwd_vec<IO, CT, OP, WANT_O, PATH, PRE>(xb, gb, db, e, g, big2, acc_s, acc_s2, acc_o);
        if (!kMayskip || pd) {
            pd[G] = db;
            pd += step;
        }
    }
    if (v < nv) {
        Vec16<E> da;
        bwd_vec<IO, CT, OP, WANT_O, PATH, PRE>(*px, *pg, da, e, g, big2, acc_s, acc_s2, acc_o);
        if (!kMayskip || pd) *pd = da;
    }
    acc_s += acc_s2;
}

// One group of `group` threads per pseudo-segment; a pseudo-segment is a
// contiguous run of elements that share one parameter.
template <int IO, int CT, int OP, bool VECT, bool WANT_O>
__global__ void __launch_bounds__(kThreads, 4) k_bwd_seg(BwdArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    constexpr bool kIo16 = IO == AB_BF16 || IO == AB_F16;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};

    const int G = a.group;
    const SegPos p = seg_pos<VEC>(a.cm, a.seg_len, a.nseg, a.nchunk, G);
    const int lane = p.lane;
    const bool valid = p.valid;
    const int64_t s = p.s, param = p.param;

    T acc_s = 0, acc_o = 0;
    if (valid) {
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
                            bwd_seg_loop<IO, CT, OP, WANT_O, PATH_PACKED, true>(px, pg, pd, lane, p.nv, G, e, g, big2, acc_s, acc_o);
                            done = true;
                        }
                    }
                    if (!done && vec_fast_ok<CT>(e, g)) {
                        bwd_seg_loop<IO, CT, OP, WANT_O, PATH_FAST, true>(px, pg, pd, lane, p.nv, G, e, g, big2, acc_s, acc_o);
                        done = true;
                    }
                }
            } else if constexpr (OP == OP_QDQ && CT != AB_F64) {
                if (pd && vec_fast_ok<CT>(e, g)) {
                    bwd_seg_loop<IO, CT, OP, WANT_O, PATH_FAST, false>(px, pg, pd, lane, p.nv, G, e, g, 0u, acc_s, acc_o);
                    done = true;
                }
            }
            if (!done) bwd_seg_loop<IO, CT, OP, WANT_O, PATH_GENERIC, false>(px, pg, pd, lane, p.nv, G, e, g, 0u, acc_s, acc_o);
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
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    constexpr int VEC = VECT ? 16 / (int)sizeof(E) : 1;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
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
};

template <int IO, int CT, int OP, bool WANT_O>
__global__ void __launch_bounds__(kThreads) k_bwd_gen(BwdGenArgs a) {
    using E = typename Elem<IO>::type;
    using A = Arith<CT>;
    using T = typename A::T;
    using C = Cvt<T, E>;
    const Grid<T> g{(T)a.qmin, (T)a.qmax, (T)a.zps, a.zps != 0.0, a.exact_edges};
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
inline BwdPlan plan_backward(const Canon &c, int io_dtype, bool ptr_aligned) { return plan_reduce(c, io_dtype, ptr_aligned); }

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
            k_fwd_seg<IO, CT, OP><<<(unsigned)sgrid, kThreads, 0, c.stream>>>(f);
            AB_LAUNCH_OK();
            return AB_OK;
        }
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
        a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
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
        a.exact_edges = exact_edges(CT, c.qmin, c.qmax);
        int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (grid > cap) grid = cap;
        if (c.go)
            k_bwd_gen<IO, CT, OP, true><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else
            k_bwd_gen<IO, CT, OP, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
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

    if (p.mode == BwdPlan::SEG) {
        const int gpc = kThreads / p.group;
        const int64_t grid = (p.nseg + gpc - 1) / gpc;
        if (grid > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        if (p.vect && c.go)
            k_bwd_seg<IO, CT, OP, true, true><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else if (p.vect)
            k_bwd_seg<IO, CT, OP, true, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else if (c.go)
            k_bwd_seg<IO, CT, OP, false, true><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
        else
            k_bwd_seg<IO, CT, OP, false, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(a);
    } else {
        const int v = p.vect ? 16 / dtype_size(IO) : 1;
        const int64_t gx = (a.row_len / v + kThreads - 1) / kThreads;
        if (gx > 2147483647LL) return fail(AB_ERR_UNSUPPORTED, "tensor too large for one launch");
        dim3 grid((unsigned)gx, (unsigned)p.row_tiles);
        if (p.vect && c.go)
            k_bwd_col<IO, CT, OP, true, true><<<grid, kThreads, 0, c.stream>>>(a);
        else if (p.vect)
            k_bwd_col<IO, CT, OP, true, false><<<grid, kThreads, 0, c.stream>>>(a);
        else if (c.go)
            k_bwd_col<IO, CT, OP, false, true><<<grid, kThreads, 0, c.stream>>>(a);
        else
            k_bwd_col<IO, CT, OP, false, false><<<grid, kThreads, 0, c.stream>>>(a);
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
            k_bwd_finish<CT, true><<<(unsigned)canon.nparam, kThreads, 0, c.stream>>>(f);
        } else {
            const int64_t grid = (canon.nparam * 32 + kThreads - 1) / kThreads;
            k_bwd_finish<CT, false><<<(unsigned)grid, kThreads, 0, c.stream>>>(f);
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
