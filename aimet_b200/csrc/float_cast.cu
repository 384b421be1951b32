// Floating-point fake-cast: simulate a narrow float format (fp16 / bf16 / fp8 variants / fp4 e2m1 /
// any exponent-mantissa split) on a wider tensor, with a per-tensor, per-channel or per-block scale.
// Follows quantization/float/quantizer.py of the reference (_float_quantize_dequantize :619-705):
//
//   xs  = x / scale                          (blockwise over the scale's shape)
//   xc  = clamp(xs, -max, max)
//   q   = fake_cast(xc)                      (two flavours, below)
//   out = q * scale
//
// fake_cast, flavour "cast": the reference converts to the torch dtype of the format and back
// (_cast_decast :704-705).  A clamped value converts by round-to-nearest-even onto the format's grid,
// subnormals included: with e = floor(log2 |xc|) taken from the exponent field (exact), the grid
// spacing is 2^(max(e, emin) - M) and q = rint(xc / spacing) * spacing.  Formats with an unsigned
// zero (the "fnuz" ones) return +0 for every zero result.
//
// fake_cast, flavour "ieee": formats without a torch dtype go through fake_cast_to_ieee_float
// (fp_quantization.py:157-214), whose per-element scale comes from floating-point logarithms
// evaluated in the tensor's dtype: floor(log2 |xc| + bias), clamped at 1, then
// 2^(that - M - bias).  The operations are repeated here one by one with the same intermediate
// rounding (in a 16-bit tensor dtype the rounded logarithm lands one binade too high for values close
// below a power of two; the reference's results are reproduced, not corrected).
//
// One 16-byte vector per thread and step, grid-stride; the pass is bound by HBM bandwidth (one read,
// one write per element).
#include <math.h>

#include "common.cuh"

namespace ab {
namespace {

struct CastArgs {
    const void *x;
    void *y;
    const float *scale;
    ChanMap cm;
    int64_t numel;
    int mantissa_bits, emin;   // cast flavour: exponent of the smallest normal number
    float maxval, bias;        // bias: the reference's 2^E - log2(max) + log2(2 - 2^-M) - 1 in the tensor dtype
    int ieee, inf_passthrough, unsigned_zero;
    // cast flavour, when 1.5 * 2^(exponent of maxval + 23 - M) is a finite float: the constants of
    // the per-element rounding constant (see cast_to_grid)
    int grid_magic;
    uint32_t emin_field, magic_add;
};

// x / s, correctly rounded, without the divide unit when the scale allows it (the same
// reciprocal-and-exact-remainder form as the affine kernels): r = RN(1 / s), q0 = RN(x r),
// rem = x - q0 s (exact in an fma), q = RN(q0 + rem r).
struct ScaleDiv {
    float s, r;
    bool fast;
};
__device__ __forceinline__ ScaleDiv make_scale_div(float s) {
    ScaleDiv d;
    d.s = s;
    d.r = __frcp_rn(s);
    const float as = fabsf(s);
    d.fast = as > 7.888609e-31f && as < 1.2676506e30f;  // 2^-100 .. 2^100
    return d;
}
__device__ __forceinline__ float div_by_scale(float x, const ScaleDiv &d) {
    if (!d.fast) return __fdiv_rn(x, d.s);
    const float q0 = __fmul_rn(x, d.r);
    float rem = __fmaf_rn(-q0, d.s, x);
    rem = fabsf(q0) < 1.2676506e30f ? rem : 0.0f;  // +-inf, NaN and absurd quotients keep q0
    return __fmaf_rn(rem, d.r, q0);
}

// A clamped value rounded to nearest even onto the format's grid, subnormals included.
__device__ __forceinline__ float cast_to_grid(float xc, const CastArgs &a) {
    float q;
    if (a.grid_magic) {
        // With e = max(exponent of xc, emin) the grid spacing is 2^(e - M); adding and subtracting
        // C = 1.5 * 2^(e + 23 - M), whose last place is that spacing, rounds xc to it (to nearest
        // even, |xc| < 2^(e + 1) being far below C / 2).  C's bits are xc's exponent field (at least
        // emin's) plus a constant.  Zero and float subnormals read as emin; NaN stays NaN.
        uint32_t ef = __float_as_uint(xc) & 0x7f800000u;
        ef = ef < a.emin_field ? a.emin_field : ef;
        const float c = __uint_as_float(ef + a.magic_add);
        q = __fsub_rn(__fadd_rn(xc, c), c);
        q = copysignf(q, xc);  // a value that rounds to zero keeps its sign, as a conversion does
    } else if (xc == 0.0f || xc != xc) {
        q = xc;
    } else {
        int e = ilogbf(xc);  // exact floor(log2 |xc|), subnormal inputs included
        if (e < a.emin) e = a.emin;
        const float spacing = ldexpf(1.0f, e - a.mantissa_bits);
        q = op_mul(rintf(op_div(xc, spacing)), spacing);
    }
    if (a.unsigned_zero && q == 0.0f) q = 0.0f;  // -0 -> +0
    return q;
}

template <int CT> __device__ __forceinline__ float fake_cast_one(float x, const ScaleDiv &sd, const CastArgs &a) {
    using A = Arith<CT>;
    const float s = sd.s;
    const float xs = A::rnd(div_by_scale(x, sd));
    const float xc = clamp_nan(xs, -a.maxval, a.maxval);
    float q;
    if (!a.ieee) {
        q = cast_to_grid(xc, a);
    } else {
        const float l = A::rnd(log2f(fabsf(xc)));
        float ls = floorf(A::rnd(op_add(l, a.bias)));
        ls = ls < 1.0f ? 1.0f : ls;  // torch.clamp(min=1): NaN stays NaN
        const float ex = A::rnd(op_sub(A::rnd(op_sub(ls, (float)a.mantissa_bits)), a.bias));
        const float sc = A::rnd(exp2f(ex));
        q = A::rnd(op_mul(rintf(A::rnd(op_div(xc, sc))), sc));
        // (the reference passes infinities through for formats that have them, but looks at the
        // clamped value, which never is one)
        if (a.inf_passthrough && isinf(xc)) q = xc;
    }
    return A::rnd(op_mul(q, s));
}

// Two elements under one scale: the roundings to a 16-bit tensor dtype are packed conversions
// (one instruction for both; the scalar conversion runs at a quarter of the rate).
template <int CT>
__device__ __forceinline__ void fake_cast_two(float x0, float x1, const ScaleDiv &sd, const CastArgs &a, float &y0,
                                              float &y1) {
    using A = Arith<CT>;
    if (a.ieee) {
        y0 = fake_cast_one<CT>(x0, sd, a);
        y1 = fake_cast_one<CT>(x1, sd, a);
        return;
    }
    float s0 = div_by_scale(x0, sd), s1 = div_by_scale(x1, sd);
    A::rnd2(s0, s1);
    const float c0 = clamp_nan(s0, -a.maxval, a.maxval), c1 = clamp_nan(s1, -a.maxval, a.maxval);
    float q0 = cast_to_grid(c0, a), q1 = cast_to_grid(c1, a);
    q0 = op_mul(q0, sd.s);
    q1 = op_mul(q1, sd.s);
    A::rnd2(q0, q1);
    y0 = q0;
    y1 = q1;
}

// IN: dtype of x; IO: dtype of y (a scale with dimensions promotes a 16-bit input to a float32
// result: the widening is done on the fly, the values are those of a converted copy).  One 16-byte
// vector of the input per thread and step.
template <int IN, int IO, int CT> __global__ void __launch_bounds__(kThreads) k_float_cast(CastArgs a) {
    pdl_prologue();
    using EI = typename Elem<IN>::type;
    using EO = typename Elem<IO>::type;
    constexpr int VEC = 16 / (int)sizeof(EI);
    constexpr int OUTV = VEC * (int)sizeof(EO) / 16;  // output vectors per input vector
    constexpr int PER = VEC / OUTV;                    // elements per output vector
    const EI *__restrict__ xp = static_cast<const EI *>(a.x);
    EO *__restrict__ yp = static_cast<EO *>(a.y);
    const int64_t nvec = a.numel / VEC;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    auto one_vector = [&](const Vec16<EI> &in, int64_t v) {
        Vec16<EO> out[OUTV];
        const int64_t e0 = v * VEC;
        const int64_t p0 = a.cm.of(e0), p1 = a.cm.of(e0 + VEC - 1);
        const ScaleDiv d0 = make_scale_div(a.scale[p0]);
        if (p0 == p1) {
#pragma unroll
            for (int i = 0; i < VEC; i += 2) {
                float y0, y1;
                fake_cast_two<CT>(to_f32(in.v[i]), to_f32(in.v[i + 1]), d0, a, y0, y1);
                out[i / PER].v[i % PER] = Cvt<float, EO>::store(y0);
                out[(i + 1) / PER].v[(i + 1) % PER] = Cvt<float, EO>::store(y1);
            }
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                const ScaleDiv d = make_scale_div(a.scale[a.cm.of(e0 + i)]);
                out[i / PER].v[i % PER] = Cvt<float, EO>::store(fake_cast_one<CT>(to_f32(in.v[i]), d, a));
            }
        }
#pragma unroll
        for (int o = 0; o < OUTV; ++o) reinterpret_cast<Vec16<EO> *>(yp)[v * OUTV + o] = out[o];
    };
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride)
        one_vector(reinterpret_cast<const Vec16<EI> *>(xp)[v], v);
    // elements beyond the last whole vector
    const int64_t t = nvec * VEC + (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (t < a.numel)
        yp[t] = Cvt<float, EO>::store(fake_cast_one<CT>(to_f32(xp[t]), make_scale_div(a.scale[a.cm.of(t)]), a));
}

template <int IN, int IO, int CT> int launch_cast(const CastArgs &a, cudaStream_t stream) {
    const int vec = 16 / dtype_size(IN);
    int64_t grid = (a.numel / vec + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    launch_pdl(k_float_cast<IN, IO, CT>, (unsigned)grid, kThreads, 0, stream, a);
    AB_LAUNCH_OK();
    return AB_OK;
}

}  // namespace
}  // namespace ab

extern "C" int aimet_b200_float_fake_cast(const void *x, void *y, const float *scale, const ab_layout *layout,
                                          int in_dtype, int io_dtype, int compute_dtype, int32_t exponent_bits,
                                          int32_t mantissa_bits, int32_t exponent_bias, double maxval, int32_t flags,
                                          void *stream) {
    using namespace ab;
    Canon canon;
    int rc = canonicalize(layout, &canon);
    if (rc != AB_OK) return rc;
    if (canon.numel == 0) return AB_OK;
    if (!canon.oci)
        return fail(AB_ERR_UNSUPPORTED, "the float fake-cast needs a layout that reduces to (outer, channel, inner)");
    if (!x || !y || !scale) return fail(AB_ERR_INVALID, "x, y and scale must not be NULL");
    if (exponent_bits < 1 || exponent_bits > 8 || mantissa_bits < 0 || mantissa_bits > 23)
        return fail(AB_ERR_INVALID, "exponent_bits must be in [1, 8] and mantissa_bits in [0, 23]");
    if (!aligned16(x) || !aligned16(y)) return fail(AB_ERR_INVALID, "x and y must be 16-byte aligned");
    if (!(maxval > 0)) return fail(AB_ERR_INVALID, "maxval must be positive");
    if (flags & ~7) return fail(AB_ERR_INVALID, "unknown flags %d", (int)flags);
    CastArgs a;
    a.x = x;
    a.y = y;
    a.scale = scale;
    a.cm = make_chan_map(canon);
    a.numel = canon.numel;
    a.mantissa_bits = mantissa_bits;
    a.emin = 1 - exponent_bias;
    a.maxval = (float)maxval;
    a.ieee = (flags & 1) ? 1 : 0;
    a.inf_passthrough = (flags & 2) ? 1 : 0;
    a.unsigned_zero = (flags & 4) ? 1 : 0;
    {
        // exponent of the largest value a clamped input can have, and whether the rounding constant
        // built on it stays finite
        int emax = 0;
        frexp(maxval, &emax);  // maxval = f * 2^emax, f in [0.5, 1): floor(log2 maxval) = emax - 1
        emax -= 1;
        a.grid_magic = (!a.ieee && mantissa_bits <= 20 && emax + 23 - mantissa_bits <= 126 && a.emin >= -126) ? 1 : 0;
        a.emin_field = (uint32_t)(a.emin + 127) << 23;
        a.magic_add = ((uint32_t)(23 - mantissa_bits) << 23) + 0x00400000u;
    }
    // the reference's bias: evaluated in double, then used in the tensor's dtype
    const double bias = pow(2.0, exponent_bits) - log2(maxval) + log2(2.0 - pow(2.0, -mantissa_bits)) - 1.0;
    a.bias = (float)bias;
    if (compute_dtype == AB_BF16) a.bias = __bfloat162float(__float2bfloat16_rn(a.bias));
    if (compute_dtype == AB_F16) a.bias = __half2float(__float2half_rn(a.bias));
    if (compute_dtype == AB_BF16) a.maxval = __bfloat162float(__float2bfloat16_rn(a.maxval));
    if (compute_dtype == AB_F16) a.maxval = __half2float(__float2half_rn(a.maxval));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define AB_CAST(INV, IOV, CTV) \
    if (in_dtype == INV && io_dtype == IOV && compute_dtype == CTV) return launch_cast<INV, IOV, CTV>(a, st);
    AB_CAST(AB_F32, AB_F32, AB_F32)
    AB_CAST(AB_BF16, AB_BF16, AB_BF16)
    AB_CAST(AB_BF16, AB_BF16, AB_F32)
    AB_CAST(AB_F16, AB_F16, AB_F16)
    AB_CAST(AB_F16, AB_F16, AB_F32)
    AB_CAST(AB_BF16, AB_F32, AB_F32)
    AB_CAST(AB_F16, AB_F32, AB_F32)
#undef AB_CAST
    return fail(AB_ERR_UNSUPPORTED, "float fake-cast: in_dtype %d, io_dtype %d with compute_dtype %d is not supported",
                in_dtype, io_dtype, compute_dtype);
}
