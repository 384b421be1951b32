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
};

template <int CT> __device__ __forceinline__ float fake_cast_one(float x, float s, const CastArgs &a) {
    using A = Arith<CT>;
    const float xs = A::rnd(op_div(x, s));
    const float xc = clamp_nan(xs, -a.maxval, a.maxval);
    float q;
    if (!a.ieee) {
        if (xc == 0.0f || xc != xc) {
            q = xc;
        } else {
            int e = ilogbf(xc);  // exact floor(log2 |xc|), subnormal inputs included
            if (e < a.emin) e = a.emin;
            const float spacing = ldexpf(1.0f, e - a.mantissa_bits);
            q = op_mul(rintf(op_div(xc, spacing)), spacing);
        }
        if (a.unsigned_zero && q == 0.0f) q = 0.0f;  // -0 -> +0
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

template <int IO, int CT> __global__ void __launch_bounds__(kThreads) k_float_cast(CastArgs a) {
    pdl_prologue();
    using E = typename Elem<IO>::type;
    constexpr int VEC = 16 / (int)sizeof(E);
    const E *__restrict__ xp = static_cast<const E *>(a.x);
    E *__restrict__ yp = static_cast<E *>(a.y);
    const int64_t nvec = a.numel / VEC;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t v = (int64_t)blockIdx.x * kThreads + threadIdx.x; v < nvec; v += stride) {
        const Vec16<E> in = reinterpret_cast<const Vec16<E> *>(xp)[v];
        Vec16<E> out;
        const int64_t e0 = v * VEC;
        const int64_t p0 = a.cm.of(e0), p1 = a.cm.of(e0 + VEC - 1);
        const float s0 = a.scale[p0];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float s = p0 == p1 ? s0 : a.scale[a.cm.of(e0 + i)];
            out.v[i] = Cvt<float, E>::store(fake_cast_one<CT>(to_f32(in.v[i]), s, a));
        }
        reinterpret_cast<Vec16<E> *>(yp)[v] = out;
    }
    // elements beyond the last whole vector
    const int64_t t = nvec * VEC + (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (t < a.numel) yp[t] = Cvt<float, E>::store(fake_cast_one<CT>(to_f32(xp[t]), a.scale[a.cm.of(t)], a));
}

template <int IO, int CT> int launch_cast(const CastArgs &a, cudaStream_t stream) {
    const int vec = 16 / dtype_size(IO);
    int64_t grid = (a.numel / vec + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    launch_pdl(k_float_cast<IO, CT>, (unsigned)grid, kThreads, 0, stream, a);
    AB_LAUNCH_OK();
    return AB_OK;
}

}  // namespace
}  // namespace ab

extern "C" int aimet_b200_float_fake_cast(const void *x, void *y, const float *scale, const ab_layout *layout,
                                          int io_dtype, int compute_dtype, int32_t exponent_bits,
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
    // the reference's bias: evaluated in double, then used in the tensor's dtype
    const double bias = pow(2.0, exponent_bits) - log2(maxval) + log2(2.0 - pow(2.0, -mantissa_bits)) - 1.0;
    a.bias = (float)bias;
    if (compute_dtype == AB_BF16) a.bias = __bfloat162float(__float2bfloat16_rn(a.bias));
    if (compute_dtype == AB_F16) a.bias = __half2float(__float2half_rn(a.bias));
    if (compute_dtype == AB_BF16) a.maxval = __bfloat162float(__float2bfloat16_rn(a.maxval));
    if (compute_dtype == AB_F16) a.maxval = __half2float(__float2half_rn(a.maxval));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define AB_CAST(IOV, CTV) \
    if (io_dtype == IOV && compute_dtype == CTV) return launch_cast<IOV, CTV>(a, st);
    AB_CAST(AB_F32, AB_F32)
    AB_CAST(AB_BF16, AB_BF16)
    AB_CAST(AB_BF16, AB_F32)
    AB_CAST(AB_F16, AB_F16)
    AB_CAST(AB_F16, AB_F32)
#undef AB_CAST
    return fail(AB_ERR_UNSUPPORTED, "float fake-cast: io_dtype %d with compute_dtype %d is not supported", io_dtype,
                compute_dtype);
}
