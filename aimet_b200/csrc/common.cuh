// Shared host/device helpers for the aimet_b200 kernels: error reporting,
// layout canonicalisation, element-type traits and the rounding-faithful
// arithmetic the affine kernels are written in.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/aimet_b200.h"

namespace ab {

// ---------------------------------------------------------------------------
// errors (thread-local message, C-ABI functions return the code)
// ---------------------------------------------------------------------------
int fail(int code, const char *fmt, ...);
void count_launch();  // bumps the process-wide kernel-launch counter

#define AB_CUDA_OK(expr)                                                                        \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess)                                                                  \
            return ::ab::fail(AB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                              __FILE__, __LINE__);                                              \
    } while (0)

#define AB_LAUNCH_OK()                                                                          \
    do {                                                                                        \
        ::ab::count_launch();                                                                   \
        cudaError_t _e = cudaPeekAtLastError();                                                 \
        if (_e != cudaSuccess)                                                                  \
            return ::ab::fail(AB_ERR_CUDA, "kernel launch failed: %s (%s:%d)",                  \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                      \
    } while (0)

// ---------------------------------------------------------------------------
// Canonical layout.  Size-1 dims are dropped and neighbouring dims merged
// whenever the parameter index stays a function of the merged coordinate.
// Most encodings end up as (O, C, I): element e uses parameter (e / I) % C.
//   per-tensor            O=1 C=1      I=numel
//   per-channel, axis a   O=prod(<a)  C=size[a]  I=prod(>a)
//   blockwise, last dim   O=1 C=numel/B I=B
// Anything else (e.g. blocks along two dims) keeps the general form.
// ---------------------------------------------------------------------------
struct Canon {
    bool oci;      // (O, C, I) form
    int64_t numel;
    int64_t nparam;  // number of (scale, offset) pairs
    int64_t O, C, I;
    int nd;  // general form, collapsed
    int64_t size[AB_MAX_DIMS];
    int64_t block[AB_MAX_DIMS];
    int64_t pstride[AB_MAX_DIMS];  // stride of dim k in the parameter array
};

int canonicalize(const ab_layout *layout, Canon *out);

inline int dtype_size(int dt) {
    switch (dt) {
        case AB_F32: return 4;
        case AB_F16: return 2;
        case AB_BF16: return 2;
        case AB_F64: return 8;
    }
    return 0;
}

int sm_count();

// Programmatic dependent launch: a kernel launched through launch_pdl may become resident while
// its predecessor in the stream is still draining; it must execute pdl_prologue() before it
// touches global memory (the wait returns once the predecessor has completed and its writes are
// visible).  The launch latency of back-to-back kernels disappears behind the predecessor's tail.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Opt a kernel in to `bytes` of dynamic shared memory (needed above 48 KB), once per device.
template <auto kernel> int opt_in_smem(size_t bytes) {
    static std::mutex mu;
    static uint64_t done = 0;
    int dev = 0;
    AB_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && ((done >> dev) & 1)) return AB_OK;
    AB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (dev < 64) done |= 1ull << dev;
    return AB_OK;
}

// ---------------------------------------------------------------------------
// element types at the boundary
// ---------------------------------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<AB_F32> { using type = float; };
template <> struct Elem<AB_F64> { using type = double; };
template <> struct Elem<AB_F16> { using type = __half; };
template <> struct Elem<AB_BF16> { using type = __nv_bfloat16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ double to_f64(double v) { return v; }

// ---------------------------------------------------------------------------
// Arithmetic in the reference's "internal dtype".  T is the register type;
// rnd() re-rounds to the internal dtype after each aten-level operation, which
// is how PyTorch evaluates elementwise ops on half-precision tensors (compute
// in float, store in the tensor dtype).  Explicit round-to-nearest intrinsics
// keep the compiler from contracting mul+add into an fma.
// ---------------------------------------------------------------------------
template <int CT> struct Arith;

// rnd2() rounds two values at once: the packed float->16-bit conversion is one
// instruction on the ALU pipe, whereas the scalar conversion goes through the
// quarter-rate conversion unit.
template <> struct Arith<AB_F32> {
    using T = float;
    static __device__ __forceinline__ T rnd(T v) { return v; }
    static __device__ __forceinline__ void rnd2(T &, T &) {}
};
template <> struct Arith<AB_BF16> {
    using T = float;
    static __device__ __forceinline__ T rnd(T v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ void rnd2(T &a, T &b) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
        const uint32_t w = *reinterpret_cast<const uint32_t *>(&p);
        a = __uint_as_float(w << 16);
        b = __uint_as_float(w & 0xffff0000u);
    }
};
template <> struct Arith<AB_F16> {
    using T = float;
    static __device__ __forceinline__ T rnd(T v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ void rnd2(T &a, T &b) {
        const float2 f = __half22float2(__floats2half2_rn(a, b));
        a = f.x;
        b = f.y;
    }
};
template <> struct Arith<AB_F64> {
    using T = double;
    static __device__ __forceinline__ T rnd(T v) { return v; }
    static __device__ __forceinline__ void rnd2(T &, T &) {}
};

__device__ __forceinline__ float op_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float op_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float op_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float op_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float op_rint(float a) { return rintf(a); }
__device__ __forceinline__ double op_add(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double op_sub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ double op_mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double op_div(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ double op_rint(double a) { return rint(a); }

// torch.clamp propagates NaN; fminf/fmaxf would swallow it.
template <typename T> __device__ __forceinline__ T clamp_nan(T v, T lo, T hi) {
    T r = v < lo ? lo : v;
    return r > hi ? hi : r;
}

// conversions between the boundary element type and the register type
template <typename T, typename E> struct Cvt;
template <> struct Cvt<float, float> {
    static __device__ __forceinline__ float load(float v) { return v; }
    static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Cvt<float, __half> {
    static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<float, __nv_bfloat16> {
    static __device__ __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<double, float> {
    static __device__ __forceinline__ double load(float v) { return (double)v; }
    static __device__ __forceinline__ float store(double v) { return __double2float_rn(v); }
};
template <> struct Cvt<double, double> {
    static __device__ __forceinline__ double load(double v) { return v; }
    static __device__ __forceinline__ double store(double v) { return v; }
};

// 16-byte vector of boundary elements
template <typename E> struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(E);
    E v[N];
};

// whole-vector conversions between a 16-byte vector and register values
template <typename T, typename E> struct VecCvt {
    static constexpr int N = 16 / sizeof(E);
    static __device__ __forceinline__ void unpack(const Vec16<E> &v, T (&out)[N]) {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = Cvt<T, E>::load(v.v[i]);
    }
    static __device__ __forceinline__ void pack(const T (&in)[N], Vec16<E> &v) {
#pragma unroll
        for (int i = 0; i < N; ++i) v.v[i] = Cvt<T, E>::store(in[i]);
    }
};
template <> struct VecCvt<float, __nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const Vec16<__nv_bfloat16> &v, float (&out)[8]) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void pack(const float (&in)[8], Vec16<__nv_bfloat16> &v) {
        __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    }
};
template <> struct VecCvt<float, __half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const Vec16<__half> &v, float (&out)[8]) {
        const __half2 *p = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(p[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void pack(const float (&in)[8], Vec16<__half> &v) {
        __half2 *p = reinterpret_cast<__half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    }
};

// parameter (scale / offset / grad) access: float32 or float64 arrays
struct ParamPtr {
    const void *p;
    int f64;
    __device__ __forceinline__ double get(int64_t i) const {
        return f64 ? static_cast<const double *>(p)[i] : (double)static_cast<const float *>(p)[i];
    }
};
struct ParamOut {
    void *p;
    int f64;
    __device__ __forceinline__ void put(int64_t i, double v) const {
        if (f64)
            static_cast<double *>(p)[i] = v;
        else
            static_cast<float *>(p)[i] = (float)v;
    }
};

// element index -> parameter index for the (O, C, I) form
struct ChanMap {
    int64_t I, C;
    int shift;     // log2(I) when I is a power of two, else -1
    int wrap;      // O > 1: parameter index wraps modulo C
    int narrow;    // numel < 2^31: 32-bit arithmetic is enough
    __device__ __forceinline__ int64_t of(int64_t e) const {
        if (C == 1) return 0;
        if (narrow) {
            uint32_t s = shift >= 0 ? ((uint32_t)e >> shift) : ((uint32_t)e / (uint32_t)I);
            return wrap ? (int64_t)(s % (uint32_t)C) : (int64_t)s;
        }
        int64_t s = shift >= 0 ? (e >> shift) : (e / I);
        return wrap ? s % C : s;
    }
};

ChanMap make_chan_map(const Canon &c);

// general form: element index -> parameter index by coordinate decomposition
struct GenMap {
    int nd;
    int64_t size[AB_MAX_DIMS];
    int64_t block[AB_MAX_DIMS];
    int64_t pstride[AB_MAX_DIMS];
    __device__ __forceinline__ int64_t of(int64_t e) const {
        int64_t p = 0;
        for (int k = nd - 1; k >= 0; --k) {
            int64_t c = e % size[k];
            e /= size[k];
            p += (c / block[k]) * pstride[k];
        }
        return p;
    }
};

GenMap make_gen_map(const Canon &c);

// ---------------------------------------------------------------------------
// How a reduction over everything that shares a parameter is cut into CTAs.
// Used by the backward pass (scale / offset gradients) and by the min/max
// statistics.  SEG: a group of threads per contiguous run ("pseudo-segment")
// of elements sharing a parameter; COL: short runs under a large outer dim are
// walked column-wise; GEN: no (O, C, I) form.
// ---------------------------------------------------------------------------
constexpr int kThreads = 256;
constexpr int kSegVecPerThread = 8;  // 16-byte vectors per thread in one chunk

struct ReducePlan {
    enum Mode { SEG, COL, GEN } mode;
    bool vect;
    int64_t seg_len, nseg, nchunk;
    int group, direct;
    int64_t rows_per_tile, row_tiles;
    int64_t npartial;
    // second stage: out[c] = reduce_{a<na} reduce_{b<nb} partial[a*sa + c*sc + b]
    int64_t na, sa, sc, nb;
};

// Depends only on the layout and the element size (plus whether the pointers
// allow 16-byte accesses), so a scratch-size query and the launch agree.
// ctas_per_sm > 0: a single long run is cut into a whole number of waves of that many CTAs per SM
ReducePlan plan_reduce(const Canon &c, int io_dtype, bool ptr_aligned, int chunk_mult = 1, int ctas_per_sm = 0);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// deterministic warp / block sums in double
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace ab
