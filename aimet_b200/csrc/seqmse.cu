// SeqMSE reconstruction loss of a Linear layer for all candidates in one launch.
//
//   out[c][n] = sum_m f( x[m,:] . w[n,:] ,  xq[m,:] . wq[c][n,:] )
//
// (SequentialMse._compute_linear_loss, seq_mse.py:403-454 of the reference, which runs two
// matmuls and three elementwise passes per candidate.)  Here the contraction runs on the 5th
// generation tensor cores: operands are staged in shared memory by TMA (128-byte swizzle),
// tcgen05.mma accumulates in tensor memory, and the epilogue reads both accumulators back with
// tcgen05.ld, forms f() and sums over the tokens without the products ever touching HBM.
//
// Orientation: the weights are the M operand (128 output channels per tile = 128 TMEM lanes), the
// tokens the N operand (256 per tile = 256 TMEM columns), so one epilogue thread owns one output
// channel and its sum over tokens is thread-local.  TMEM holds x.w^T of the tile in columns
// [0,256) for the whole unit and the product of the current candidate in columns [256,512).
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 TMEM allocation + MMA issue, warps 2-5
// epilogue (one per TMEM lane quadrant).  Every wait is bounded: on a time-out the kernel raises
// the status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace ab {
namespace {

constexpr int BM = 128;      // output channels per tile (MMA M, TMEM lanes)
constexpr int BN = 256;      // tokens per tile (MMA N, TMEM columns per accumulator)
constexpr int BK = 64;       // K elements per pipeline stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;   // K elements per tcgen05.mma (16-bit operands)
constexpr int STAGES = 4;
constexpr int kSeqThreads = 192;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 512;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;  // 2 s per wait

// status codes written by the kernel
enum { ST_OK = 0, ST_TIMEOUT_PRODUCER = 1, ST_TIMEOUT_MMA = 2, ST_TIMEOUT_EPILOGUE = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the abort flag was raised or the time-out expired (in which case
// it raises the flag and records `code`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > kWaitTimeoutNs) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused for swizzled K-major
// layouts (encoded as 1), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffff) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct SeqArgs {
    int64_t M, N, K;
    int num_cand;
    int n_ct, n_tt;   // channel tiles, token tiles
    int loss_kind;    // 0 squared, 1 absolute, 2 squared + square of the second product
    int lowp;         // 0 none, 1 round like bfloat16, 2 round like float16
    uint32_t idesc;
    float *partial;   // [n_tt][num_cand][N][nvals]
    int *status;
};

__device__ __forceinline__ float round_lowp(float v, int lowp) {
    if (lowp == 1) return __bfloat162float(__float2bfloat16_rn(v));
    if (lowp == 2) return __half2float(__float2half_rn(v));
    return v;
}

__global__ void __launch_bounds__(kSeqThreads, 1)
k_seqmse(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wq,
         const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xq, SeqArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (size_t)STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S] accumulator full, [2S+1] accumulator empty
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = smem_u32(bars + STAGES);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES);
    const uint32_t bar_acc_empty = smem_u32(bars + 2 * STAGES + 1);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // contiguous range of (channel tile, token tile) units for this CTA
    const int64_t units = (int64_t)a.n_ct * a.n_tt;
    const int64_t u0 = units * blockIdx.x / gridDim.x;
    const int64_t u1 = units * (blockIdx.x + 1) / gridDim.x;
    const int kblocks = (int)((a.K + BK - 1) / BK);
    const int passes = a.num_cand + 1;  // pass 0 = x.w^T, pass g = candidate g-1

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t u = u0; u < u1 && ok; ++u) {
                const int ct = (int)(u / a.n_tt), tt = (int)(u % a.n_tt);
                for (int g = 0; g < passes && ok; ++g) {
                    const CUtensorMap *ma = g == 0 ? &tm_w : &tm_wq;
                    const CUtensorMap *mb = g == 0 ? &tm_x : &tm_xq;
                    const int row_a = g == 0 ? ct * BM : (int)((int64_t)(g - 1) * a.N) + ct * BM;
                    for (int kb = 0; kb < kblocks; ++kb) {
                        ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.status, ST_TIMEOUT_PRODUCER);
                        if (!ok) break;
                        const uint32_t sa = base + stage * STAGE_BYTES;
                        mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
                        tma_load_2d(sa, ma, kb * BK, row_a, bar_full + 8 * stage);
                        tma_load_2d(sa + A_BYTES, mb, kb * BK, tt * BN, bar_full + 8 * stage);
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int64_t event = 0;  // index of the next accumulator hand-over to the epilogue
            bool ok = true;
            for (int64_t u = u0; u < u1 && ok; ++u) {
                for (int g = 0; g < passes && ok; ++g) {
                    // do not overwrite an accumulator the epilogue may still be reading:
                    //   pass 0 overwrites x.w^T, last read by the previous unit's final event;
                    //   pass g >= 2 overwrites the candidate accumulator read by event - 1
                    if ((g == 0 && event > 0) || g >= 2) {
                        ok = mbar_wait(bar_acc_empty, (uint32_t)((event - 1) & 1), abort_flag, a.status, ST_TIMEOUT_MMA);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (g == 0 ? 0 : BN);
                    for (int kb = 0; kb < kblocks; ++kb) {
                        ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, a.status, ST_TIMEOUT_MMA);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t sa = base + stage * STAGE_BYTES;
                        const uint64_t da = make_smem_desc(sa);
                        const uint64_t db = make_smem_desc(sa + A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // advance 32 bytes (16 elements) inside the swizzled 128-byte row
                            umma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), a.idesc,
                                     (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        umma_commit(bar_empty + 8 * stage);  // frees the stage once these MMAs have read it
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    if (ok && g >= 1) {
                        umma_commit(bar_acc_full);
                        ++event;
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5, one TMEM lane quadrant each ----------------
        const int quad = warp & 3;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const int nvals = a.loss_kind == 2 ? 2 : 1;
        int64_t event = 0;
        bool ok = true;
        for (int64_t u = u0; u < u1 && ok; ++u) {
            const int ct = (int)(u / a.n_tt), tt = (int)(u % a.n_tt);
            const int64_t n = (int64_t)ct * BM + quad * 32 + lane;
            for (int g = 1; g < passes && ok; ++g, ++event) {
                ok = mbar_wait(bar_acc_full, (uint32_t)(event & 1), abort_flag, a.status, ST_TIMEOUT_EPILOGUE);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                float s0 = 0.f, s1 = 0.f;
#pragma unroll 1
                for (int chunk = 0; chunk < BN / 32; ++chunk) {
                    uint32_t rx[32], ry[32];
                    tmem_ld32(tmem_base + lane_base + chunk * 32, rx);
                    tmem_ld32(tmem_base + lane_base + BN + chunk * 32, ry);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float xw = __uint_as_float(rx[j]), y = __uint_as_float(ry[j]);
                        if (a.lowp) {
                            xw = round_lowp(xw, a.lowp);
                            y = round_lowp(y, a.lowp);
                        }
                        const float d = xw - y;
                        float f = a.loss_kind == 1 ? fabsf(d) : d * d;
                        if (a.lowp) f = round_lowp(f, a.lowp);
                        s0 += f;
                        if (a.loss_kind == 2) s1 += a.lowp ? round_lowp(y * y, a.lowp) : y * y;
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_acc_empty);
                if (n < a.N) {
                    float *p = a.partial + (((int64_t)tt * a.num_cand + (g - 1)) * a.N + n) * nvals;
                    p[0] = s0;
                    if (nvals == 2) p[1] = s1;
                }
            }
        }
    }

    // teardown: every role has left its loop (normally or through the abort flag)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// out[c][n][v] = sum over token tiles, in tile order (deterministic)
__global__ void k_seqmse_reduce(const float *partial, float *out, int n_tt, int64_t per_tile) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_tile) return;
    float s = 0.f;
    for (int t = 0; t < n_tt; ++t) s += partial[(int64_t)t * per_tile + i];
    out[i] = s;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []() {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// row-major [rows][K] 16-bit matrix, boxes of BK columns x box_rows rows, 128-byte swizzle,
// out-of-range elements read as zero
int make_map(CUtensorMap *map, const void *ptr, int64_t rows, int64_t K, int box_rows, int io_dtype) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(AB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = io_dtype == AB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return AB_OK;
}

}  // namespace
}  // namespace ab

extern "C" int64_t aimet_b200_seqmse_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t num_cand) {
    (void)K;
    if (M <= 0 || N <= 0 || num_cand <= 0) return ab::fail(AB_ERR_INVALID, "M, N and num_cand must be positive");
    const int64_t n_tt = (M + ab::BN - 1) / ab::BN;
    return n_tt * num_cand * N * 2 * (int64_t)sizeof(float);
}

extern "C" int aimet_b200_seqmse_linear_loss(const void *x, const void *xq, const void *w, const void *wq, int64_t M,
                                             int64_t N, int64_t K, int32_t num_cand, int io_dtype, int loss_kind,
                                             int lowp_epilogue, float *out, int32_t *status, void *scratch,
                                             int64_t scratch_bytes, void *stream) {
    using namespace ab;
    if (io_dtype != AB_BF16 && io_dtype != AB_F16)
        return fail(AB_ERR_UNSUPPORTED, "seqmse_linear_loss takes bfloat16 or float16 operands");
    if (M <= 0 || N <= 0 || K <= 0 || num_cand <= 0) return fail(AB_ERR_INVALID, "M, N, K and num_cand must be positive");
    if (K % 8 != 0) return fail(AB_ERR_UNSUPPORTED, "K must be a multiple of 8 (16-byte rows for TMA), got %lld", (long long)K);
    if (loss_kind < 0 || loss_kind > 2) return fail(AB_ERR_INVALID, "loss_kind must be 0, 1 or 2");
    if (!x || !xq || !w || !wq || !out || !status) return fail(AB_ERR_INVALID, "NULL pointer argument");
    for (const void *p : {x, xq, w, wq})
        if (!aligned16(p)) return fail(AB_ERR_INVALID, "operands must be 16-byte aligned");
    if ((int64_t)num_cand * N >= ((int64_t)1 << 31) || M >= ((int64_t)1 << 31))
        return fail(AB_ERR_UNSUPPORTED, "row counts must fit 31 bits");
    const int64_t need = aimet_b200_seqmse_scratch_bytes(M, N, K, num_cand);
    if (!scratch || scratch_bytes < need)
        return fail(AB_ERR_SCRATCH, "seqmse needs %lld bytes of scratch, got %lld", (long long)need, (long long)scratch_bytes);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CUtensorMap tm_w, tm_wq, tm_x, tm_xq;
    int rc;
    if ((rc = make_map(&tm_w, w, N, K, BM, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_wq, wq, (int64_t)num_cand * N, K, BM, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_x, x, M, K, BN, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_xq, xq, M, K, BN, io_dtype)) != AB_OK) return rc;

    static std::once_flag attr_once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once, []() {
        attr_err = cudaFuncSetAttribute(k_seqmse, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    });
    if (attr_err != cudaSuccess)
        return fail(AB_ERR_CUDA, "cannot reserve %zu bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(attr_err));

    SeqArgs a;
    a.M = M;
    a.N = N;
    a.K = K;
    a.num_cand = num_cand;
    a.n_ct = (int)((N + BM - 1) / BM);
    a.n_tt = (int)((M + BN - 1) / BN);
    a.loss_kind = loss_kind;
    a.lowp = lowp_epilogue ? (io_dtype == AB_BF16 ? 1 : 2) : 0;
    const uint32_t fmt = io_dtype == AB_BF16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    a.partial = static_cast<float *>(scratch);
    a.status = status;

    AB_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
    const int64_t units = (int64_t)a.n_ct * a.n_tt;
    int grid = sm_count();
    if (units < grid) grid = (int)units;
    k_seqmse<<<grid, kSeqThreads, SMEM_BYTES, st>>>(tm_w, tm_wq, tm_x, tm_xq, a);
    AB_LAUNCH_OK();
    const int nvals = loss_kind == 2 ? 2 : 1;
    const int64_t per_tile = (int64_t)num_cand * N * nvals;
    k_seqmse_reduce<<<(unsigned)((per_tile + 255) / 256), 256, 0, st>>>(a.partial, out, a.n_tt, per_tile);
    AB_LAUNCH_OK();
    return AB_OK;
}
