// SeqMSE reconstruction loss of a Linear layer for all candidates (and all input-channel blocks)
// in one launch.
//
//   out[c][n][b] = sum_m f( x[m,Kb] . w[n,Kb] ,  xq[m,Kb] . wq[c][n,Kb] )     Kb = columns of block b
//
// (SequentialMse._compute_linear_loss, seq_mse.py:403-454 of the reference, which runs two batched
// matmuls and three elementwise passes per candidate.)  Here the contraction runs on the 5th
// generation tensor cores: operands are staged in shared memory by TMA (128-byte swizzle),
// tcgen05.mma accumulates in tensor memory, and the epilogue reads the accumulators back with
// tcgen05.ld, forms f() and sums over the tokens without the products ever touching HBM.
//
// Orientation: the weights are the M operand (128 output channels per tile = 128 TMEM lanes), the
// tokens the N operand (256 per tile = 256 TMEM columns), so one epilogue thread owns one output
// channel and its sum over tokens is thread-local.
//
// Tensor memory holds two full accumulators, columns [0,256) and [256,512), used in turn by
// consecutive passes.  The product x.w^T of a tile ("reference pass") is moved into registers by the
// epilogue warps (128 values per thread) as soon as it is complete and stays there for all the
// candidates of the tile, so both accumulators are free for candidates: the MMAs of candidate g+1
// run while the epilogue reads candidate g.
//
// Work items are (channel tile, token tile, block, candidate).  Whole waves of tiles are walked in
// step, one tile per worker and all its candidates in turn, so that workers which share an operand
// tile ask for it at the same time (one read from HBM, the rest from L2); what is left over after
// the last full wave runs as a wave too if it fills most of one, and is otherwise cut at the
// granularity of one candidate pass, a worker recomputing the reference pass of a tile it enters
// in the middle.
//
// A worker is one CTA, or, for long passes with a reference product, a pair of CTAs (cluster of two,
// cta_group::2, M = 256): each CTA stages its own channel tile and half of the token tile, the leader
// issues the MMAs for both, tcgen05.commit with cluster multicast signals the barriers of both, the
// partner's epilogue arrives on the leader's barrier through the cluster's shared window.  No TMA
// load uses multicast.
//
// Warp roles (384 threads, three groups of four warps): warp 0 TMA producer, warp 1 TMEM allocation
// + MMA issue (the warp walks its loop uniformly, one elected lane issues a whole stage as
// straight-line code), warps 2-3 idle, warps 4-11 epilogue (two per TMEM lane quadrant, one per half
// of the columns).  The first group gives registers up (setmaxnreg 56) and the epilogue groups take
// them (224): an epilogue thread holds 128 values of the reference product, and at the 168 registers
// a thread of this CTA gets by default its loop spilled (23 local-memory loads per pass and warp,
// which a pass of a 64-channel block, four MMAs and a whole epilogue, cannot hide).  Every wait is
// bounded: on a time-out the kernel raises the status word, all roles leave their loops, TMEM is
// freed and the kernel returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace ab {
namespace {

constexpr int BM = 128;      // output channels per tile (MMA M, TMEM lanes)
constexpr int BN = 256;      // tokens per tile (MMA N, TMEM columns per accumulator)
constexpr int BK = 64;       // K elements per pipeline stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;   // K elements per tcgen05.mma (16-bit operands)
constexpr int kEpiWarps = 8;                 // two per TMEM lane quadrant
// Three groups of four warps: producer, MMA issue and two idle warps; then the epilogue warps.
// Registers can only be moved between warps in such groups of four.
constexpr int kSeqThreads = 128 + 32 * kEpiWarps;
constexpr int kRegsFew = 56, kRegsMany = 224;  // 4 * 56 + 8 * 224 = 12 * 168, the compiled allocation
constexpr int kHalfCols = BN / 2;            // columns of one epilogue thread
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t TMEM_COLS = 512;          // two accumulators of BN columns
// A CTA on its own stages the whole token tile; a CTA of a pair stages half of it (the tensor cores
// of both read both halves), which leaves room for a deeper ring.
template <bool PAIR> struct Ring {
    static constexpr int kStages = PAIR ? 6 : 4;
    static constexpr int kTokenRows = PAIR ? BN / 2 : BN;  // rows of the token operand per CTA and stage
    static constexpr uint32_t kStageBytes = A_BYTES + kTokenRows * BK * 2;
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};
constexpr unsigned long long kWaitTimeoutNs = 2000000000ull;  // 2 s per wait
constexpr int64_t kSegLen = 512;  // columns per segment of a contraction without reference product

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
                                          int code, unsigned long long limit_ns = kWaitTimeoutNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) {
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

// --- a pair of CTAs (cluster of two) working on one tile with the tensor cores of both SMs ---
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// a tile into this CTA's shared memory, completion counted on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the barrier at this offset in both CTAs of the pair, once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
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
template <bool PAIR>
__device__ __forceinline__ void umma_issue(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
    if (PAIR)
        umma_f16_pair(d_tmem, adesc, bdesc, idesc, accumulate);
    else
        umma_f16(d_tmem, adesc, bdesc, idesc, accumulate);
}
template <bool PAIR> __device__ __forceinline__ void umma_commit_to(uint32_t bar) {
    if (PAIR)
        umma_commit_pair(bar);
    else
        umma_commit(bar);
}
// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct SeqArgs {
    int64_t M, N, K;   // tokens, output channels, input channels (all blocks)
    int64_t Kb;        // input channels per block (multiple of 16 when there are several blocks)
    int64_t seg_len;   // columns per segment (multiple of BK); a block has num_seg segments
    int num_seg;
    int num_blocks;
    int num_cand;
    int n_ct, n_tt;    // channel tiles, token tiles
    int loss_kind;     // 0 squared, 1 absolute, 2 squared + square of the second product,
                       // 3 squared + square of the first product
    int lowp;          // 0 none, 1 round like bfloat16, 2 round like float16
    uint32_t idesc;
    float *partial;    // [2 * n_tt][num_cand][N][num_blocks][nvals]
    int *status;
    unsigned long long timeout_ns;
};

// two values at a time: one packed conversion (full rate; the scalar one runs on the conversion
// pipe at a quarter of it) and two unpacking bit operations
__device__ __forceinline__ void round_lowp2(float &a, float &b, int lowp) {
    if (lowp == 1) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        const uint32_t u = *reinterpret_cast<const uint32_t *>(&h);
        a = __uint_as_float(u << 16);
        b = __uint_as_float(u & 0xffff0000u);
    } else if (lowp == 2) {
        const float2 f = __half22float2(__floats2half2_rn(a, b));
        a = f.x;
        b = f.y;
    }
}

// The sequence of passes of one CTA, identical in every role.
//
// A unit is (channel tile, token tile, block); an item is (unit, candidate).  Units are dealt out in
// waves of one unit per CTA: all CTAs then walk the candidates of their units in step, so the CTAs
// that share a tile ask for the same operand data at the same time (one read from HBM, the rest
// from L2).  The units left
// over after the last full wave are cut at item granularity, every CTA taking an equal share of
// (unit, candidate) pairs, so that a weight shard with fewer tiles than SMs still occupies all
// of them.  For every unit it touches a CTA first runs the reference pass (g == -1) when the kernel
// has one.  Without a reference product a candidate's columns may be cut into segments, one pass
// each, which the epilogue adds up in registers.
struct Pass {
    int ct, tt, blk, g, seg;
};
struct PassIter {
    // 32-bit throughout (the host refuses problems with 2^31 items or more): every thread of the
    // CTA walks this sequence, and in the epilogue warps its state competes for registers with the
    // reference product
    int wave_unit, full_units, i, i1, done_unit, cur_unit;
    int wave_g, cur_g, seg_left;
    int num_cand, n_tt, num_blocks, num_seg;
    bool has_ref, ref_pending;
    int n_ct, width, rank;
    int G;
    // the remainder's position as (unit, candidate) and the decoded tile of the current unit: both
    // advance without divisions (a block of 64 input channels is one short pass)
    int rem_u, dec_unit;
    int rem_g, dec_ct, dec_tt, dec_blk;
    // `pair`: the workers are pairs of CTAs; a pair's unit spans two channel tiles, one per CTA
    __device__ PassIter(const SeqArgs &a, bool ref, bool pair) {
        width = pair ? 2 : 1;
        rank = pair ? (int)(blockIdx.x & 1u) : 0;
        n_ct = (a.n_ct + width - 1) / width;
        const int64_t units = (int64_t)n_ct * a.n_tt * a.num_blocks;
        G = (int)(gridDim.x / width);
        const int64_t me = blockIdx.x / width;
        int64_t full = units / G * G;
        // Left-over units that would fill most of a wave are run as one (some workers idle): walked
        // in step a pass takes 26 us, against 33 us for workers that start in the middle of
        // different units and ask for different candidates' weights at the same time, which beats
        // the even split once the left-over exceeds about three quarters of a wave.
        if ((units - full) * 100 >= 77 * (int64_t)G) full = units;
        full_units = (int)full;
        wave_unit = (int)me;
        wave_g = 0;
        const int64_t items = (units - full) * a.num_cand;
        i = (int)(items * me / G);
        i1 = (int)(items * (me + 1) / G);
        rem_u = i / a.num_cand;
        rem_g = i - rem_u * a.num_cand;
        dec_unit = -1;
        dec_ct = dec_tt = dec_blk = 0;
        done_unit = -1;
        cur_unit = 0;
        cur_g = 0;
        seg_left = 0;
        num_cand = a.num_cand;
        n_tt = a.n_tt;
        num_blocks = a.num_blocks;
        num_seg = a.num_seg;
        has_ref = ref;
        ref_pending = false;
    }
    __device__ bool next_item() {
        if (wave_unit < full_units) {
            cur_unit = wave_unit;
            cur_g = wave_g;
            if (++wave_g == num_cand) {
                wave_g = 0;
                wave_unit += G;
            }
            return true;
        }
        if (i < i1) {
            cur_unit = full_units + rem_u;
            cur_g = rem_g;
            ++i;
            if (++rem_g == num_cand) {
                rem_g = 0;
                ++rem_u;
            }
            return true;
        }
        return false;
    }
    __device__ bool next(Pass &p) {
        if (seg_left == 0) {
            if (!next_item()) return false;
            seg_left = num_seg;
            if (has_ref && cur_unit != done_unit) {
                done_unit = cur_unit;
                ref_pending = true;
            }
        }
        if (cur_unit != dec_unit) {
            dec_unit = cur_unit;
            const int t = cur_unit / num_blocks;
            dec_blk = cur_unit - t * num_blocks;
            // token-tile major: the CTAs of a wave share few token tiles (the larger operand tile) and
            // spread over the channel tiles (measured: 4 % faster than channel-tile major)
            dec_tt = t / n_ct;
            dec_ct = (t - dec_tt * n_ct) * width + rank;
        }
        p.blk = dec_blk;
        p.tt = dec_tt;
        p.ct = dec_ct;
        if (ref_pending) {
            ref_pending = false;
            p.g = -1;
            p.seg = 0;
            return true;
        }
        p.g = cur_g;
        p.seg = num_seg - seg_left;
        --seg_left;
        return true;
    }
};

// One thread's share of a candidate pass: its kHalfCols accumulator columns against the values in
// xw[] (the reference product, or the earlier segments' sum), summed.  KIND / LOWP >= 0 fix the loss
// and the rounding at compile time, -1 leaves them to the run-time arguments.  Chunks of 16 columns,
// the next one requested before the current one is used.
template <bool HAS_REF, int KIND, int LOWP>
__device__ __forceinline__ void candidate_epilogue(uint32_t t0, const float (&xw)[kHalfCols], bool first_seg, int kind_rt,
                                                   int lowp_rt, float &s0, float &s1) {
    const int kind = KIND >= 0 ? KIND : kind_rt;
    const int lowp = LOWP >= 0 ? LOWP : lowp_rt;
    constexpr int CW = 16;
    uint32_t ca[CW], cb[CW];
    tmem_ld16(t0, ca);
#pragma unroll
    for (int ch = 0; ch < kHalfCols / CW; ++ch) {
        tmem_ld_wait();
        if (ch + 1 < kHalfCols / CW) {
            if (ch & 1)
                tmem_ld16(t0 + (ch + 1) * CW, ca);
            else
                tmem_ld16(t0 + (ch + 1) * CW, cb);
        }
#pragma unroll
        for (int j = 0; j < CW; j += 2) {
            float y0 = __uint_as_float((ch & 1) ? cb[j] : ca[j]);
            float y1 = __uint_as_float((ch & 1) ? cb[j + 1] : ca[j + 1]);
            float d0, d1;
            if (HAS_REF) {
                if (lowp) round_lowp2(y0, y1, lowp);
                d0 = xw[ch * CW + j] - y0;
                d1 = xw[ch * CW + j + 1] - y1;
            } else {  // the candidate's whole contraction
                d0 = y0 + (first_seg ? 0.f : xw[ch * CW + j]);
                d1 = y1 + (first_seg ? 0.f : xw[ch * CW + j + 1]);
            }
            float f0 = kind == 1 ? fabsf(d0) : d0 * d0;
            float f1 = kind == 1 ? fabsf(d1) : d1 * d1;
            if (lowp) round_lowp2(f0, f1, lowp);
            s0 += f0;
            s0 += f1;
            if (kind == 2) {
                float q0 = y0 * y0, q1 = y1 * y1;
                if (lowp) round_lowp2(q0, q1, lowp);
                s1 += q0;
                s1 += q1;
            }
        }
    }
}

template <bool HAS_REF, bool PAIR>
__global__ void __launch_bounds__(kSeqThreads, 1)
k_seqmse(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wq,
         const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_xq, SeqArgs a) {
    using R = Ring<PAIR>;
    constexpr int STAGES = R::kStages;
    constexpr uint32_t STAGE_BYTES = R::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(aligned + (size_t)STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty
    const uint32_t bar_full = smem_u32(bars);
    const uint32_t bar_empty = smem_u32(bars + STAGES);
    const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES);
    const uint32_t bar_acc_empty = smem_u32(bars + 2 * STAGES + 2);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // In a pair the CTA of rank 0 leads: it issues the MMAs for both, so the barriers that the MMA
    // thread waits on (operands landed, accumulator read out) are the leader's and collect the
    // arrivals of both CTAs; the barriers that the MMA thread signals (stage free, accumulator
    // complete) exist in both CTAs and are signalled together.
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const uint32_t lead_full = PAIR ? map_to_rank(bar_full, 0) : bar_full;
    const uint32_t lead_acc_empty = PAIR ? map_to_rank(bar_acc_empty, 0) : bar_acc_empty;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, (PAIR ? 2 : 1) * 32 * kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // one warp of each CTA of a pair allocates: both get the same columns
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the partner's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const unsigned long long limit = a.timeout_ns;
    // The epilogue threads keep 128 values of the reference product in registers and want as many
    // accumulator columns in flight from TMEM as they can get; the producer and the MMA warp need
    // little.  The first group of four warps hands registers over to the other two.
    // (Each of the two instructions is executed by whole groups of four warps and dominates the
    // code of its roles, which is how the compiler knows each role's allowance.)

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsFew));
    if (warp == 0) {
        // ---------------- TMA producer (in a pair: each CTA loads its own channel tile and its half
        // of the token tile) ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            PassIter it(a, HAS_REF, PAIR);
            Pass p;
            while (ok && it.next(p)) {
                const CUtensorMap *ma = p.g < 0 ? &tm_w : &tm_wq;
                const CUtensorMap *mb = p.g < 0 ? &tm_x : &tm_xq;
                const int row_a = p.g < 0 ? p.ct * BM : (int)((int64_t)p.g * a.N) + p.ct * BM;
                const int row_b = p.tt * BN + (int)rank * R::kTokenRows;
                const int64_t seg0 = (int64_t)p.seg * a.seg_len;
                const int64_t len = a.Kb - seg0 < a.seg_len ? a.Kb - seg0 : a.seg_len;
                const int col0 = (int)((int64_t)p.blk * a.Kb + seg0);
                const int kblocks = (int)((len + BK - 1) / BK);
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, a.status, ST_TIMEOUT_PRODUCER, limit);
                    if (!ok) break;
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    if (PAIR) {
                        // the leader's barrier counts the bytes of both CTAs (a partner's bytes may
                        // land before the leader has announced them: the phase cannot complete
                        // without the leader's arrival)
                        if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * STAGE_BYTES);
                        tma_load_2d_pair(sa, ma, col0 + kb * BK, row_a, lead_full + 8 * stage);
                        tma_load_2d_pair(sa + A_BYTES, mb, col0 + kb * BK, row_b, lead_full + 8 * stage);
                    } else {
                        mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
                        tma_load_2d(sa, ma, col0 + kb * BK, row_a, bar_full + 8 * stage);
                        tma_load_2d(sa + A_BYTES, mb, col0 + kb * BK, row_b, bar_full + 8 * stage);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue (in a pair: by the leader, for both CTAs) ----------------
        // The whole warp walks the loop and one elected lane issues: all the loop's values are then
        // uniform over the warp, which lets the operand descriptors be formed where the MMA
        // instruction reads them.  (Issued from a one-lane branch, every MMA cost about 200 cycles
        // whatever its size; a 128 x 256 x 16 MMA takes 128 at full rate.)
        if (rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t pass = 0;  // passes issued by this CTA: accumulator = pass & 1
            bool ok = true;
            PassIter it(a, HAS_REF, PAIR);
            Pass p;
            while (ok && it.next(p)) {
                const uint32_t buf = pass & 1u, use = pass >> 1;
                // the accumulator must have been read out by the epilogue of its previous pass
                // (a fresh barrier lets the first use through)
                ok = mbar_wait(bar_acc_empty + 8 * buf, (use & 1u) ^ 1u, abort_flag, a.status, ST_TIMEOUT_MMA, limit);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int64_t seg0 = (int64_t)p.seg * a.seg_len;
                const int64_t len = a.Kb - seg0 < a.seg_len ? a.Kb - seg0 : a.seg_len;
                const int kblocks = (int)((len + BK - 1) / BK);
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, a.status, ST_TIMEOUT_MMA, limit);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    const uint64_t da = make_smem_desc(sa);
                    const uint64_t db = make_smem_desc(sa + A_BYTES);
                    // the last stage of a block may reach beyond it: only the block's own columns
                    // count (a block is a multiple of 16 columns, or, if it is the only one, the
                    // columns beyond it are zero-filled by TMA)
                    const int64_t left = len - (int64_t)kb * BK;
                    const int ksteps = left >= BK ? BK / UMMA_K : (int)((left + UMMA_K - 1) / UMMA_K);
                    if (elect_one()) {
                        // a step advances 32 bytes (16 elements) inside the swizzled 128-byte row; a
                        // whole stage is straight-line code
                        if (ksteps == BK / UMMA_K) {
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                umma_issue<PAIR>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), a.idesc,
                                                 (kb > 0 || k > 0) ? 1u : 0u);
                        } else {
                            for (int k = 0; k < ksteps; ++k)
                                umma_issue<PAIR>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), a.idesc,
                                                 (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        // frees the stage (in both CTAs) once these MMAs have read it
                        umma_commit_to<PAIR>(bar_empty + 8 * stage);
                    }
                    __syncwarp();
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok && elect_one()) umma_commit_to<PAIR>(bar_acc_full + 8 * buf);
                __syncwarp();
                ++pass;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMany));
        // ---------------- epilogue: warps 4..11 ----------------
        // a warp may only read the TMEM lanes of its quadrant (warp index mod 4); the two warps of a
        // quadrant take one half of the accumulator's columns each
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const uint32_t lane_base = ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * kHalfCols);
        const int nvals = a.loss_kind >= 2 ? 2 : 1;
        const int lowp = a.lowp, kind = a.loss_kind;
        // with a reference pass: the reference product of this thread's channel and columns;
        // without: the sum of the segments of the current candidate seen so far
        float xw[kHalfCols];
        float sref = 0.f;  // sum of squares of the reference product
        uint32_t pass = 0;
        bool ok = true;
        PassIter it(a, HAS_REF, PAIR);
        Pass p;
        while (ok && it.next(p)) {
            const uint32_t buf = pass & 1u, use = pass >> 1;
            ++pass;
            ok = mbar_wait(bar_acc_full + 8 * buf, use & 1u, abort_flag, a.status, ST_TIMEOUT_EPILOGUE, limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + lane_base + buf * BN;
            const bool first_seg = p.seg == 0, last_seg = p.seg == a.num_seg - 1;
            if ((HAS_REF && p.g < 0) || (!HAS_REF && !last_seg)) {
                // move the accumulator into registers: the reference product, or one more segment
                if (HAS_REF) sref = 0.f;
#pragma unroll
                for (int ch = 0; ch < kHalfCols / 16; ++ch) {
                    uint32_t r[16];
                    tmem_ld16(t0 + ch * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
                        if (HAS_REF) {
                            if (lowp) round_lowp2(v0, v1, lowp);
                            if (kind == 3) {  // the signal power, for the signal-to-noise loss
                                float q0 = v0 * v0, q1 = v1 * v1;
                                if (lowp) round_lowp2(q0, q1, lowp);
                                sref += q0;
                                sref += q1;
                            }
                            xw[ch * 16 + j] = v0;
                            xw[ch * 16 + j + 1] = v1;
                        } else {
                            xw[ch * 16 + j] = v0 + (first_seg ? 0.f : xw[ch * 16 + j]);
                            xw[ch * 16 + j + 1] = v1 + (first_seg ? 0.f : xw[ch * 16 + j + 1]);
                        }
                    }
                }
                tc_fence_before();
                if (PAIR)
                    mbar_arrive_cluster(lead_acc_empty + 8 * buf);
                else
                    mbar_arrive(bar_acc_empty + 8 * buf);
                continue;
            }
            float s0 = 0.f, s1 = 0.f;
            // the two usual cases (squared error, plain or rounded like bfloat16) as straight-line
            // code without run-time switches: a pass of a 64-channel block is all epilogue, and the
            // general form is several times the instructions
            if (kind == 0 && lowp == 0)
                candidate_epilogue<HAS_REF, 0, 0>(t0, xw, first_seg, kind, lowp, s0, s1);
            else if (kind == 0 && lowp == 1)
                candidate_epilogue<HAS_REF, 0, 1>(t0, xw, first_seg, kind, lowp, s0, s1);
            else
                candidate_epilogue<HAS_REF, -1, -1>(t0, xw, first_seg, kind, lowp, s0, s1);
            tc_fence_before();
            if (PAIR)
                mbar_arrive_cluster(lead_acc_empty + 8 * buf);
            else
                mbar_arrive(bar_acc_empty + 8 * buf);
            const int64_t n = (int64_t)p.ct * BM + quad * 32 + lane;
            if (n < a.N) {
                const int64_t sub = (int64_t)p.tt * 2 + half;
                float *out = a.partial +
                             (((sub * a.num_cand + p.g) * a.N + n) * a.num_blocks + p.blk) * nvals;
                out[0] = s0;
                if (nvals == 2) out[1] = kind == 3 ? sref : s1;
            }
        }
    }

    // teardown: every role has left its loop (normally or through the abort flag)
    // (in a pair: in both CTAs, so neither leaves while the other may still signal its barriers)
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    tc_fence_after();
    if (warp == 1) {
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// out[i] = sum over token sub-tiles, in tile order (deterministic)
__global__ void k_seqmse_reduce(const float *partial, float *out, int n_sub, int64_t per_tile) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= per_tile) return;
    float s = 0.f;
    for (int t = 0; t < n_sub; ++t) s += partial[(int64_t)t * per_tile + i];
    out[i] = s;
}

// A wait that nothing completes: exercises the bounded wait's give-up path (status word, return)
// without any fault.  One warp waits on a barrier no one arrives at.
__global__ void k_wait_selftest(int *status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, ST_TIMEOUT_EPILOGUE, limit_ns);
    if (ok) atomicCAS(status, 0, -1);  // the wait claimed a completion that never happened
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

// The kernel moves registers between its warp groups: 4 x kRegsFew + 8 x kRegsMany must not exceed
// what the CTA was given at launch (12 warps x the compiled register count), or the warps asking for
// more would wait for registers that never come.  Checked once per kernel, before its first launch.
template <auto kernel> int check_register_allowance() {
    static std::mutex mu;
    static int state = 0;  // 0 unknown, 1 fine, -1 refused
    std::lock_guard<std::mutex> lock(mu);
    if (state == 0) {
        cudaFuncAttributes attr;
        AB_CUDA_OK(cudaFuncGetAttributes(&attr, kernel));
        state = (kSeqThreads / 32) * attr.numRegs >= 4 * kRegsFew + kEpiWarps * kRegsMany ? 1 : -1;
    }
    if (state < 0)
        return fail(AB_ERR_CUDA, "the loss kernel was compiled with fewer registers than its warp groups exchange");
    return AB_OK;
}

// How many CTA pairs the device runs at once (0: the paired kernel cannot be used), per device.
int pair_cluster_count(int *out) {
    static int cached[64];
    static bool known[64];
    static std::mutex mu;
    int dev = 0;
    AB_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) {
        *out = 0;
        return AB_OK;
    }
    if (!known[dev]) {
        int rc = opt_in_smem<k_seqmse<true, true>>(Ring<true>::kSmemBytes);
        if (rc != AB_OK) return rc;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (unsigned)sm_count());
        cfg.blockDim = dim3(kSeqThreads);
        cfg.dynamicSmemBytes = Ring<true>::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, k_seqmse<true, true>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        cached[dev] = n;
        known[dev] = true;
    }
    *out = cached[dev];
    return AB_OK;
}

int64_t blocks_scratch_bytes(int64_t M, int64_t N, int32_t num_blocks, int32_t num_cand) {
    const int64_t n_tt = (M + BN - 1) / BN;
    return 2 * n_tt * num_cand * N * num_blocks * 2 * (int64_t)sizeof(float);
}

}  // namespace
}  // namespace ab

extern "C" int64_t aimet_b200_seqmse_blocks_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t num_blocks,
                                                          int32_t num_cand) {
    (void)K;
    if (M <= 0 || N <= 0 || num_cand <= 0 || num_blocks <= 0)
        return ab::fail(AB_ERR_INVALID, "M, N, num_blocks and num_cand must be positive");
    return ab::blocks_scratch_bytes(M, N, num_blocks, num_cand);
}

extern "C" int64_t aimet_b200_seqmse_scratch_bytes(int64_t M, int64_t N, int64_t K, int32_t num_cand) {
    return aimet_b200_seqmse_blocks_scratch_bytes(M, N, K, 1, num_cand);
}

extern "C" int aimet_b200_seqmse_linear_loss_blocks(const void *x, const void *xq, const void *w, const void *wq,
                                                    int64_t M, int64_t N, int64_t K, int32_t num_blocks,
                                                    int32_t num_cand, int io_dtype, int loss_kind, int lowp_epilogue,
                                                    int has_reference, float *out, int32_t *status, void *scratch,
                                                    int64_t scratch_bytes, void *stream) {
    using namespace ab;
    if (io_dtype != AB_BF16 && io_dtype != AB_F16)
        return fail(AB_ERR_UNSUPPORTED, "seqmse_linear_loss takes bfloat16 or float16 operands");
    if (M <= 0 || N <= 0 || K <= 0 || num_cand <= 0 || num_blocks <= 0)
        return fail(AB_ERR_INVALID, "M, N, K, num_blocks and num_cand must be positive");
    if (K % num_blocks != 0) return fail(AB_ERR_INVALID, "K (%lld) is not a multiple of num_blocks (%d)", (long long)K, (int)num_blocks);
    const int64_t Kb = K / num_blocks;
    if (K % 8 != 0) return fail(AB_ERR_UNSUPPORTED, "K must be a multiple of 8 (16-byte rows for TMA), got %lld", (long long)K);
    if (num_blocks > 1 && Kb % 16 != 0)
        return fail(AB_ERR_UNSUPPORTED, "the input channels of one block (%lld) must be a multiple of 16", (long long)Kb);
    if (loss_kind < 0 || loss_kind > 3) return fail(AB_ERR_INVALID, "loss_kind must be 0, 1, 2 or 3");
    if (!has_reference && loss_kind == 3) return fail(AB_ERR_INVALID, "loss_kind 3 needs the reference product");
    if (!has_reference) {  // the first product is absent: its operands are never read
        x = xq;
        w = wq;
    }
    if (!x || !xq || !w || !wq || !out || !status) return fail(AB_ERR_INVALID, "NULL pointer argument");
    for (const void *p : {x, xq, w, wq})
        if (!aligned16(p)) return fail(AB_ERR_INVALID, "operands must be 16-byte aligned");
    if ((int64_t)num_cand * N >= ((int64_t)1 << 31) || M >= ((int64_t)1 << 31) || K >= ((int64_t)1 << 31))
        return fail(AB_ERR_UNSUPPORTED, "row and column counts must fit 31 bits");
    if (((N + BM - 1) / BM) * ((M + BN - 1) / BN) * num_blocks * num_cand >= ((int64_t)1 << 31))
        return fail(AB_ERR_UNSUPPORTED, "tiles x blocks x candidates must fit 31 bits");
    const int64_t need = blocks_scratch_bytes(M, N, num_blocks, num_cand);
    if (!scratch || scratch_bytes < need)
        return fail(AB_ERR_SCRATCH, "seqmse needs %lld bytes of scratch, got %lld", (long long)need, (long long)scratch_bytes);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SeqArgs a;
    a.M = M;
    a.N = N;
    a.K = K;
    a.Kb = Kb;
    a.num_blocks = num_blocks;
    a.num_cand = num_cand;
    a.n_ct = (int)((N + BM - 1) / BM);
    a.n_tt = (int)((M + BN - 1) / BN);
    a.loss_kind = loss_kind;
    a.lowp = lowp_epilogue ? (io_dtype == AB_BF16 ? 1 : 2) : 0;
    a.partial = static_cast<float *>(scratch);
    a.status = status;
    a.timeout_ns = kWaitTimeoutNs;
    // Without a reference product the caller has formed differences itself and wants them summed
    // accurately: the tensor core truncates its accumulator after every step, a bias that grows
    // with the number of steps, so a long contraction is cut into segments of kSegLen columns
    // whose sums are added in registers (round to nearest).
    a.seg_len = has_reference ? ((Kb + BK - 1) / BK) * BK : kSegLen;
    a.num_seg = (int)((Kb + a.seg_len - 1) / a.seg_len);

    // With a reference product, at least two channel tiles and long passes, pairs of CTAs share a
    // token tile: each CTA stages half of it and the tensor cores of both SMs read both halves,
    // which takes a third off the operand bytes an SM has to pull in per pass.  Short passes are
    // bound by the epilogue and the hand-over between the roles, which costs twice as much across
    // two CTAs, and stay single.  Measured on the 4096-channel layer cut into blocks: 512 channels
    // per block 5.3 ms paired against 6.1-6.6 ms single, 256 channels 7.3-7.8 ms against 5.8 ms.
    int pair_clusters = 0;
    if (has_reference && a.n_ct >= 2 && Kb >= 512) {
        int rc2 = pair_cluster_count(&pair_clusters);
        if (rc2 != AB_OK) return rc2;
    }
    const bool pair = pair_clusters > 0;

    CUtensorMap tm_w, tm_wq, tm_x, tm_xq;
    int rc;
    const int token_rows = pair ? Ring<true>::kTokenRows : Ring<false>::kTokenRows;
    if ((rc = make_map(&tm_w, w, has_reference ? N : (int64_t)num_cand * N, K, BM, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_wq, wq, (int64_t)num_cand * N, K, BM, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_x, x, M, K, token_rows, io_dtype)) != AB_OK) return rc;
    if ((rc = make_map(&tm_xq, xq, M, K, token_rows, io_dtype)) != AB_OK) return rc;

    const uint32_t fmt = io_dtype == AB_BF16 ? 1u : 0u;
    const uint32_t mma_m = pair ? 2 * BM : BM;  // a pair's MMA spans the channel tiles of both CTAs
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((mma_m >> 4) << 24);

    AB_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
    if (pair) {
        const int64_t items = (int64_t)((a.n_ct + 1) / 2) * a.n_tt * num_blocks * num_cand;
        int clusters = pair_clusters;
        if (items < clusters) clusters = (int)items;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(2 * clusters));
        cfg.blockDim = dim3(kSeqThreads);
        cfg.dynamicSmemBytes = Ring<true>::kSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if ((rc = check_register_allowance<k_seqmse<true, true>>()) != AB_OK) return rc;
        AB_CUDA_OK(cudaLaunchKernelEx(&cfg, k_seqmse<true, true>, tm_w, tm_wq, tm_x, tm_xq, a));
    } else {
        // the opt-in to more than 48 KB of shared memory is a per-device attribute of the kernel
        if ((rc = opt_in_smem<k_seqmse<true, false>>(Ring<false>::kSmemBytes)) != AB_OK) return rc;
        if ((rc = opt_in_smem<k_seqmse<false, false>>(Ring<false>::kSmemBytes)) != AB_OK) return rc;
        if ((rc = check_register_allowance<k_seqmse<true, false>>()) != AB_OK) return rc;
        if ((rc = check_register_allowance<k_seqmse<false, false>>()) != AB_OK) return rc;
        const int64_t items = (int64_t)a.n_ct * a.n_tt * num_blocks * num_cand;
        int grid = sm_count();
        if (items < grid) grid = (int)items;
        if (has_reference)
            k_seqmse<true, false><<<grid, kSeqThreads, Ring<false>::kSmemBytes, st>>>(tm_w, tm_wq, tm_x, tm_xq, a);
        else
            k_seqmse<false, false><<<grid, kSeqThreads, Ring<false>::kSmemBytes, st>>>(tm_w, tm_wq, tm_x, tm_xq, a);
    }
    AB_LAUNCH_OK();
    const int nvals = loss_kind >= 2 ? 2 : 1;
    const int64_t per_tile = (int64_t)num_cand * N * num_blocks * nvals;
    k_seqmse_reduce<<<(unsigned)((per_tile + 255) / 256), 256, 0, st>>>(a.partial, out, 2 * a.n_tt, per_tile);
    AB_LAUNCH_OK();
    return AB_OK;
}

extern "C" int aimet_b200_seqmse_linear_loss(const void *x, const void *xq, const void *w, const void *wq, int64_t M,
                                             int64_t N, int64_t K, int32_t num_cand, int io_dtype, int loss_kind,
                                             int lowp_epilogue, float *out, int32_t *status, void *scratch,
                                             int64_t scratch_bytes, void *stream) {
    return aimet_b200_seqmse_linear_loss_blocks(x, xq, w, wq, M, N, K, 1, num_cand, io_dtype, loss_kind,
                                                lowp_epilogue, 1, out, status, scratch, scratch_bytes, stream);
}

extern "C" int aimet_b200_seqmse_wait_selftest(int32_t *status, int64_t limit_us, void *stream) {
    using namespace ab;
    if (!status) return fail(AB_ERR_INVALID, "status must not be NULL");
    if (limit_us <= 0 || limit_us > 1000000) return fail(AB_ERR_INVALID, "limit_us must be in (0, 1000000]");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AB_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), st));
    k_wait_selftest<<<1, 32, 0, st>>>(status, (unsigned long long)limit_us * 1000ull);
    AB_LAUNCH_OK();
    return AB_OK;
}
