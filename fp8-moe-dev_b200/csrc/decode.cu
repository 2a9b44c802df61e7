// Decode path: the whole layer for a batch of at most eight tokens as ONE cooperative kernel.
//
// With a handful of tokens every active expert has at most eight rows, the layer is nothing
// but streaming the active experts' weights once (44 MB per expert), and what the staged
// chain of five kernels spends between those streams -- four kernel boundaries, the permute,
// the padding of every expert to a 128-row tensor-core tile, TMEM set-up, the cross-CTA
// split-K hand-over -- costs more than the streams themselves.  Here:
//   * every CTA routes the (<= 8) tokens itself, with the same warp-per-token routine as the
//     staged chain, and derives the same active-expert table, so nothing has to be exchanged
//     before the first weight byte is requested;
//   * phase 1 (GEMM1 + SwiGLU): a unit is 8 SwiGLU columns of one active expert = 8 linear +
//     8 gated rows of W1, i.e. exactly one 16-row A tile of the warp-level
//     mma.sync.m16n8k32 (e4m3 x e4m3 -> fp32), with the expert's <= 8 token rows as the 8-wide
//     B tile.  The weights arrive by TMA, 16 rows x 1 KB per step (two boxes of 8 rows in
//     phase 1, one of 16 in phase 2) through a ring of four steps per half CTA; the warps
//     split K, promote per 128-K block with the two scales like the staged kernel, and meet
//     in shared memory.  (Per-thread loads and per-row bulk copies both left the HBM two
//     thirds idle: the first for the loads in flight a thread can hold, the second for the
//     rate at which one thread can issue sixteen copies per step.)
//     In the accumulator layout a thread owns the linear and the gated value of the same
//     (column, token), so SwiGLU needs no exchange.  v = silu(gate) * lin goes to a small
//     fp32 scratch (the 1x128 requantisation needs whole 128-column blocks, which span units);
//   * grid barrier; phase 2 (GEMM2): each CTA requantises the rows of its expert from the
//     scratch (same arithmetic as the staged epilogue), streams 16 rows of W2 per unit the
//     same way, and writes bf16 y rows; grid barrier; phase 3 is the weighted combine.
// The first weights of phase 2 are requested before the barrier, so the barrier and the
// requantisation hide behind their latency.  Every wait (mbarriers, grid barriers) is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "decode.cuh"
#include "layer.cuh"
#include "ptx.cuh"
#include "route_token.cuh"

namespace moe {

namespace {

constexpr int kDecWarps = 16;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kHalfWarps = 8;                           // the CTA works as two halves of 8 warps
constexpr int kHalfThreads = kHalfWarps * 32;
constexpr int kDecMaxActive = kDecodeMaxTokens * kTopK; // 64 (token, expert) pairs at most
constexpr int kHidStride = kHidden + 64;                // row strides that spread rows over the banks
constexpr int kA2Stride = kInter + 64;
constexpr int kG1Cols = 8;                              // SwiGLU columns of a phase-1 unit
constexpr int kG1Units = kInter / kG1Cols;              // 256 per expert
constexpr int kG2Cols = 16;                             // output columns of a phase-2 unit
constexpr int kG2Units = kHidden / kG2Cols;             // 448 per expert
// A step = 16 weight rows x 1 KB of K (8 K blocks, one per warp of the half).
constexpr int kStepRows = 16;
constexpr int kStepK = kHalfWarps * kBlock;             // 1024 bytes of every row
constexpr int kStepStride = kStepK;                     // rows of a step lie densely, as TMA writes them
constexpr int kStepBytes = kStepRows * kStepK;          // 16 KB arrive per step
constexpr int kG1Steps = kHidden / kStepK;              // 7 per phase-1 unit
constexpr int kG2Steps = kInter / kStepK;               // 2 per phase-2 unit
constexpr int kRing = 4;                                // steps in flight per half
constexpr int kCoopRouteTokens = 2;                     // up to here the CTA routes a token together
static_assert(kHidden % kStepK == 0 && kInter % kStepK == 0, "K splits into whole steps");
static_assert(2 * kDecodeMaxTokens * kA2Stride <= kDecodeMaxTokens * kHidStride, "phase 2 rows reuse the hidden-row area");

struct DecodeShared {
    int n_active, n_rows, abort, pad;
    int pair_count[kDecodeMaxTokens];
    int pair_le[kDecodeMaxTokens][kTopK];
    int pair_slot[kDecodeMaxTokens][kTopK];
    int pair_row[kDecodeMaxTokens][kTopK];
    float pair_w[kDecodeMaxTokens][kTopK];
    int act_expert[kDecMaxActive], act_m[kDecMaxActive], act_row0[kDecMaxActive];
    int act_tok[kDecMaxActive][kDecodeMaxTokens];
    int expert_slot[kMaxLocalExperts];
    // routing scratch
    float r_gscore[kDecodeMaxTokens][kNumGroups];
    int r_kept[kDecodeMaxTokens][kTopKGroup];
    int r_count[kDecodeMaxTokens][kTopKGroup][32];
    int r_idx[kDecodeMaxTokens][kTopK];
    float r_sel[kDecodeMaxTokens][kTopK];
    float hid_scale[kDecodeMaxTokens][kHiddenBlocks];      // [token][kb]
    float a2_scale[2][kDecodeMaxTokens][kInterBlocks];     // per half: [slot][kb] of the requantised rows
    alignas(8) uint64_t full_bar[2][kRing];
    alignas(8) uint64_t empty_bar[2][kRing];
    alignas(8) uint64_t hid_bar;
    alignas(16) float red[2][2][kHalfWarps][128];          // per half, by unit parity: the warps' partial sums
    // phase 1: the hidden rows of all tokens; phase 2: each half's requantised rows of its expert
    alignas(128) uint8_t rows[kDecodeMaxTokens * kHidStride];
    alignas(128) uint8_t wring[2][kRing][kStepRows * kStepStride];
};
static_assert(sizeof(DecodeShared) <= 227 * 1024, "decode kernel shared memory");

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Untiled bulk copy global -> shared memory of this CTA, completion counted on an mbarrier.
// Both addresses and the size are multiples of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 128-K block of the warp-level MMA tile: `arow` points at this K block in weight row r of
// the staged step (row r + 8 lies 8 strides further), `brow` at the same K block of token slot
// r's row; r = lane / 4, c = lane % 4.  A thread takes bytes [16c, 16c+16) and [64+16c, 64+16c+16)
// of the block from each; which 4 bytes feed which k index of the MMA is the same for A and B,
// and a dot product does not care about more.  (The choice cannot depend on the row: a product
// pairs the A bytes of one lane group with the B bytes of another.  The weight rows are 1 KB apart,
// so rows r and r + 1, which share a shared-memory access phase, collide two-way; that is cheap.)
__device__ __forceinline__ void mma_block(float (&acc)[4], const uint8_t* arow, const uint8_t* brow) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int off = 64 * h;
        const uint4 lo = *reinterpret_cast<const uint4*>(arow + off);
        const uint4 hi = *reinterpret_cast<const uint4*>(arow + 8 * kStepStride + off);
        const uint4 b = *reinterpret_cast<const uint4*>(brow + off);
        mma_e4m3(acc, lo.x, hi.x, lo.y, hi.y, b.x, b.y);
        mma_e4m3(acc, lo.z, hi.z, lo.w, hi.w, b.z, b.w);
    }
}

// All CTAs of the (cooperative, co-resident) grid meet here: one release-add on `counter`, then
// acquire-polls until all have arrived.  The kernel has two barriers on two counters; CTA 0 clears
// the second one before it arrives at the first (nobody can reach the second barrier earlier) and
// the first one after it has passed the second (everybody has left the first by then), so a launch
// finds and leaves the state it needs without a generation word.  Bounded: a CTA that waits longer
// than the limit records the failure and returns false; its peers run into the same limit.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, Control* ctrl, DecodeShared* sh)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        const uint64_t t0 = global_timer_ns();
        uint32_t it = 0;
        while (ld_acquire_gpu(counter) < gridDim.x) {
            if ((++it & 0x3fu) == 0u && global_timer_ns() - t0 > kWaitLimitNs) {
                atomicCAS(&ctrl->status, kStatusOk, kStatusDecodeTimeout);
                sh->abort = 1;
                break;
            }
        }
    }
    __syncthreads();
    return sh->abort == 0;
}

__global__ void __launch_bounds__(kDecThreads, 1) decode_layer_kernel(
    DecodeArgs a, const __grid_constant__ CUtensorMap tmap_w1, const __grid_constant__ CUtensorMap tmap_w2, Workspace ws)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    DecodeShared* sh = reinterpret_cast<DecodeShared*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;   // MMA fragment coordinates
    const int T = a.T, E = a.num_local_experts;
    const bool clocked = blockIdx.x == 0 && tid == 0;
    auto stamp = [&](int i) { if (clocked) ws.ctrl->dec_time[i] = global_timer_ns(); };
    // A failure that an earlier launch recorded stays in the status word until the host has read it
    // (moe_fp8_b200_check clears it together with any arrival counts that launch left on the grid
    // barriers).  Until then this kernel does nothing: with stale counts its barriers would open early.
    // Every CTA reads the same word; within one launch it can only change after a full wait limit.
    if (__ldcg(&ws.ctrl->status) != kStatusOk) return;
    stamp(0);
    volatile int* abort_flag = &sh->abort;

    // The tokens' hidden rows start moving before anything else: nothing depends on routing here.
    if (tid == 0) {
        sh->abort = 0;
        prefetch_tmap(&tmap_w1);
        prefetch_tmap(&tmap_w2);
        const uint32_t hb = smem_u32(&sh->hid_bar);
        mbar_init(hb, 1);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < kRing; ++j) {
                mbar_init(smem_u32(&sh->full_bar[h][j]), 1);
                mbar_init(smem_u32(&sh->empty_bar[h][j]), kHalfWarps);
            }
        fence_mbar_init();
        mbar_expect_tx(hb, (uint32_t)T * kHidden);
        for (int t = 0; t < T; ++t)
            bulk_g2s(smem_u32(sh->rows + t * kHidStride), a.hidden + (size_t)t * kHidden, kHidden, hb);
        if (blockIdx.x == 0) ws.ctrl->dec_phase = 0;   // second barrier's counter, see grid_barrier
    }
    for (int q = tid; q < T * kHiddenBlocks; q += kDecThreads) {
        const int t = q % T, kb = q / T;
        sh->hid_scale[t][kb] = __ldg(a.hscale + q);   // [56, T] -> [token][kb]
    }

    // ------------------------------------------------------------------ routing (every CTA)
    // For one or two tokens: the same selection as route_token_warp (route_token.cuh), spread over
    // the CTA's 16 warps, because the single-warp routine's chain of dependent reductions (about
    // 4 us) would be the longest serial stretch of the kernel.  Scores and their order-preserving keys go to
    // shared memory; one warp per (token, group) forms the group score; one thread per token keeps
    // the four best groups; then the eight argmax rounds are replaced by counting, for each of the
    // 128 live scores, how many of the others beat it (higher key, or equal key and earlier in the
    // reference's tie order): the score with count k is the k-th pick.  Same picks, same order.
    if (tid < kMaxLocalExperts) sh->expert_slot[tid] = -1;
    float* r_s = reinterpret_cast<float*>(&sh->wring[1][kRing - 1][0]);                 // [T][256], idle ring slot
    uint32_t* r_key = reinterpret_cast<uint32_t*>(r_s + kDecodeMaxTokens * kNumExperts);  // [T][256]
    static_assert(2 * kDecodeMaxTokens * kNumExperts * 4 <= kStepRows * kStepStride, "routing scratch fits a ring slot");
    stamp(12);
    if (T <= kCoopRouteTokens) {
        for (int q = tid; q < T * kNumExperts; q += kDecThreads) {
            const float l = __ldg(a.logits + q);
            const float sig = 1.0f / (1.0f + __expf(-l));
            r_s[q] = sig;
            r_key[q] = float_to_ordered(sig + __bfloat162float(a.bias[q & (kNumExperts - 1)]));
        }
        for (int q = tid; q < T * kTopKGroup * 32; q += kDecThreads) (&sh->r_count[0][0][0])[q] = 0;
        __syncthreads();
        for (int task = warp; task < T * kNumGroups; task += kDecWarps) {   // group score = two largest of the group
            const uint32_t key = r_key[task * 32 + lane];
            const uint32_t k1 = __reduce_max_sync(0xffffffffu, key);
            const uint32_t holders = __ballot_sync(0xffffffffu, key == k1);
            uint32_t k2 = k1;
            if (__popc(holders) < 2) k2 = __reduce_max_sync(0xffffffffu, key == k1 ? 0u : key);
            if (lane == 0) sh->r_gscore[task / kNumGroups][task % kNumGroups] = ordered_to_float(k1) + ordered_to_float(k2);
        }
        __syncthreads();
        if (tid < T) {   // four best groups, lowest index first on ties
            uint32_t kept_mask = 0;
            for (int k = 0; k < kTopKGroup; ++k) {
                float best = kNegSentinel;
                int best_i = -1;
                for (int i = 0; i < kNumGroups; ++i) {
                    const float gsc = sh->r_gscore[tid][i];
                    if (!((kept_mask >> i) & 1u) && gsc > best) { best = gsc; best_i = i; }
                }
                if (best_i >= 0) {
                    kept_mask |= 1u << best_i;
                    sh->r_kept[tid][k] = best_i;
                } else {
                    sh->r_kept[tid][k] = k;   // unreachable with finite scores; keeps the indices valid
                }
            }
        }
        __syncthreads();
        // count[t][j][lane]: how many live scores beat score `lane` of the j-th kept group; the work of one
        // (token, group) is split over four warps, one per opposing group
        for (int task = warp; task < T * kTopKGroup * kTopKGroup; task += kDecWarps) {
            const int t = task / (kTopKGroup * kTopKGroup), j = (task / kTopKGroup) % kTopKGroup, part = task % kTopKGroup;
            const int g = sh->r_kept[t][j], g2 = sh->r_kept[t][part];
            const uint32_t key = r_key[t * kNumExperts + g * 32 + lane];
            const uint32_t tie = (uint32_t)g * 32u + (__brev((uint32_t)lane) >> 27);
            const uint32_t* other = r_key + t * kNumExperts + g2 * 32;
            int beat = 0;
    #pragma unroll 8
            for (int l2 = 0; l2 < 32; ++l2) {
                const uint32_t key2 = other[l2];
                const uint32_t tie2 = (uint32_t)g2 * 32u + (__brev((uint32_t)l2) >> 27);
                beat += (key2 > key || (key2 == key && tie2 < tie)) ? 1 : 0;
            }
            atomicAdd(&sh->r_count[t][j][lane], beat);
        }
        __syncthreads();
        for (int task = warp; task < T * kTopKGroup; task += kDecWarps) {
            const int t = task / kTopKGroup, j = task % kTopKGroup;
            const int rank = sh->r_count[t][j][lane];
            if (rank < kTopK) {
                const int ge = sh->r_kept[t][j] * 32 + lane;
                sh->r_idx[t][rank] = ge;
                sh->r_sel[t][rank] = r_s[t * kNumExperts + ge];
            }
        }
        __syncthreads();
    } else if (warp < T) {
        // more tokens than that: one warp per token runs the staged chain's routine, the tokens in parallel
        int idx[kTopK];
        float wn[kTopK];
        route_token_warp(a.logits + (size_t)warp * kNumExperts, a.bias, lane, idx, wn);
        if (lane < kTopK) {
            int my_idx = 0;
            float my_s = 0.0f;
#pragma unroll
            for (int k = 0; k < kTopK; ++k)
                if (k == lane) { my_idx = idx[k]; my_s = wn[k]; }
            sh->r_idx[warp][lane] = my_idx;
            sh->r_sel[warp][lane] = my_s;   // already normalised
        }
    }
    if (T > kCoopRouteTokens) __syncthreads();
    stamp(8);
    if (tid < T) {
        const int t = tid;
        int idx[kTopK];
        float wn[kTopK];
        float sumw = 1e-20f;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) { idx[k] = sh->r_idx[t][k]; sumw += sh->r_sel[t][k]; }
        const float inv = 1.0f / sumw;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) wn[k] = T <= kCoopRouteTokens ? sh->r_sel[t][k] * inv : sh->r_sel[t][k];
        if (blockIdx.x == 0) {
#pragma unroll
            for (int k = 0; k < kTopK; ++k) {
                ws.topk_idx[(size_t)t * kTopK + k] = idx[k];
                ws.topk_weight[(size_t)t * kTopK + k] = wn[k];
            }
        }
        int n_pairs = 0;
        int p_le[kTopK];
        float p_w[kTopK];
#pragma unroll
        for (int i = 0; i < kTopK; ++i) { p_le[i] = 0; p_w[i] = 0.0f; }
        const int shards = E / kShardExperts;
        for (int sdx = 0; sdx < shards; ++sdx)
            dispatch_one_shard(idx, wn, sdx, a.local_expert_offset, a.pol, a.rsf, n_pairs, p_le, p_w);
        sh->pair_count[t] = n_pairs;
#pragma unroll
        for (int i = 0; i < kTopK; ++i) { sh->pair_le[t][i] = p_le[i]; sh->pair_w[t][i] = p_w[i]; }
        stamp(9);
    }
    __syncthreads();
    if (tid == 0) {
        // active experts in order of first use, rows of an expert in token order: the same in
        // every CTA, so unit u means the same thing everywhere
        int n_active = 0;
        for (int t = 0; t < T; ++t) {
            const int np = sh->pair_count[t];
            for (int p = 0; p < np; ++p) {
                const int le = sh->pair_le[t][p];
                int ai = sh->expert_slot[le];
                if (ai < 0) {
                    ai = n_active++;
                    sh->expert_slot[le] = ai;
                    sh->act_expert[ai] = le;
                    sh->act_m[ai] = 0;
                }
                const int slot = sh->act_m[ai]++;
                sh->act_tok[ai][slot] = t;
                sh->pair_slot[t][p] = slot;
            }
        }
        int rows = 0;
        for (int ai = 0; ai < n_active; ++ai) { sh->act_row0[ai] = rows; rows += sh->act_m[ai]; }
        sh->n_active = n_active;
        sh->n_rows = rows;
        stamp(10);
    }
    __syncthreads();
    if (tid < T * kTopK) {
        const int t = tid / kTopK, p = tid % kTopK;
        if (p < sh->pair_count[t]) sh->pair_row[t][p] = sh->act_row0[sh->expert_slot[sh->pair_le[t][p]]] + sh->pair_slot[t][p];
    }
    if (blockIdx.x == 0) {   // the tables other entry points and the tests read
        if (tid < T) ws.pair_count[tid] = sh->pair_count[tid];
        if (tid < T * kTopK) {
            const int t = tid / kTopK, p = tid % kTopK;
            if (p < sh->pair_count[t]) {
                ws.pair_code[tid] = ((uint32_t)sh->pair_le[t][p] << 24) | (uint32_t)sh->pair_slot[t][p];
                ws.pair_weight[tid] = sh->pair_w[t][p];
            }
        }
        if (tid < E) {
            const int ai = sh->expert_slot[tid];
            ws.ctrl->expert_rows[tid] = ai >= 0 ? sh->act_m[ai] : 0;
        }
    }
    stamp(11);
    __syncthreads();
    const int n_active = sh->n_active;
    stamp(1);
    float* act = ws.splitk_partial;   // [rows, 2048] fp32 SwiGLU output (the split-K scratch is idle on this path)

    // The 16 warps work as two independent halves of 8 (named barriers 1 and 2): a half is one
    // worker with its own unit range, weight ring and reduction buffer, so an SM always has two
    // units in flight and the unit ranges are twice as fine.  Thread 0 of a half is its producer:
    // it issues the bulk copies of a step (16 rows x 1 KB) as soon as the ring slot is free -- of
    // the next unit and, before the grid barrier, of the next phase as well.  Warp hw of the half
    // consumes K block hw of every step.
    const int half = warp >> 3, hw = warp & (kHalfWarps - 1), htid = tid & (kHalfThreads - 1);
    const int workers = (int)gridDim.x * 2, wk = (int)blockIdx.x * 2 + half;
    const int bar_id = 1 + half;
    const bool producer = htid == 0;
    const int units1 = n_active * kG1Units, units2 = n_active * kG2Units;
    const int u1_begin = (int)((long long)units1 * wk / workers), u1_end = (int)((long long)units1 * (wk + 1) / workers);
    const int u2_begin = (int)((long long)units2 * wk / workers), u2_end = (int)((long long)units2 * (wk + 1) / workers);
    const int S1 = (u1_end - u1_begin) * kG1Steps, S2 = (u2_end - u2_begin) * kG2Steps;
    int issued = 0;     // steps issued so far by this half's producer (both phases)
    int consumed = 0;   // steps consumed so far by this half
    bool ok = true;

    // producer only: step s of phase 1 (s < S1) or phase 2 (s - S1)
    auto issue = [&](int s) -> bool {
        const int slot = issued & (kRing - 1);
        if (issued >= kRing &&
            !mbar_wait(smem_u32(&sh->empty_bar[half][slot]), (uint32_t)((issued / kRing - 1) & 1), abort_flag))
            return false;
        const uint32_t bar = smem_u32(&sh->full_bar[half][slot]);
        const uint32_t dst = smem_u32(&sh->wring[half][slot][0]);
        mbar_expect_tx(bar, kStepBytes);
        if (s < S1) {
            const int u = u1_begin + s / kG1Steps, i = s % kG1Steps;
            const int row = sh->act_expert[u / kG1Units] * kGemm1Out + (u % kG1Units) * kG1Cols;
            tma_load_2d(dst, &tmap_w1, bar, i * (kStepK / 4), row);                              // 8 linear rows
            tma_load_2d(dst + 8 * kStepStride, &tmap_w1, bar, i * (kStepK / 4), row + kInter);   // 8 gated rows
        } else {
            const int s2 = s - S1;
            const int u = u2_begin + s2 / kG2Steps, i = s2 % kG2Steps;
            tma_load_2d(dst, &tmap_w2, bar, i * (kStepK / 4), sh->act_expert[u / kG2Units] * kHidden + (u % kG2Units) * kG2Cols);
        }
        ++issued;
        return true;
    };
    // everybody: wait for the next step's bytes; returns the ring slot
    auto acquire = [&]() -> const uint8_t* {
        const int slot = consumed & (kRing - 1);
        if (!mbar_wait(smem_u32(&sh->full_bar[half][slot]), (uint32_t)((consumed / kRing) & 1), abort_flag)) ok = false;
        return &sh->wring[half][slot][0];
    };
    auto release = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh->empty_bar[half][consumed & (kRing - 1)]));
        ++consumed;
    };

    if (producer) {
        for (int s = 0; s < kRing && s < S1 + S2 && ok; ++s)
            if (s < S1 || S1 == 0) ok = issue(s);   // phase-2 steps are not issued ahead of phase 1 here, see below
    }
    // the hidden rows must have landed before the first MMA
    if (!mbar_wait(smem_u32(&sh->hid_bar), 0u, abort_flag)) ok = false;

    // ------------------------------------------------------------------ phase 1: GEMM1 + SwiGLU
    {
        int ai = 0, g = 0, m = 0;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // The weight scales of a unit's K blocks sit in lanes 0..13 of the warp that uses them (7
        // linear, 7 gated), fetched one unit ahead so that no step waits for them.
        auto unit_scales = [&](int u) -> float {
            float v = 0.0f;
            if (u < u1_end && lane < 2 * kG1Steps) {
                const int e = sh->act_expert[u / kG1Units], gg = u % kG1Units;
                const int blk = gg / (kBlock / kG1Cols) + (lane >= kG1Steps ? kInter / kBlock : 0);
                const int kb = hw + kHalfWarps * (lane % kG1Steps);
                v = __ldg(a.s1 + ((size_t)e * (kGemm1Out / kBlock) + blk) * kHiddenBlocks + kb);
            }
            return v;
        };
        float sc_cur = 0.0f, sc_next = unit_scales(u1_begin);
        for (int s = 0; s < S1 && ok; ++s) {
            const int u = u1_begin + s / kG1Steps, i = s % kG1Steps;
            if (i == 0) {   // a new unit
                ai = u / kG1Units;
                g = u % kG1Units;
                m = sh->act_m[ai];
                sc_cur = sc_next;
                sc_next = unit_scales(u + 1);
                acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            }
            const int kb = hw + kHalfWarps * i;
            const float sl = __shfl_sync(0xffffffffu, sc_cur, i), sg = __shfl_sync(0xffffffffu, sc_cur, kG1Steps + i);
            const int tok = sh->act_tok[ai][r < m ? r : 0];
            const uint8_t* wst = acquire();
            if (!ok) break;
            float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            mma_block(raw, wst + r * kStepStride + hw * kBlock + 16 * c, sh->rows + tok * kHidStride + kb * kBlock + 16 * c);
            release();
            if (producer && s + kRing < S1 + S2) {
                // phase-2 steps may be issued from here on: their slots were phase-1 slots that are now free
                if (!issue(s + kRing)) { ok = false; }
            }
            const int t0 = sh->act_tok[ai][2 * c < m ? 2 * c : 0], t1 = sh->act_tok[ai][2 * c + 1 < m ? 2 * c + 1 : 0];
            const float sa0 = sh->hid_scale[t0][kb], sa1 = sh->hid_scale[t1][kb];
            acc[0] = fmaf(raw[0], sa0 * sl, acc[0]);
            acc[1] = fmaf(raw[1], sa1 * sl, acc[1]);
            acc[2] = fmaf(raw[2], sa0 * sg, acc[2]);
            acc[3] = fmaf(raw[3], sa1 * sg, acc[3]);
            if (i == kG1Steps - 1) {   // the unit is complete: add the eight warps' partial sums
                float* red = &sh->red[half][u & 1][0][0];
                *reinterpret_cast<float4*>(red + hw * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                named_bar_sync(bar_id, kHalfThreads);
                if (htid < 64) {
                    const int l = htid & 31, jj = htid >> 5;
                    float lin = 0.0f, gate = 0.0f;
#pragma unroll
                    for (int w = 0; w < kHalfWarps; ++w) {
                        lin += red[w * 128 + l * 4 + jj];
                        gate += red[w * 128 + l * 4 + 2 + jj];
                    }
                    const int slot = 2 * (l & 3) + jj, col = g * kG1Cols + (l >> 2);
                    if (slot < m) {
                        const float x1 = round_bf16(lin), x2 = round_bf16(gate);
                        const float silu = a.silu_exact ? x2 / (1.0f + __expf(-x2))
                                                        : x2 * (0.5f * (x2 * rsqrtf(fmaf(x2, x2, 4.0f)) + 1.0f));
                        act[(size_t)(sh->act_row0[ai] + slot) * kInter + col] = silu * x1;
                    }
                }
            }
        }
    }
    if (producer && S1 == 0 && ok) {   // nothing to do in phase 1: start phase 2's first steps now
        for (int s = issued; s < kRing && s < S2 && ok; ++s) ok = issue(s);
    }

    // A half that gave up on a wait still lets its bulk copies land before the CTA may exit.
    auto give_up = [&]() {
        atomicCAS(&ws.ctrl->status, kStatusOk, kStatusDecodeTimeout);
        sh->abort = 1;
        if (producer) {
            for (int g = consumed; g < issued; ++g) {
                const uint32_t bar = smem_u32(&sh->full_bar[half][g & (kRing - 1)]);
                const uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(bar, (uint32_t)((g / kRing) & 1)) && global_timer_ns() - t0 < kWaitLimitNs) {}
            }
        }
    };

    // ------------------------------------------------------------------ phase 2: requant + GEMM2
    stamp(2);
    if (!ok) give_up();
    if (!grid_barrier(&ws.ctrl->dec_count, ws.ctrl, sh)) {
        if (ok) give_up();
        return;
    }
    stamp(3);
    {
        uint8_t* a2rows = sh->rows + half * (kDecodeMaxTokens * kA2Stride);
        float(*a2s)[kInterBlocks] = sh->a2_scale[half];
        int staged = -1, ai = 0, hg = 0, m = 0;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        auto unit_scales2 = [&](int u) -> float {   // lanes 0 and 1: this warp's two K blocks, one unit ahead
            float v = 0.0f;
            if (u < u2_end && lane < kG2Steps) {
                const int e = sh->act_expert[u / kG2Units], hh = u % kG2Units;
                v = __ldg(a.s2 + ((size_t)e * kHiddenBlocks + hh / (kBlock / kG2Cols)) * kInterBlocks + hw + kHalfWarps * lane);
            }
            return v;
        };
        float sc_cur = 0.0f, sc_next = unit_scales2(u2_begin);
        for (int s = 0; s < S2 && ok; ++s) {
            const int u = u2_begin + s / kG2Steps, i = s % kG2Steps;
            if (i == 0) {
                ai = u / kG2Units;
                hg = u % kG2Units;
                m = sh->act_m[ai];
                if (ai != staged) {
                    named_bar_sync(bar_id, kHalfThreads);   // the half is done with the previous expert's rows
                    // 1x128 requantisation of the expert's rows, as in the staged GEMM1 epilogue:
                    // scale = amax / 448 (1 if the block is zero), payload e4m3(v * (1 / scale))
                    for (int item = hw; item < m * kInterBlocks; item += kHalfWarps) {
                        const int slot = item / kInterBlocks, ib = item % kInterBlocks;
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(
                            act + (size_t)(sh->act_row0[ai] + slot) * kInter + ib * kBlock) + lane);
                        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                        const float sc = amax > 0.0f ? amax / 448.0f : 1.0f;
                        const float inv = 1.0f / sc;
                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x * inv, v.y * inv), __NV_SATFINITE, __NV_E4M3);
                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z * inv, v.w * inv), __NV_SATFINITE, __NV_E4M3);
                        *reinterpret_cast<uint32_t*>(a2rows + slot * kA2Stride + ib * kBlock + lane * 4) = lo | (hi << 16);
                        if (lane == 0) a2s[slot][ib] = sc;
                    }
                    named_bar_sync(bar_id, kHalfThreads);
                    staged = ai;
                }
                sc_cur = sc_next;
                sc_next = unit_scales2(u + 1);
                acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            }
            const int kb = hw + kHalfWarps * i;
            const float sw = __shfl_sync(0xffffffffu, sc_cur, i);
            const uint8_t* wst = acquire();
            if (!ok) break;
            float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            mma_block(raw, wst + r * kStepStride + hw * kBlock + 16 * c, a2rows + r * kA2Stride + kb * kBlock + 16 * c);
            release();
            if (producer && s + kRing < S2) {
                if (!issue(S1 + s + kRing)) { ok = false; }
            }
            const float sa0 = a2s[2 * c][kb] * sw, sa1 = a2s[2 * c + 1][kb] * sw;
            acc[0] = fmaf(raw[0], sa0, acc[0]);
            acc[1] = fmaf(raw[1], sa1, acc[1]);
            acc[2] = fmaf(raw[2], sa0, acc[2]);
            acc[3] = fmaf(raw[3], sa1, acc[3]);
            if (i == kG2Steps - 1) {
                float* red = &sh->red[half][u & 1][0][0];
                *reinterpret_cast<float4*>(red + hw * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                named_bar_sync(bar_id, kHalfThreads);
                if (htid < 128) {
                    const int l = htid >> 2, q = htid & 3;
                    const int slot = 2 * (l & 3) + (q & 1), hrow = hg * kG2Cols + (l >> 2) + 8 * (q >> 1);
                    float sum = 0.0f;
#pragma unroll
                    for (int w = 0; w < kHalfWarps; ++w) sum += red[w * 128 + l * 4 + q];
                    if (slot < m) ws.y[(size_t)(sh->act_row0[ai] + slot) * kHidden + hrow] = __float2bfloat16_rn(sum);
                }
            }
        }
    }
    if (!ok) give_up();

    // ------------------------------------------------------------------ phase 3: weighted combine
    stamp(4);
    if (!grid_barrier(&ws.ctrl->dec_phase, ws.ctrl, sh)) return;
    if (blockIdx.x == 0 && tid == 0) ws.ctrl->dec_count = 0;   // everybody has left the first barrier
    stamp(5);
    {
        constexpr int kChunks = kHidden / 8;   // 16-byte chunks of a row
        for (int i = blockIdx.x * kDecThreads + tid; i < T * kChunks; i += gridDim.x * kDecThreads) {
            const int t = i / kChunks, ch = i % kChunks;
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
            const int np = sh->pair_count[t];
            for (int p = 0; p < np; ++p) {
                const float w = sh->pair_w[t][p];
                const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(ws.y + (size_t)sh->pair_row[t][p] * kHidden) + ch);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h2[j]);
                    acc[2 * j] += f.x * w;
                    acc[2 * j + 1] += f.y * w;
                }
            }
            uint4 packed;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            reinterpret_cast<uint4*>(a.out + (size_t)t * kHidden)[ch] = packed;
        }
    }
    stamp(6);
}

}  // namespace

int decode_max_ctas_per_sm()
{
    if (cudaFuncSetAttribute(decode_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)sizeof(DecodeShared)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_layer_kernel, kDecThreads, sizeof(DecodeShared)) !=
        cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

cudaError_t launch_decode_layer(const DecodeArgs& args, const void* tmap_w1, const void* tmap_w2, const Workspace& ws,
                                int num_ctas, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_ctas);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = sizeof(DecodeShared);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident: the grid barriers need it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_layer_kernel, args, *static_cast<const CUtensorMap*>(tmap_w1),
                              *static_cast<const CUtensorMap*>(tmap_w2), ws);
}

}  // namespace moe
