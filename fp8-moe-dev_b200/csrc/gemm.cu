// Stage 4 and 5 of the layer: the two FP8 block-scaled grouped GEMMs as persistent,
// warp-specialised tcgen05 kernels.
//
//   GEMM1  D[m, 0:4096] = sum_kb (A1[m, kb] . W1[e, :, kb]^T) * (sA1[kb, m] * sW1[e, n/128, kb])
//          fused epilogue: bf16 rounding of D, SwiGLU (x1 = D[:, n], x2 = D[:, 2048 + n]),
//          per-row 1x128 absmax, e4m3 requantisation -> A2, sA2.
//   GEMM2  Y[m, 0:7168] = sum_kb (A2[m, kb] . W2[e, :, kb]^T) * (sA2[kb, m] * sW2[e, h/128, kb]) -> bf16
//
// The arithmetic (what is accumulated in fp32, where bf16/e4m3 rounding happens) follows
// the reference's readable statement of the same math: kernel/moe_fp8.cu:1239-1312 (GEMM1),
// :1801-1837 (SwiGLU + requant), :2055-2110 (GEMM2).  The reference executes it with a
// CUTLASS grouped GEMM or closed TRTLLM cubins plus separate SwiGLU kernels; this file
// replaces all of them.
//
// Structure of one CTA (384 threads, one CTA per SM, 128 x 256 output tile):
//   warp 0      TMA producer: 128x128 B A tile + 256x128 B weight tile per 128-wide K block,
//               3-stage shared-memory ring (4 in the split-K kernel), SWIZZLE_128B, one mbarrier pair per stage
//   warp 1      MMA issuer: 4 x tcgen05.mma (M128 N256 K32, e4m3 -> fp32) per K block into one
//               of two 256-column TMEM accumulator stages, overwrite mode on the first
//   warp 2      TMEM allocation / release
//   warps 4-11  promotion: after each K block, tcgen05.ld of the raw block product, multiply by
//               the row scale x weight-block scale, add into fp32 registers (the scales are
//               arbitrary fp32 values, so the block-scaled MMA kinds cannot be used); each thread
//               owns one row and 128 of the tile's 256 columns.  When a tile's K loop ends they
//               round the accumulators to bf16 into a 64 KB shared-memory tile and go straight on
//               to the next tile's K loop
//   warps 2-3   tile epilogue, off the promotion warps' critical path: from the bf16 tile either
//               SwiGLU + 1x128 requantisation + stores (GEMM1, a warp per row, the row's 128
//               output bytes in one coalesced store) or four TMA tile stores (GEMM2)
// (The split-K instantiation for batches of at most four tokens keeps the epilogue in the
// promotion warps: its tiles hold at most four rows.)
// Every mbarrier wait is bounded; a wait that runs out sets the CTA's abort flag, all roles
// unwind, TMEM is released and the error is reported through Control::status.
#include <cuda.h>
#include <cuda_fp8.h>

#include "layer.cuh"
#include "ptx.cuh"

namespace moe {

constexpr int kGemmThreads = 384;
constexpr int kTileN = 256;
constexpr int kATileBytes = kTileM * kBlock;   // 16384
constexpr int kBTileBytes = kTileN * kBlock;   // 32768
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kTmemCols = 512;
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;

constexpr int kSplitKMaxRows = 4;    // split-K is used for batches of at most this many tokens
constexpr int kSplitKMaxSplit = 14;  // 56 K blocks / 4

static_assert(kHiddenBlocks / 4 <= kSplitKMaxSplit, "split-K register array too small");

constexpr int kMaxStages = 4;
struct GemmShared {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t amax_bar[2];
    uint64_t splitk_bar;
    uint64_t tile_full;    // the bf16 tile in shared memory is complete (8 promotion warps arrive)
    uint64_t tile_empty;   // the epilogue warps are done with it
    uint32_t tmem_base;
    int abort;
    int splitk_last;
};
// What follows the barriers depends on the instantiation: GEMM1 and the split-K kernels keep
// small exchange arrays there, the plain GEMM2 its output staging for TMA stores.
struct GemmScratch {
    alignas(16) float splitk_sum[kSplitKMaxRows][256];   // read and written as float4
    float amax[2][2][kTileM];
};
// The finished tile on its way to the epilogue warps: 128 rows x 256 bf16 columns as four panels of
// 64 columns.  A panel is 128 rows of 128 bytes in the 128-byte swizzle (16-byte chunk index XOR
// row mod 8): what a TMA tile store with SWIZZLE_128B reads, and conflict-free both for the
// promotion threads (one row each) and for the epilogue warps (one row per warp).
constexpr int kPanelCols = 64;
constexpr int kPanelBytes = kTileM * kPanelCols * 2;                // 16 KB
constexpr int kTilePanels = kTileN / kPanelCols;                    // 4
constexpr int kTileStageBytes = kTilePanels * kPanelBytes;          // 64 KB
constexpr size_t kGemmCoreBytes = 1024;                             // GemmShared, padded: the panels want 1 KB alignment
static_assert(sizeof(GemmShared) <= kGemmCoreBytes, "barrier block grew");

// Operand ring depth: four stages for the split-K kernel, three where 64 KB go to the tile hand-off.
template <bool SPLITK>
__host__ __device__ constexpr int gemm_stages() { return SPLITK ? 4 : 3; }

template <int MODE, bool SPLITK>
constexpr size_t gemm_smem_bytes() {
    return 1024 + (size_t)gemm_stages<SPLITK>() * kStageBytes + kGemmCoreBytes +
           (SPLITK ? sizeof(GemmScratch) : (size_t)kTileStageBytes);
}
static_assert(gemm_smem_bytes<2, false>() <= 227 * 1024 && gemm_smem_bytes<1, true>() <= 227 * 1024, "shared memory");
// Batches of at most 64 tokens: an expert has at most 64 rows, so the activation box is 64 rows high (8 KB instead
// of 16 KB per stage; the MMAs still multiply 128 rows, the upper 64 read whatever follows and are never stored)
// and the room goes to a fourth operand stage: 128 KB instead of 96 KB of weights in flight per SM, which is what
// a batch that only streams weights wants.
constexpr int kSmallATileBytes = kATileBytes / 2;
constexpr int kSmallAStages = 4;
constexpr int kSmallAMaxTokens = 64;
constexpr size_t kSmallASmemBytes = 1024 + (size_t)kSmallAStages * (kSmallATileBytes + kBTileBytes) + kGemmCoreBytes + kTileStageBytes;
static_assert(kSmallASmemBytes <= 227 * 1024, "shared memory");

struct TileCoord {
    int e, n, row0, rows;
};

// Tile id -> (expert, n tile, first packed row, valid rows).  Tiles of one expert are
// numbered n-major / m-minor so that CTAs working on neighbouring ids share a weight tile.
__device__ __forceinline__ TileCoord decode_tile(const Workspace& ws, int id, int n_tiles_n) {
    // one 16-byte record per tile: {expert, first tile of the expert, its tile count, its rows}
    const int4 info = ws.tile_info[id / n_tiles_n];
    const int local = id - info.y * n_tiles_n;
    const int n = local / info.z;
    const int j = local - n * info.z;
    const int left = info.w - j * kTileM;
    TileCoord c;
    c.e = info.x;
    c.n = n;
    c.row0 = (info.y + j) * kTileM;
    c.rows = left < kTileM ? left : kTileM;
    return c;
}

// Work units.  Normally one unit = one tile over the whole K range.  When there are at most
// half as many tiles as CTAs (decode-sized batches) every tile is cut into `split` K ranges so
// that all SMs stream weights; the partial tiles are summed by the last unit to finish.
struct UnitPlan {
    int units, split;
};
template <bool SPLITK>
__device__ __forceinline__ UnitPlan plan_units(int KBLOCKS, int total_tiles, int num_ctas) {
    UnitPlan p;
    p.split = 1;
    if (SPLITK && total_tiles > 0 && total_tiles < num_ctas) {
        // rounds x (K blocks per unit + reduction overhead, about six K blocks' worth), units capped
        // by the scratch slots; ties keep the smaller split
        int best = KBLOCKS;
        for (int s = 2; s <= KBLOCKS / 4 && s <= kSplitKMaxSplit && total_tiles * s <= kSplitKSlots; ++s) {
            const int rounds = (total_tiles * s + num_ctas - 1) / num_ctas;
            const int cost = rounds * ((KBLOCKS + s - 1) / s + 6);
            if (cost < best) { best = cost; p.split = s; }
        }
    }
    p.units = total_tiles * p.split;
    return p;
}
// K-block range [kb0, kb1) of split `s` out of `split`
__device__ __forceinline__ void unit_range(int KBLOCKS, int s, int split, int& kb0, int& kb1) {
    kb0 = (KBLOCKS * s) / split;
    kb1 = (KBLOCKS * (s + 1)) / split;
}

// Split-K: sums the partial rows of one tile over its `split` units into shared memory.  Called by
// the 256 promotion threads of the last unit to finish; thread `et` owns one float4 of the
// (kSplitKMaxRows x 256) block, all splits' loads are in flight together and are added in split
// order.  Kept out of line so that its registers do not weigh on the K loop.
__device__ __noinline__ void splitk_sum_partials(const float* partial, float* sum_smem, int tile_id, int split,
                                                 int rows, int et)
{
    const int r = et >> 6, c4 = et & 63;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) {
        const float4* src =
            reinterpret_cast<const float4*>(partial + ((size_t)(tile_id * split) * kSplitKMaxRows + r) * 256) + c4;
        float4 v[kSplitKMaxSplit];
#pragma unroll
        for (int sp = 0; sp < kSplitKMaxSplit; ++sp)
            if (sp < split) v[sp] = __ldcg(src + (size_t)sp * (kSplitKMaxRows * 256 / 4));
#pragma unroll
        for (int sp = 0; sp < kSplitKMaxSplit; ++sp)
            if (sp < split) { sum.x += v[sp].x; sum.y += v[sp].y; sum.z += v[sp].z; sum.w += v[sp].w; }
    }
    reinterpret_cast<float4*>(sum_smem)[et] = sum;
}

// tcgen05.wait::ld with the destination registers as in/out operands, so that the
// compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tmem_ld_wait2(uint32_t (&a)[32], uint32_t (&b)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                   "+r"(a[8]), "+r"(a[9]), "+r"(a[10]), "+r"(a[11]), "+r"(a[12]), "+r"(a[13]), "+r"(a[14]),
                   "+r"(a[15]), "+r"(a[16]), "+r"(a[17]), "+r"(a[18]), "+r"(a[19]), "+r"(a[20]), "+r"(a[21]),
                   "+r"(a[22]), "+r"(a[23]), "+r"(a[24]), "+r"(a[25]), "+r"(a[26]), "+r"(a[27]), "+r"(a[28]),
                   "+r"(a[29]), "+r"(a[30]), "+r"(a[31]), "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]),
                   "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]), "+r"(b[8]), "+r"(b[9]), "+r"(b[10]),
                   "+r"(b[11]), "+r"(b[12]), "+r"(b[13]), "+r"(b[14]), "+r"(b[15]), "+r"(b[16]), "+r"(b[17]),
                   "+r"(b[18]), "+r"(b[19]), "+r"(b[20]), "+r"(b[21]), "+r"(b[22]), "+r"(b[23]), "+r"(b[24]),
                   "+r"(b[25]), "+r"(b[26]), "+r"(b[27]), "+r"(b[28]), "+r"(b[29]), "+r"(b[30]), "+r"(b[31])
                 :
                 : "memory");
}

// acc[OFF + j] += raw[j] * s for 32 accumulator columns.  PACKED uses the two-wide fp32 FMA of
// sm_100: same IEEE result per element and the same FMA-pipe time, but half the issue slots.
// That matters because the MMA-issuing thread shares its scheduler with two of these warps: long
// bursts of scalar FMAs starve it (measured: 728 -> 592 cycles per K block in an isolated
// two-stage pipeline when the promotion uses the packed form).
template <int OFF, bool PACKED>
__device__ __forceinline__ void promote32(float (&acc)[128], const uint32_t (&r)[32], float s) {
    if (PACKED) {
        const float2 s2 = make_float2(s, s);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const float2 d = __ffma2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), s2,
                                        make_float2(acc[OFF + j], acc[OFF + j + 1]));
            acc[OFF + j] = d.x;
            acc[OFF + j + 1] = d.y;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[OFF + j] = fmaf(__uint_as_float(r[j]), s, acc[OFF + j]);
    }
}

// Scale load that the compiler cannot sink towards its use: issued (as volatile asm) one
// K block ahead, so that its L2 latency is covered by the whole block's promotion work.
__device__ __forceinline__ float ld_scale_early(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float round_bf16(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

// MODE 1: GEMM1 + SwiGLU + requant (K = 7168).  MODE 2: GEMM2 -> bf16 Y (K = 2048).
// SPLITK compiles the split-K path in; the plain instantiation carries none of its code
// (having it in the main kernel cost 5-7 % on mid-size batches through register pressure).
// GENERIC takes hidden / intermediate from Workspace::geo instead of the reference's 7168 / 2048
// (hidden a multiple of 256, intermediate of 128, at most 64 K blocks each); the reference's
// geometry keeps its compile-time instantiation.
template <int MODE, bool SPLITK, bool GENERIC = false, bool SMALLA = false>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(
    const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
    const __grid_constant__ CUtensorMap tmap_out, Workspace ws, const float2* __restrict__ w_scale_packed, int silu_exact)
{
    static_assert(!(GENERIC && SPLITK), "the split-K kernel exists for the reference's geometry only");
    const int hidden = GENERIC ? ws.geo.hidden : kHidden;
    const int inter = GENERIC ? ws.geo.inter : kInter;
    const int kKBlocks = ((MODE == 1) ? hidden : inter) / kBlock;                   // 56 / 16
    const int kTilesN = (MODE == 1) ? (inter / kBlock) : (hidden / kTileN);         // 16 / 28
    static_assert(!(SMALLA && (SPLITK || GENERIC)), "the 64-row activation box is a variant of the plain kernel");
    constexpr int kStages = SMALLA ? kSmallAStages : gemm_stages<SPLITK>();
    constexpr int kABytes = SMALLA ? kSmallATileBytes : kATileBytes;
    constexpr int kStageSize = kABytes + kBTileBytes;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    GemmShared* sh = reinterpret_cast<GemmShared*>(smem_raw + (base - raw_addr) + (size_t)kStages * kStageSize);
    uint8_t* after_core = reinterpret_cast<uint8_t*>(sh) + kGemmCoreBytes;   // 1 KB aligned
    GemmScratch* sc = reinterpret_cast<GemmScratch*>(after_core);           // split-K kernels only
    (void)sc;
    uint8_t* tile_stage = after_core;                                       // others: the bf16 tile (64 KB)
    (void)tile_stage;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&sh->acc_full[s]), 1);
            mbar_init(smem_u32(&sh->acc_empty[s]), kEpilogueWarps);
            mbar_init(smem_u32(&sh->amax_bar[s]), kEpilogueThreads);
        }
        mbar_init(smem_u32(&sh->splitk_bar), kEpilogueThreads);
        mbar_init(smem_u32(&sh->tile_full), kEpilogueWarps);
        mbar_init(smem_u32(&sh->tile_empty), MODE == 1 ? 2 : 1);
        sh->abort = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (MODE == 2 && !SPLITK) prefetch_tmap(&tmap_out);
    }
    // Everything above is independent of earlier kernels; from here on their results are read.
    pdl_wait();
    const int total_tiles = ws.num_tiles[0] * kTilesN;
    const UnitPlan plan = plan_units<SPLITK>(kKBlocks, total_tiles, (int)gridDim.x);
    if ((int)blockIdx.x >= plan.units) return;  // nothing for this CTA: leave before touching TMEM
    if (warp == 2) {
        tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    volatile int* abort_flag = &sh->abort;

    if (warp < 4) {
        // register split: 56 per thread for the producer warpgroup, 224 for the two promotion
        // warpgroups (128 * 56 + 256 * 224 <= 64 K registers per SM)
        setmaxnreg_dec<56>();
        if (warp == 0 && lane == 0) {
            // ------------------------------------------------------------ TMA producer
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < plan.units; u += gridDim.x) {
                const TileCoord tc = decode_tile(ws, u / plan.split, kTilesN);
                int kb0, kb1;
                unit_range(kKBlocks, u % plan.split, plan.split, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!mbar_wait(smem_u32(&sh->empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t full = smem_u32(&sh->full[s]);
                    mbar_expect_tx(full, kStageSize);
                    const uint32_t a_dst = base + s * kStageSize;
                    const uint32_t b_dst = a_dst + kABytes;
                    tma_load_2d(a_dst, &tmap_a, full, kb * kBlock, tc.row0);
                    if (ws.w_tiled) {
                        // tile-ordered copy of the weights: the operand of (expert, n tile, K block) is one
                        // contiguous 32 KB piece
                        tma_load_2d(b_dst, &tmap_b, full, 0, ((tc.e * kTilesN + tc.n) * kKBlocks + kb) * kTileN);
                    } else if (MODE == 1) {
                        tma_load_3d(b_dst, &tmap_b, full, kb * kBlock, tc.n * kBlock, tc.e);
                        tma_load_3d(b_dst + kBTileBytes / 2, &tmap_b, full, kb * kBlock, inter + tc.n * kBlock, tc.e);
                    } else {
                        tma_load_3d(b_dst, &tmap_b, full, kb * kBlock, tc.n * kTileN, tc.e);
                    }
                }
            }
            if (!ok) {
                // Leave only after this thread's copies in flight have landed (bounded).
                const uint32_t pending = it < (uint32_t)kStages ? it : (uint32_t)kStages;
                for (uint32_t j = 1; j <= pending; ++j) {
                    const uint32_t jt = it - j;
                    const uint32_t s = jt % kStages;
                    const uint32_t ph = (jt / kStages) & 1u;
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(smem_u32(&sh->full[s]), ph)) {
                        if (global_timer_ns() - t0 > kWaitLimitNs / 4) break;
                    }
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ------------------------------------------------------------ MMA issuer
            const uint32_t idesc = make_idesc_e4m3(kTileM, kTileN);
            uint32_t it = 0;
            bool ok = true;
            bool next_full_ready = false;
            for (int u = blockIdx.x; ok && u < plan.units; u += gridDim.x) {
                int kb0, kb1;
                unit_range(kKBlocks, u % plan.split, plan.split, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t as = it & 1u;
                    const uint32_t aph = (it >> 1) & 1u;
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    // The operand stage is normally long since loaded; its barrier was already
                    // probed while the previous block's MMAs ran (next_full_ready), which keeps
                    // that probe's latency off the release -> issue chain below.
                    if (!next_full_ready && !mbar_wait(smem_u32(&sh->full[s]), ph, abort_flag)) { ok = false; break; }
                    const uint32_t a_addr = base + s * kStageSize;
                    const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
                    const uint64_t bdesc = make_kmajor_sw128_desc(a_addr + kABytes);
                    const uint32_t d = tmem_base + as * kTileN;
                    if (!mbar_wait(smem_u32(&sh->acc_empty[as]), aph ^ 1u, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < kBlock / 32; ++k) {
                        // 32 e4m3 = 32 B along K inside the 128 B swizzled row: +2 in 16 B units.
                        umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&sh->empty[s]));
                    tc_commit(smem_u32(&sh->acc_full[as]));
                    {
                        const uint32_t nit = it + 1;
                        next_full_ready = mbar_try_wait(smem_u32(&sh->full[nit % kStages]), (nit / kStages) & 1u);
                    }
                }
            }
        } else if (!SPLITK && warp >= 2) {
            // ------------------------------------------------------------ tile epilogue
            // Runs one tile behind the promotion warps, while they are in the next tile's K loop.
            const int ew = warp - 2;
            uint32_t ti = 0;
            bool ok = MODE == 1 || ew == 0;   // GEMM2's stores need one thread only
            for (int u = blockIdx.x; ok && u < plan.units; u += gridDim.x, ++ti) {
                const TileCoord tc = decode_tile(ws, u, kTilesN);
                ok = mbar_wait(smem_u32(&sh->tile_full), ti & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (MODE == 2) {
                    // Y: four 128-row x 64-column tile stores.  Rows past the tile's valid rows land in
                    // the expert's padding, which nobody reads.
                    if (lane == 0) {
#pragma unroll
                        for (int p = 0; p < kTilePanels; ++p)
                            tma_store_2d(&tmap_out, smem_u32(tile_stage + p * kPanelBytes), tc.n * kTileN + p * kPanelCols,
                                         tc.row0);
                        bulk_commit_group();
                        bulk_wait_group_read<0>();   // the panels have been read: they may be overwritten
                        mbar_arrive(smem_u32(&sh->tile_empty));
                    }
                    __syncwarp();
                } else {
                    // GEMM1: D was rounded to bf16 on its way here (the reference materialises it in
                    // bf16).  Of each row, lane l owns SwiGLU columns 4l..4l+3 of the tile's
                    // 128-column block: x1 from panels 0-1 (linear branch), x2 from panels 2-3 (gated
                    // branch); v = silu(x2) * x1 in fp32, row absmax by shuffles, scale = amax / 448
                    // (1 for an all-zero block), e4m3 codes -> 128 coalesced bytes per row.
                    const int r_begin = ew * (kTileM / 2);
                    const int r_end = tc.rows < (ew + 1) * (kTileM / 2) ? tc.rows : (ew + 1) * (kTileM / 2);
                    const uint32_t pan = (uint32_t)(lane >> 4) * kPanelBytes;
                    const uint32_t chunk = (uint32_t)(lane & 15) >> 1, sub = (uint32_t)(lane & 1) * 8u;
                    // The generic instantiation takes four rows per pass, so that their shared-memory loads,
                    // shuffles and conversions overlap: with few K blocks per tile (a small hidden size) the
                    // epilogue warps set GEMM1's pace.  With the reference's 56 K blocks they have time to
                    // spare, and one row per pass leaves more issue slots to the promotion warps they share
                    // their schedulers with (measured: four rows per pass cost 1.3 % there).
                    constexpr int kRowsPerPass = GENERIC ? 4 : 1;
                    for (int r0 = r_begin; r0 < r_end; r0 += kRowsPerPass) {
                        float v[kRowsPerPass][4], amax[kRowsPerPass];
#pragma unroll
                        for (int u4 = 0; u4 < kRowsPerPass; ++u4) {
                            const int r = r0 + u4;   // < 128: rows past r_end hold stale data and are not stored
                            const uint8_t* src = tile_stage + pan + r * 128 + ((chunk ^ (uint32_t)(r & 7)) << 4) + sub;
                            const uint2 l1 = *reinterpret_cast<const uint2*>(src);
                            const uint2 l2 = *reinterpret_cast<const uint2*>(src + 2 * kPanelBytes);
                            const float x1[4] = {__uint_as_float(l1.x << 16), __uint_as_float(l1.x & 0xffff0000u),
                                                 __uint_as_float(l1.y << 16), __uint_as_float(l1.y & 0xffff0000u)};
                            const float x2[4] = {__uint_as_float(l2.x << 16), __uint_as_float(l2.x & 0xffff0000u),
                                                 __uint_as_float(l2.y << 16), __uint_as_float(l2.y & 0xffff0000u)};
                            amax[u4] = 0.0f;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float silu = silu_exact ? x2[j] / (1.0f + __expf(-x2[j]))
                                                              : x2[j] * (0.5f * (x2[j] * rsqrtf(fmaf(x2[j], x2[j], 4.0f)) + 1.0f));
                                v[u4][j] = silu * x1[j];
                                amax[u4] = fmaxf(amax[u4], fabsf(v[u4][j]));
                            }
                        }
#pragma unroll
                        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                            for (int u4 = 0; u4 < kRowsPerPass; ++u4) amax[u4] = fmaxf(amax[u4], __shfl_xor_sync(0xffffffffu, amax[u4], off));
                        }
#pragma unroll
                        for (int u4 = 0; u4 < kRowsPerPass; ++u4) {
                            const int r = r0 + u4;
                            if (r < r_end) {
                                const float scale = (amax[u4] > 0.0f) ? (amax[u4] / 448.0f) : 1.0f;
                                const float inv_scale = 1.0f / scale;
                                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[u4][0] * inv_scale, v[u4][1] * inv_scale),
                                                                             __NV_SATFINITE, __NV_E4M3);
                                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[u4][2] * inv_scale, v[u4][3] * inv_scale),
                                                                             __NV_SATFINITE, __NV_E4M3);
                                const int grow = tc.row0 + r;
                                reinterpret_cast<uint32_t*>(ws.a2 + (size_t)grow * inter + tc.n * kBlock)[lane] = lo | (hi << 16);
                                if (lane == 0) ws.sfa2[(size_t)tc.n * ws.m_cap + grow] = scale;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sh->tile_empty));
                }
            }
            if (MODE == 2 && ew == 0 && lane == 0) bulk_wait_group<0>();   // stores performed before the CTA leaves
        }
    } else {
        // ---------------------------------------------------------------- promotion + epilogue
        setmaxnreg_inc<224>();
        const int ew = warp - 4;
        const int h = ew >> 2;       // which 128 of the tile's 256 accumulator columns
        const int q = warp & 3;      // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        // accumulator column of the four 32-column chunks this thread promotes: columns 64h..64h+63 of the
        // tile's first 128-column half and 128+64h..128+64h+63 of its second (GEMM1: linear and gated branch)
        const uint32_t c0 = (uint32_t)(64 * h);
        const uint32_t c1 = c0 + 32;
        const uint32_t c2 = (uint32_t)(128 + 64 * h);
        const uint32_t c3 = c2 + 32;

        uint32_t it = 0;
        uint32_t tile_iter = 0;
        bool ok = true;
        uint32_t splitk_uses = 0;
        for (int u = blockIdx.x; ok && u < plan.units; u += gridDim.x) {
            const int tile_id = u / plan.split;
            const TileCoord tc = decode_tile(ws, tile_id, kTilesN);
            int kb0, kb1;
            unit_range(kKBlocks, u % plan.split, plan.split, kb0, kb1);
            const int grow = tc.row0 + row;
            const float* sfa = ((MODE == 1) ? ws.sfa1 : ws.sfa2) + grow;
            // The tile's weight-block scales for all K blocks, from the pre-laid-out copy (one float2 per
            // K block, see repack_weight_scales_kernel): lane l keeps the entries of K blocks l and l + 32,
            // a K block's pair then comes from a shuffle instead of two dependent global loads.
            const float2* sw_tile = w_scale_packed + ((size_t)tc.e * kTilesN + tc.n) * kKBlocks;
            const float2 sw_a = (lane < kKBlocks) ? __ldg(sw_tile + lane) : make_float2(0.0f, 0.0f);
            const float2 sw_b = (kKBlocks > 32 && lane + 32 < kKBlocks) ? __ldg(sw_tile + lane + 32) : make_float2(0.0f, 0.0f);
            // .x scales the tile's first 128-column block (GEMM1: linear branch), .y its second (gated branch)
            const float mine_a = sw_a.x, other_a = sw_a.y;
            const float mine_b = sw_b.x, other_b = sw_b.y;
            float acc[128];
#pragma unroll
            for (int j = 0; j < 128; ++j) acc[j] = 0.0f;
            const bool warp_has_rows = q * 32 < tc.rows;

            float sa_n = ld_scale_early(sfa + (size_t)kb0 * ws.m_cap);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const float lo_w = __shfl_sync(0xffffffffu, (kKBlocks > 32 && kb >= 32) ? mine_b : mine_a, kb & 31);
                const float hi_w = __shfl_sync(0xffffffffu, (kb >= 32) ? other_b : other_a, kb & 31);
                const float s_lo = sa_n * lo_w;
                const float s_hi = sa_n * hi_w;
                if (kb + 1 < kb1) sa_n = ld_scale_early(sfa + (size_t)(kb + 1) * ws.m_cap);
                const uint32_t as = it & 1u;
                const uint32_t aph = (it >> 1) & 1u;
                ok = mbar_wait(smem_u32(&sh->acc_full[as]), aph, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (!warp_has_rows) {
                    // none of this warp's 32 rows is a routed row (short expert tail): nothing to
                    // promote, release the accumulator stage at once
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[as]));
                    continue;
                }
                const uint32_t t = lane_addr + as * kTileN;
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(t + c0, r0);
                tmem_ld_32x32(t + c1, r1);
                tmem_ld_wait2(r0, r1);
                promote32<0, true>(acc, r0, s_lo);
                tmem_ld_32x32(t + c2, r0);
                promote32<32, true>(acc, r1, s_lo);
                tmem_ld_32x32(t + c3, r1);
                tmem_ld_wait2(r0, r1);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[as]));
                promote32<64, true>(acc, r0, s_hi);
                promote32<96, true>(acc, r1, s_hi);
            }
            if (!ok) break;

            if (!SPLITK) {
                // Hand the tile to the epilogue warps: accumulators rounded to bf16 (what both the
                // GEMM1 and the GEMM2 result are rounded to anyway) into the shared-memory panels, a
                // thread's first 64 columns into panel pa, its other 64 into panel pb.  The panels
                // were released a whole K loop ago, so the wait below does not block in practice.
                if (tile_iter > 0) {
                    ok = mbar_wait(smem_u32(&sh->tile_empty), (tile_iter - 1) & 1u, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                if (warp_has_rows) {
                    const int pa = h, pb = 2 + h;
                    uint8_t* ra = tile_stage + pa * kPanelBytes + row * 128;
                    uint8_t* rb = tile_stage + pb * kPanelBytes + row * 128;
                    const uint32_t sw = (uint32_t)(row & 7);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4 pk;
                        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(acc[8 * c + 2 * i], acc[8 * c + 2 * i + 1]);
                        *reinterpret_cast<uint4*>(ra + (((uint32_t)c ^ sw) << 4)) = pk;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            h2[i] = __floats2bfloat162_rn(acc[64 + 8 * c + 2 * i], acc[64 + 8 * c + 2 * i + 1]);
                        *reinterpret_cast<uint4*>(rb + (((uint32_t)c ^ sw) << 4)) = pk;
                    }
                    if (MODE == 2) fence_proxy_async_smem();   // the TMA stores read these writes
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh->tile_full));
                ++tile_iter;
                continue;
            }
            const bool valid = row < tc.rows;
            if (SPLITK && plan.split > 1) {
                // Split-K reduction (batches of at most kSplitKMaxRows tokens, so a tile has at most
                // that many routed rows).  Every unit parks its partial rows in global scratch and
                // takes a ticket; the last unit of the tile sums all partials -- one float4 per
                // thread, all splits' loads in flight together, fixed split order -- into shared
                // memory, from where the owning threads pick up their accumulators again.
                float4* mine = reinterpret_cast<float4*>(ws.splitk_partial + ((size_t)u * kSplitKMaxRows + row) * 256 +
                                                         (size_t)h * 128);
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        __stcg(mine + j, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
                    __threadfence();
                }
                const uint32_t bar = smem_u32(&sh->splitk_bar);
                mbar_arrive(bar);
                ok = mbar_wait(bar, splitk_uses & 1u, abort_flag);
                ++splitk_uses;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (threadIdx.x == 4 * 32) {
                    const int ticket = atomicAdd(&ws.ctrl->splitk_ticket[tile_id], 1);
                    const int last = (ticket == plan.split - 1) ? 1 : 0;
                    if (last) ws.ctrl->splitk_ticket[tile_id] = 0;
                    sh->splitk_last = last;
                }
                mbar_arrive(bar);
                ok = mbar_wait(bar, splitk_uses & 1u, abort_flag);
                ++splitk_uses;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (!sh->splitk_last) continue;
                __threadfence();
                splitk_sum_partials(ws.splitk_partial, &sc->splitk_sum[0][0], tile_id, plan.split, tc.rows,
                                    (int)threadIdx.x - 4 * 32);
                mbar_arrive(bar);
                ok = mbar_wait(bar, splitk_uses & 1u, abort_flag);
                ++splitk_uses;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (valid) {
                    const float4* src = reinterpret_cast<const float4*>(&sc->splitk_sum[row][h * 128]);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float4 v = src[j];
                        acc[4 * j] = v.x; acc[4 * j + 1] = v.y; acc[4 * j + 2] = v.z; acc[4 * j + 3] = v.w;
                    }
                }
            }
            if (MODE == 1) {
                // D is rounded to bf16 (the reference materialises it in bf16), then
                // v = silu(x2) * x1 in fp32, absmax over the row's 128-column block.
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const float x1 = round_bf16(acc[j]);
                    const float x2 = round_bf16(acc[64 + j]);
                    const float silu = silu_exact ? x2 / (1.0f + __expf(-x2))
                                                  : x2 * (0.5f * (x2 * rsqrtf(fmaf(x2, x2, 4.0f)) + 1.0f));
                    const float v = silu * x1;
                    acc[j] = v;
                    amax = fmaxf(amax, fabsf(v));
                }
                const uint32_t tp = tile_iter & 1u;
                sc->amax[tp][h][row] = amax;
                mbar_arrive(smem_u32(&sh->amax_bar[tp]));
                ok = mbar_wait(smem_u32(&sh->amax_bar[tp]), (tile_iter >> 1) & 1u, abort_flag);
                ++tile_iter;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const float maxv = fmaxf(amax, sc->amax[tp][h ^ 1][row]);
                const float scale = (maxv > 0.0f) ? (maxv / 448.0f) : 1.0f;
                const float inv_scale = 1.0f / scale;
                if (valid) {
                    uint4* dst = reinterpret_cast<uint4*>(ws.a2 + (size_t)grow * inter + tc.n * kBlock + 64 * h);
#pragma unroll
                    for (int v8 = 0; v8 < 2; ++v8) {
                        uint4 pk[2];
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint32_t wd[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int j = (v8 * 2 + q) * 16 + i * 4;
                                const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                                    make_float2(acc[j] * inv_scale, acc[j + 1] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                                const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                                    make_float2(acc[j + 2] * inv_scale, acc[j + 3] * inv_scale), __NV_SATFINITE, __NV_E4M3);
                                wd[i] = lo | (hi << 16);
                            }
                            pk[q] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
                        }
                        st_global_32B(dst + 2 * v8, pk[0], pk[1]);
                    }
                    if (h == 0) ws.sfa2[(size_t)tc.n * ws.m_cap + grow] = scale;
                }
            } else {
                if (valid) {
                    // acc[0..63] are columns 64h.., acc[64..127] columns 128 + 64h.. of the tile
                    uint4* dst = reinterpret_cast<uint4*>(ws.y + (size_t)grow * hidden + tc.n * kTileN + 64 * h);
#pragma unroll
                    for (int v8 = 0; v8 < 8; ++v8) {
                        uint4 pk[2];
#pragma unroll
                        for (int q2 = 0; q2 < 2; ++q2) {
                            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk[q2]);
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                h2[i] = __floats2bfloat162_rn(acc[v8 * 16 + q2 * 8 + 2 * i], acc[v8 * 16 + q2 * 8 + 2 * i + 1]);
                        }
                        st_global_32B(dst + (v8 < 4 ? 0 : 8) + 2 * v8, pk[0], pk[1]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && sh->abort != 0) {
        atomicCAS(&ws.ctrl->status, kStatusOk, MODE == 1 ? kStatusGemm1Timeout : kStatusGemm2Timeout);
    }
}

// ---------------------------------------------------------------------------------------
// Weight-scale pre-layout, run once per pair of scale tensors (the handle remembers their
// addresses): the promotion wants, per output tile and K block, the two 128x128-block scales the
// tile's 256 accumulator columns use.  In the operator's layout those lie kInterBlocks rows apart
// (GEMM1: [E, 32, 56], linear-branch block n and gated-branch block 16 + n) or in neighbouring
// rows (GEMM2: [E, 56, 16], blocks 2n and 2n + 1); here they become one float2 per (expert, tile,
// K block), the order the promotion walks.  This is the counterpart of the reference's cached
// scale transposes (kernel/moe_fp8.cu:981-994, cached per scale pointer at :3007-3014, 3501-3508).
// ---------------------------------------------------------------------------------------
__global__ void repack_weight_scales_kernel(const float* __restrict__ s1, const float* __restrict__ s2,
                                            float2* __restrict__ p1, float2* __restrict__ p2, int num_experts,
                                            Geometry geo)
{
    const int hb = geo.hidden / kBlock, ib = geo.inter / kBlock;   // 56 / 16 K blocks
    const int kN1 = ib;                    // 16 GEMM1 tiles per expert
    const int kN2 = geo.hidden / kTileN;   // 28 GEMM2 tiles per expert
    const int per1 = kN1 * hb, per2 = kN2 * ib;
    const int total = num_experts * (per1 + per2);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int e = i / (per1 + per2);
        const int r = i - e * (per1 + per2);
        if (r < per1) {
            const int n = r / hb, kb = r - n * hb;
            const float* src = s1 + ((size_t)e * (2 * kN1) + n) * hb + kb;
            p1[(size_t)e * per1 + r] = make_float2(src[0], src[(size_t)kN1 * hb]);
        } else {
            const int r2 = r - per1;
            const int n = r2 / ib, kb = r2 - n * ib;
            const float* src = s2 + ((size_t)e * hb + 2 * n) * ib + kb;
            p2[(size_t)e * per2 + r2] = make_float2(src[0], src[ib]);
        }
    }
}

size_t packed_scale_floats(int mode, int num_experts, const Geometry& geo)
{
    const size_t hb = geo.hidden / kBlock, ib = geo.inter / kBlock;
    return 2 * (size_t)num_experts * (mode == 1 ? ib * hb : (size_t)(geo.hidden / kTileN) * ib);
}

cudaError_t launch_repack_weight_scales(const float* s1, const float* s2, float* p1, float* p2, int num_experts,
                                        const Geometry& geo, cudaStream_t stream)
{
    repack_weight_scales_kernel<<<64, 256, 0, stream>>>(s1, s2, reinterpret_cast<float2*>(p1), reinterpret_cast<float2*>(p2),
                                                        num_experts, geo);
    return cudaGetLastError();
}

// Tile-ordered copy of one weight tensor: for every (expert, n tile, K block) the 256 x 128-byte
// operand the K loop loads becomes one contiguous 32 KB piece (GEMM1: 128 linear rows of the n
// tile, then its 128 gated rows), so that a TMA box reads whole DRAM pages instead of 256 pieces
// of 128 bytes that lie a weight row apart.  One warp per source row, read once front to back.
// The reference keeps such a per-pointer pre-layout of W1 (kernel/moe_fp8.cu:981-994, 3007-3014).
__global__ void __launch_bounds__(256) tile_weights_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                           int mode, int num_experts, Geometry geo)
{
    const int k_bytes = mode == 1 ? geo.hidden : geo.inter;
    const int rows = mode == 1 ? 2 * geo.inter : geo.hidden;
    const int kblocks = k_bytes / kBlock;
    const int tiles_n = rows / kTileN;
    const int lane = threadIdx.x & 31;
    const long long total_rows = (long long)num_experts * rows;
    for (long long gr = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); gr < total_rows; gr += (long long)gridDim.x * 8) {
        const int e = (int)(gr / rows);
        const int r = (int)(gr - (long long)e * rows);
        int n, in_tile;
        if (mode == 1) {
            const int half = r >= geo.inter;
            const int rr = r - half * geo.inter;
            n = rr / kBlock;
            in_tile = half * kBlock + (rr - n * kBlock);
        } else {
            n = r / kTileN;
            in_tile = r - n * kTileN;
        }
        const uint4* s4 = reinterpret_cast<const uint4*>(src + (size_t)gr * k_bytes);
        uint8_t* tile0 = dst + ((size_t)(e * tiles_n + n) * kblocks * kTileN + in_tile) * kBlock;
        for (int c = lane; c < k_bytes / 16; c += 32) {
            const int kb = c >> 3;
            *reinterpret_cast<uint4*>(tile0 + (size_t)kb * kTileN * kBlock + (c & 7) * 16) = __ldg(s4 + c);
        }
    }
}

cudaError_t launch_tile_weights(int mode, const void* src, void* dst, int num_experts, const Geometry& geo, int num_sms,
                                cudaStream_t stream)
{
    tile_weights_kernel<<<num_sms * 8, 256, 0, stream>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), mode,
                                                         num_experts, geo);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Host side: tensor maps and launch.
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// rows x K bytes (K contiguous), optionally batched over experts; box = 128 B x box_rows.
int encode_kmajor_u8_map(void* out_map, const void* base, uint64_t k_bytes, uint64_t rows, uint64_t batch,
                         uint32_t box_rows)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    CUtensorMap* m = static_cast<CUtensorMap*>(out_map);
    CUresult r;
    if (batch == 0) {
        const cuuint64_t dims[2] = {k_bytes, rows};
        const cuuint64_t strides[1] = {k_bytes};
        const cuuint32_t box[2] = {(cuuint32_t)kBlock, box_rows};
        const cuuint32_t es[2] = {1, 1};
        r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[3] = {k_bytes, rows, batch};
        const cuuint64_t strides[2] = {k_bytes, k_bytes * rows};
        const cuuint32_t box[3] = {(cuuint32_t)kBlock, box_rows, 1};
        const cuuint32_t es[3] = {1, 1, 1};
        r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

// rows x row_bytes viewed as 32-bit words, no swizzle; box = 1 KB of a row x box_rows rows
// (the decode kernel's weight steps).
int encode_rows_1k_map(void* out_map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    CUtensorMap* m = static_cast<CUtensorMap*>(out_map);
    const cuuint64_t dims[2] = {row_bytes / 4, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {256, box_rows};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

// bf16 [rows, cols] row-major output; box = 64 columns x 128 rows with the 128-byte swizzle (one panel
// of GEMM2's finished tile).
int encode_out_bf16_map(void* out_map, void* base, uint64_t cols, uint64_t rows)
{
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    CUtensorMap* m = static_cast<CUtensorMap*>(out_map);
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kPanelCols, (cuuint32_t)kTileM};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)r;
}

size_t tensor_map_bytes() { return sizeof(CUtensorMap); }

cudaError_t configure_gemm_kernels()
{
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)gemm_smem_bytes<1, false>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes<2, false>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes<1, true>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes<2, true>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes<1, false>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemm_smem_bytes<2, false>());
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<1, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmallASmemBytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_gemm_kernel<2, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmallASmemBytes);
    return e;
}

int gemm_tiles_n(int mode, const Geometry& geo) { return mode == 1 ? geo.inter / kBlock : geo.hidden / kTileN; }

cudaError_t launch_grouped_gemm(int mode, const void* tmap_a, const void* tmap_b, const void* tmap_out, const Workspace& ws,
                                const float* w_scale_packed, int silu_exact, int num_ctas, int split_k, int small_a,
                                cudaStream_t stream)
{
    const float2* w_scale = reinterpret_cast<const float2*>(w_scale_packed);
    const CUtensorMap* ma = static_cast<const CUtensorMap*>(tmap_a);
    const CUtensorMap* mb = static_cast<const CUtensorMap*>(tmap_b);
    const CUtensorMap* mo = static_cast<const CUtensorMap*>(tmap_out);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_ctas < 1 ? 1 : num_ctas);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!ws.geo.is_reference()) {
        // other geometries: the generic instantiations (no split-K form; the caller does not ask for one)
        cfg.dynamicSmemBytes = gemm_smem_bytes<1, false>();
        if (split_k) return cudaErrorInvalidValue;
        if (mode == 1) return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<1, false, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
        return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<2, false, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
    }
    if (small_a && !split_k) {
        // at most 64 tokens: tmap_a is the 64-row view of the packed activations
        cfg.dynamicSmemBytes = kSmallASmemBytes;
        if (mode == 1)
            return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<1, false, false, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
        return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<2, false, false, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
    }
    if (mode == 1) {
        cfg.dynamicSmemBytes = split_k ? gemm_smem_bytes<1, true>() : gemm_smem_bytes<1, false>();
        if (split_k) return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<1, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
        return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<1, false>, *ma, *mb, *mo, ws, w_scale, silu_exact);
    }
    cfg.dynamicSmemBytes = split_k ? gemm_smem_bytes<2, true>() : gemm_smem_bytes<2, false>();
    if (split_k) return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<2, true>, *ma, *mb, *mo, ws, w_scale, silu_exact);
    return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<2, false>, *ma, *mb, *mo, ws, w_scale, silu_exact);
}

}  // namespace moe
