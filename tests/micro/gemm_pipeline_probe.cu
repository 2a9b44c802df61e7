// Micro-benchmark of the grouped GEMM's inner pipeline on ONE SM (or one CTA on each of N SMs), without
// real data and (but for the *_tma forms) without TMA: the MMA-issuing thread, the two 256-column TMEM accumulator stages and the
// eight promotion warps with the kernel's own handshake (ptx.cuh of the package).  It reports SM cycles
// per 128-wide K block (and the wall time) for a few forms of the loop:
//   mma_only            4 x tcgen05.mma M128 N256 K32 per K block, promotion warps release the stage at once
//   mma_only_n128       the same block issued as 8 x M128 N128 K32 (what a finer accumulator split would need)
//   drain               promotion warps read the whole stage from TMEM (4 x 32 columns each), no arithmetic
//   promote_scalar      + fp32 scale-and-add with scalar FMAs
//   promote_packed      + the packed two-wide FMA the kernel uses
//   ring                + the operand ring's barrier traffic on the issuing thread, with no data behind it: a
//                       stand-in producer, the wait for a full stage (probed one block ahead, as in the kernel)
//                       and the second tcgen05.commit that frees the stage
//   ring_scales         + the kernel's per-block scale handling in the promotion warps (two shuffles, a global
//                       load issued one block ahead, two multiplies): the kernel's loop minus TMA and tiles
//   ring_scales_relayed the stage is freed by a promotion warp's plain arrive instead of a second commit
//   ring_scales_two     two MMA-issuing threads, one per accumulator stage
//   ring_scales_tma     ring_scales with a real producer: per K block one 128 x 128-byte and one 256 x 128-byte TMA
//                       box (48 KB) from a 58 MB buffer into a three-stage ring, as in the kernel; groups of six CTAs
//                       share their weight boxes, so that with many CTAs the boxes come from L2 as they do there
//   ring_scales_two_tma the same with two issuing threads
//   ring_far_tma, ring_far_two_tma     the row-scale load of the next K block reads a new line of a 7 MB array
//                       every block (an L1 miss, as in the kernel) instead of a 4 KB array
//   ring_far2_two_tma   ... issued two K blocks ahead
//   ring_farlate_tma, ring_farlate_two_tma   ... issued after the wait for the accumulator stage, not before it
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -I <package>/csrc gemm_pipeline_probe.cu
//   ring_scales_tma_m64 ring_scales_tma with M = 64 instructions
// Run:   ./a.out [ctas=1] [k_blocks=4000] [name filter]   (every wait is bounded; a failed wait ends the kernel)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"
using namespace moe;

enum : int {
    F_N128 = 1,         // 128-column MMA instructions
    F_LOADS = 2,        // promotion warps read the stage
    F_FMA_SCALAR = 4,   // ... and promote with scalar FMAs
    F_FMA_PACKED = 8,   // ... or with packed FMAs
    F_RING = 16,        // operand-ring barriers on the issuing thread
    F_SCALES = 32,      // per-block scale handling in the promotion warps
    F_RELAY = 64,       // a promotion warp frees the operand stage
    F_TWO = 128,        // two issuing threads (warps 1 and 3)
    F_TMA = 256,        // a real TMA producer behind the ring
    F_FAR = 512,        // the per-block scale load misses L1 (a new line of a large array per K block, as in the kernel)
    F_AHEAD2 = 1024,    // ... and is issued two K blocks ahead instead of one
    F_LATE = 2048,      // ... or is issued after the wait for the accumulator stage instead of before it
    F_M64 = 4096,       // M = 64 instructions (same operands in shared memory, half of the rows multiplied)
};
constexpr int kScaleRows = 32768;   // the far scale array: [56 K blocks][kScaleRows] floats (7 MB)
constexpr int kOperandRows = 8192, kOperandK = 7168;   // the buffer the TMA forms read (58 MB)
constexpr int kStageBytes = 48 * 1024;

__device__ __forceinline__ void wait_loads(uint32_t (&a)[32], uint32_t (&b)[32]) {
    // tcgen05.wait::ld with the destination registers as in/out operands (no use may move above it)
#define R8(x, o) "+r"(x[o]), "+r"(x[o + 1]), "+r"(x[o + 2]), "+r"(x[o + 3]), "+r"(x[o + 4]), "+r"(x[o + 5]), "+r"(x[o + 6]), "+r"(x[o + 7])
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : R8(a, 0), R8(a, 8), R8(a, 16), R8(a, 24), R8(b, 0), R8(b, 8), R8(b, 16), R8(b, 24)
                 :
                 : "memory");
#undef R8
}

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

// The operand ring has three stages; its barriers come as one full / empty pair per K block of a window of
// six, so that with two issuing threads (even / odd K blocks) every pair is always used by the same thread
// and its phases are seen in order (a parity wait cannot tell a phase from the one two before it).
constexpr int kRingStages = 3;
constexpr int kRingBars = 6;

template <int FORM>
__global__ void __launch_bounds__(384, 1) probe(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                float* out, long long* cycles, int iters) {
    constexpr bool kN128 = FORM & F_N128, kLoads = FORM & F_LOADS, kFma = FORM & (F_FMA_SCALAR | F_FMA_PACKED);
    constexpr bool kPacked = FORM & F_FMA_PACKED, kRing = FORM & F_RING, kScales = FORM & F_SCALES;
    constexpr bool kRelay = FORM & F_RELAY, kTwo = FORM & F_TWO, kTma = FORM & F_TMA;
    constexpr bool kFar = FORM & F_FAR, kAhead2 = FORM & F_AHEAD2, kLate = FORM & F_LATE, kM64 = FORM & F_M64;
    __shared__ uint32_t slot;
    __shared__ uint64_t acc_full[2], acc_empty[2];
    __shared__ uint64_t st_full[kRingBars], st_empty[kRingBars];
    __shared__ int abort_word;
    extern __shared__ __align__(1024) uint8_t tiles[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&acc_full[s]), 1); mbar_init(smem_u32(&acc_empty[s]), 8); }
        for (int s = 0; s < kRingBars; ++s) { mbar_init(smem_u32(&st_full[s]), 1); mbar_init(smem_u32(&st_empty[s]), 1); }
        abort_word = 0;
        fence_mbar_init();
    }
    if (warp == 2) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t base = slot;
    volatile int* abort_flag = &abort_word;
    if (warp < 4) {
        setmaxnreg_dec<56>();
        if (kRing && warp == 0 && lane == 0) {
            // stand-in for the TMA producer: same barrier traffic, no data
            int it = 0;
            for (; it < iters; ++it) {
                if (it >= kRingStages) {
                    const int pit = it - kRingStages;   // the K block that last used this stage
                    if (!mbar_wait(smem_u32(&st_empty[pit % kRingBars]), (pit / kRingBars) & 1, abort_flag)) break;
                }
                const uint32_t full = smem_u32(&st_full[it % kRingBars]);
                if (kTma) {
                    const uint32_t dst = ((smem_u32(tiles) + 1023u) & ~1023u) + (uint32_t)(it % kRingStages) * kStageBytes;
                    const int kb = it % (kOperandK / 128), tile = it / (kOperandK / 128);
                    mbar_expect_tx(full, kStageBytes);
                    tma_load_2d(dst, &map_a, full, kb * 128, (int)(((blockIdx.x * 7u + tile) * 128u) % kOperandRows));
                    tma_load_2d(dst + 16384, &map_b, full, kb * 128, (int)((((blockIdx.x / 6u) * 13u + tile) * 256u) % kOperandRows));
                } else {
                    mbar_arrive(full);
                }
            }
            if (kTma && it < iters) {
                // a wait ran out: leave only after the copies still in flight have landed (bounded)
                for (int j = it > kRingStages ? it - kRingStages : 0; j < it; ++j)
                    mbar_wait(smem_u32(&st_full[j % kRingBars]), (j / kRingBars) & 1, abort_flag);
            }
        }
        if ((warp == 1 || (kTwo && warp == 3)) && lane == 0) {
            const uint32_t mine = warp == 3 ? 1u : 0u;
            const int step = kTwo ? 2 : 1;
            const uint32_t tb = (smem_u32(tiles) + 1023u) & ~1023u;   // without TMA the operand bytes are whatever the SM holds
            uint64_t ad = make_kmajor_sw128_desc(tb), bd = make_kmajor_sw128_desc(tb + 16384);
            const uint32_t idesc = make_idesc_e4m3(kM64 ? 64 : 128, 256), idesc128 = make_idesc_e4m3(128, 128);
            const long long t0 = clock64();
            bool next_ready = false;
            for (int it = 0; it < iters; ++it) {
                const uint32_t as = it & 1, aph = (it >> 1) & 1;
                if (kTwo && as != mine) continue;
                if (kRing && !next_ready && !mbar_wait(smem_u32(&st_full[it % kRingBars]), (it / kRingBars) & 1, abort_flag)) break;
                if (!mbar_wait(smem_u32(&acc_empty[as]), aph ^ 1, abort_flag)) break;
                tc_fence_after();
                if (kTma) {
                    const uint32_t st = tb + (uint32_t)(it % kRingStages) * kStageBytes;
                    ad = make_kmajor_sw128_desc(st);
                    bd = make_kmajor_sw128_desc(st + 16384);
                }
                if (kN128) {
                    for (int hh = 0; hh < 2; ++hh)
                        for (int kk = 0; kk < 4; ++kk)
                            umma_f8(base + as * 256 + 128 * hh, ad + 2 * kk, bd + 1024 * hh + 2 * kk, idesc128, kk > 0);
                } else {
                    for (int kk = 0; kk < 4; ++kk) umma_f8(base + as * 256, ad + 2 * kk, bd + 2 * kk, idesc, kk > 0);
                }
                if (kRing && !kRelay) tc_commit(smem_u32(&st_empty[it % kRingBars]));
                tc_commit(smem_u32(&acc_full[as]));
                if (kRing) next_ready = mbar_try_wait(smem_u32(&st_full[(it + step) % kRingBars]), ((it + step) / kRingBars) & 1);
            }
            if (blockIdx.x == 0 && warp == 1) cycles[0] = clock64() - t0;
        }
    } else {
        setmaxnreg_inc<224>();
        const int q = warp & 3, h = (warp - 4) >> 2;
        const uint32_t la = base + ((uint32_t)(q * 32) << 16);
        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; ++j) acc[j] = 0.f;
        uint32_t r0[32], r1[32];
        float sa_n = 1.0f, sa_n2 = 1.0f;
        const float* far = out + 4096 + (blockIdx.x * 128 + (warp & 3) * 32 + lane) % (kScaleRows - 4096);
        for (int it = 0; it < iters; ++it) {
            const uint32_t as = it & 1, aph = (it >> 1) & 1;
            float s_lo = 1.0f + it * 1e-9f, s_hi = 1.0f - it * 1e-9f;
            if (kScales) {
                const float lo_w = __shfl_sync(0xffffffffu, s_lo, it & 31), hi_w = __shfl_sync(0xffffffffu, s_hi, it & 31);
                s_lo = sa_n * lo_w;
                s_hi = sa_n * hi_w;
                if (kFar && !kLate) {
                    // row scale of K block it + 1 (or it + 2): line (it % 56) of the [56][rows] array, at a row offset
                    // that moves with the tile, so that no line is met twice in a row
                    const int nit = it + (kAhead2 ? 2 : 1);
                    const float* src = far + (size_t)(nit % 56) * kScaleRows + (size_t)((nit / 56) % 32) * 128;
                    if (kAhead2) {
                        sa_n = sa_n2;
                        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sa_n2) : "l"(src));
                    } else {
                        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sa_n) : "l"(src));
                    }
                } else if (!kFar) {
                    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(sa_n) : "l"(out + 1024 + ((it * 128 + threadIdx.x) & 1023)));
                }
            }
            bool ok = mbar_wait(smem_u32(&acc_full[as]), aph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (kScales && kFar && kLate) {
                const int nit = it + 1;
                asm volatile("ld.global.nc.f32 %0, [%1];"
                             : "=f"(sa_n)
                             : "l"(far + (size_t)(nit % 56) * kScaleRows + (size_t)((nit / 56) % 32) * 128));
            }
            if (kRing && kRelay && warp == 4 && lane == 0) mbar_arrive(smem_u32(&st_empty[it % kRingBars]));
            if (!kLoads) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
                continue;
            }
            const uint32_t t = la + as * 256 + 128 * h;
            tmem_ld_32x32(t, r0);
            tmem_ld_32x32(t + 32, r1);
            wait_loads(r0, r1);
            if (kFma) promote32<0, kPacked>(acc, r0, s_lo);
            tmem_ld_32x32(t + 64, r0);
            if (kFma) promote32<32, kPacked>(acc, r1, s_lo);
            tmem_ld_32x32(t + 96, r1);
            wait_loads(r0, r1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
            if (kFma) { promote32<64, kPacked>(acc, r0, s_hi); promote32<96, kPacked>(acc, r1, s_hi); }
            else acc[0] += __uint_as_float(r0[0]) + __uint_as_float(r1[31]);   // keeps the loads alive, nothing more
        }
        float sum = 0;
#pragma unroll
        for (int j = 0; j < 128; ++j) sum += acc[j];
        if (blockIdx.x == 0) out[threadIdx.x] = sum;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(base, 512); }
    if (threadIdx.x == 0 && blockIdx.x == 0) cycles[1] = abort_word;
}

// pseudo-random e4m3 bytes with the top exponent bit clear (finite, |x| < 2), so that the tensor pipe toggles as
// it does on real operands
__global__ void fill_operands(uint32_t* p, size_t words) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t x = (uint32_t)i * 2654435761u + 12345u;
        x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
        p[i] = x & 0xBFBFBFBFu;
    }
}

static CUtensorMap g_map_a, g_map_b;
static const char* g_only = nullptr;   // argv[3]: run only the forms whose name contains it

// [kOperandRows, kOperandK] bytes, K contiguous; box = 128 bytes x box_rows with the 128-byte swizzle
static bool encode_map(CUtensorMap* m, void* base, uint32_t box_rows) {
    typedef CUresult (*Fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                           const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                           CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
    const cuuint64_t dims[2] = {kOperandK, kOperandRows};
    const cuuint64_t strides[1] = {kOperandK};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return reinterpret_cast<Fn>(p)(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int FORM>
static int run(const char* name, int ctas, int iters, float* out, long long* d) {
    const int smem = (FORM & F_TMA) ? 3 * kStageBytes + 2048 : 50 * 1024;
    cudaFuncSetAttribute(probe<FORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (g_only && !strstr(name, g_only)) return 0;
    cudaMemset(d, 0, 64);
    cudaEvent_t ev0, ev1;
    cudaEventCreate(&ev0);
    cudaEventCreate(&ev1);
    cudaEventRecord(ev0);
    probe<FORM><<<ctas, 384, smem>>>(g_map_a, g_map_b, out, d, iters);
    cudaEventRecord(ev1);
    const cudaError_t e = cudaDeviceSynchronize();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, ev0, ev1);
    long long h[2] = {0, 0};
    cudaMemcpy(h, d, sizeof h, cudaMemcpyDeviceToHost);
    printf("%-20s %8.1f cycles per K block   (%s%s)   %.1f ns per K block\n", name, (double)h[0] / iters, cudaGetErrorString(e),
           h[1] ? ", a wait ran out" : "", ms * 1e6 / iters);
    return (e == cudaSuccess && h[1] == 0) ? 0 : 1;
}

int main(int argc, char** argv) {
    const int ctas = argc > 1 ? atoi(argv[1]) : 1;
    const int iters = argc > 2 ? atoi(argv[2]) : 4000;
    g_only = argc > 3 ? argv[3] : nullptr;
    float* out;
    long long* d;
    const size_t out_bytes = 16384 + sizeof(float) * 56 * (size_t)kScaleRows;
    cudaMalloc(&out, out_bytes);
    cudaMemset(out, 0, out_bytes);
    cudaMalloc(&d, 64);
    void* operands;
    cudaMalloc(&operands, (size_t)kOperandRows * kOperandK);
    fill_operands<<<1024, 256>>>(static_cast<uint32_t*>(operands), (size_t)kOperandRows * kOperandK / 4);
    if (!encode_map(&g_map_a, operands, 128) || !encode_map(&g_map_b, operands, 256)) {
        printf("cuTensorMapEncodeTiled failed\n");
        return 1;
    }
    printf("ctas %d, K blocks %d\n", ctas, iters);
    constexpr int kPromote = F_LOADS | F_FMA_PACKED;
    int bad = 0;
    bad |= run<0>("mma_only", ctas, iters, out, d);
    bad |= run<F_N128>("mma_only_n128", ctas, iters, out, d);
    bad |= run<F_LOADS>("drain", ctas, iters, out, d);
    bad |= run<F_LOADS | F_FMA_SCALAR>("promote_scalar", ctas, iters, out, d);
    bad |= run<kPromote>("promote_packed", ctas, iters, out, d);
    bad |= run<kPromote | F_RING>("ring", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES>("ring_scales", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_RELAY>("ring_scales_relayed", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TWO>("ring_scales_two", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TMA>("ring_scales_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TWO | F_TMA>("ring_scales_two_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TMA | F_FAR>("ring_far_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TWO | F_TMA | F_FAR>("ring_far_two_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TWO | F_TMA | F_FAR | F_AHEAD2>("ring_far2_two_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TMA | F_M64>("ring_scales_tma_m64", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TMA | F_FAR | F_LATE>("ring_farlate_tma", ctas, iters, out, d);
    bad |= run<kPromote | F_RING | F_SCALES | F_TWO | F_TMA | F_FAR | F_LATE>("ring_farlate_two_tma", ctas, iters, out, d);
    return bad;
}
