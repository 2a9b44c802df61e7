// Micro-benchmark of the grouped GEMM's inner pipeline on ONE SM (or one CTA on each of N SMs), without
// TMA and without real data: the MMA-issuing thread, the two 256-column TMEM accumulator stages and the
// eight promotion warps with the kernel's own handshake (ptx.cuh of the package).  It reports SM cycles
// per 128-wide K block for a few forms of the loop, which is where the figures quoted in the design notes
// about the promotion pipeline come from:
//   mma_only        4 x tcgen05.mma M128 N256 K32 per K block, promotion warps release the stage at once
//   mma_only_n128   the same block issued as 8 x M128 N128 K32 (what a finer accumulator split would need)
//   drain           promotion warps read the whole stage from TMEM (4 x 32 columns each), no arithmetic
//   promote_scalar  + fp32 scale-and-add with scalar FMAs
//   promote_packed  + the packed two-wide FMA the kernel uses
// Build: nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -I <package>/csrc gemm_pipeline_probe.cu
// Run:   ./a.out [ctas=1] [k_blocks=4000]     (every wait is bounded; a failed wait ends the kernel)
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "ptx.cuh"
using namespace moe;

enum Form { kMmaOnly = 0, kMmaOnlyN128 = 1, kDrain = 2, kPromoteScalar = 3, kPromotePacked = 4 };

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

template <int FORM>
__global__ void __launch_bounds__(384, 1) probe(float* out, long long* cycles, int iters) {
    __shared__ uint32_t slot;
    __shared__ uint64_t acc_full[2], acc_empty[2];
    __shared__ int abort_word;
    extern __shared__ __align__(1024) uint8_t tiles[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&acc_full[s]), 1); mbar_init(smem_u32(&acc_empty[s]), 8); }
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
        if (warp == 1 && lane == 0) {
            const uint32_t tb = (smem_u32(tiles) + 1023u) & ~1023u;   // operand bytes are whatever the SM holds
            const uint64_t ad = make_kmajor_sw128_desc(tb), bd = make_kmajor_sw128_desc(tb + 16384);
            const uint32_t idesc = make_idesc_e4m3(128, 256), idesc128 = make_idesc_e4m3(128, 128);
            const long long t0 = clock64();
            for (int it = 0; it < iters; ++it) {
                const uint32_t as = it & 1, aph = (it >> 1) & 1;
                if (!mbar_wait(smem_u32(&acc_empty[as]), aph ^ 1, abort_flag)) break;
                tc_fence_after();
                if (FORM == kMmaOnlyN128) {
                    for (int hh = 0; hh < 2; ++hh)
                        for (int kk = 0; kk < 4; ++kk)
                            umma_f8(base + as * 256 + 128 * hh, ad + 2 * kk, bd + 1024 * hh + 2 * kk, idesc128, kk > 0);
                } else {
                    for (int kk = 0; kk < 4; ++kk) umma_f8(base + as * 256, ad + 2 * kk, bd + 2 * kk, idesc, kk > 0);
                }
                tc_commit(smem_u32(&acc_full[as]));
            }
            if (blockIdx.x == 0) cycles[0] = clock64() - t0;
        }
    } else {
        setmaxnreg_inc<224>();
        const int q = warp & 3, h = (warp - 4) >> 2;
        const uint32_t la = base + ((uint32_t)(q * 32) << 16);
        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; ++j) acc[j] = 0.f;
        uint32_t r0[32], r1[32];
        for (int it = 0; it < iters; ++it) {
            const uint32_t as = it & 1, aph = (it >> 1) & 1;
            const float s_lo = 1.0f + it * 1e-9f, s_hi = 1.0f - it * 1e-9f;
            bool ok = mbar_wait(smem_u32(&acc_full[as]), aph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (FORM == kMmaOnly || FORM == kMmaOnlyN128) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[as]));
                continue;
            }
            const uint32_t t = la + as * 256 + 128 * h;
            constexpr bool kFma = FORM >= kPromoteScalar, kPacked = FORM == kPromotePacked;
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

template <int FORM>
static int run(const char* name, int ctas, int iters, float* out, long long* d) {
    cudaFuncSetAttribute(probe<FORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 50 * 1024);
    cudaMemset(d, 0, 64);
    probe<FORM><<<ctas, 384, 50 * 1024>>>(out, d, iters);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h[2] = {0, 0};
    cudaMemcpy(h, d, sizeof h, cudaMemcpyDeviceToHost);
    printf("%-15s %8.1f cycles per K block   (%s%s)\n", name, (double)h[0] / iters, cudaGetErrorString(e),
           h[1] ? ", a wait ran out" : "");
    return (e == cudaSuccess && h[1] == 0) ? 0 : 1;
}

int main(int argc, char** argv) {
    const int ctas = argc > 1 ? atoi(argv[1]) : 1;
    const int iters = argc > 2 ? atoi(argv[2]) : 4000;
    float* out;
    long long* d;
    cudaMalloc(&out, 4096);
    cudaMalloc(&d, 64);
    printf("ctas %d, K blocks %d\n", ctas, iters);
    int bad = 0;
    bad |= run<kMmaOnly>("mma_only", ctas, iters, out, d);
    bad |= run<kMmaOnlyN128>("mma_only_n128", ctas, iters, out, d);
    bad |= run<kDrain>("drain", ctas, iters, out, d);
    bad |= run<kPromoteScalar>("promote_scalar", ctas, iters, out, d);
    bad |= run<kPromotePacked>("promote_packed", ctas, iters, out, d);
    return bad;
}
