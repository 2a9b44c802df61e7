// Quantise-on-entry: bf16 activations [T, 7168] -> e4m3 [T, 7168] plus one fp32 scale per
// (token, 128-column block), stored block-major [56, T] -- the producer of the layer's
// `hidden_states` / `hidden_states_scale` arguments (kernel/moe_fp8.cu:2665-2666 in the
// reference, which expects them already quantised).  The scheme is the 1x128 one the layer
// itself applies to the SwiGLU output (kernel/moe_fp8.cu:1823-1830): scale = amax / 448
// (1 where the block is all zero); the payload is e4m3_rn_satfinite(x / scale) with a true
// division, so that x ~= q * scale as the layer's GEMM1 assumes.
//
// HBM-bound: 2 B read + 1 B written per element, 4 B per block.  One warp per token, eight
// tokens per CTA; each half-warp owns every other 128-column block (16 lanes x 16 B = one
// block), so a lane keeps four independent 16-byte loads in flight.  The scales of a CTA's
// eight tokens are staged in shared memory and written as 32-byte runs of the [56, T] array.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "layer.cuh"
#include "ptx.cuh"

namespace moe {

constexpr int kQuantTokensPerCta = 8;
constexpr int kQuantThreads = 32 * kQuantTokensPerCta;

__global__ void __launch_bounds__(kQuantThreads) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                      uint8_t* __restrict__ q,
                                                                      float* __restrict__ scale_out, int T)
{
    __shared__ float s_scale[kHiddenBlocks][kQuantTokensPerCta];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int t0 = blockIdx.x * kQuantTokensPerCta;
    const int t = t0 + warp;
    pdl_launch_dependents();
    pdl_wait();
    if (t < T) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * kHidden);
        uint2* dst = reinterpret_cast<uint2*>(q + (size_t)t * kHidden);
        constexpr int kIters = kHiddenBlocks / 2;   // 28 blocks per half-warp
        constexpr int kUnroll = 4;
        static_assert(kIters % kUnroll == 0, "unroll must divide the block count");
        for (int it0 = 0; it0 < kIters; it0 += kUnroll) {
            uint4 raw[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kb = 2 * (it0 + u) + half;
                raw[u] = __ldg(src + kb * 16 + l16);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kb = 2 * (it0 + u) + half;
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                float v[8];
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h2[j]);
                    v[2 * j] = f.x;
                    v[2 * j + 1] = f.y;
                    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
                // maximum over the 16 lanes of this half-warp (xor offsets < 16 stay inside it)
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
                uint32_t w[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                        make_float2(__fdiv_rn(v[4 * i], scale), __fdiv_rn(v[4 * i + 1], scale)), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                        make_float2(__fdiv_rn(v[4 * i + 2], scale), __fdiv_rn(v[4 * i + 3], scale)), __NV_SATFINITE, __NV_E4M3);
                    w[i] = lo | (hi << 16);
                }
                dst[kb * 16 + l16] = make_uint2(w[0], w[1]);
                if (l16 == 0) s_scale[kb][warp] = scale;
            }
        }
    }
    __syncthreads();
    // [56, T]: for each block the CTA's eight tokens are consecutive
    for (int i = threadIdx.x; i < kHiddenBlocks * kQuantTokensPerCta; i += kQuantThreads) {
        const int kb = i / kQuantTokensPerCta, w = i % kQuantTokensPerCta;
        if (t0 + w < T) scale_out[(size_t)kb * T + t0 + w] = s_scale[kb][w];
    }
}

cudaError_t launch_quantize_rows(const void* x, void* q, float* scale_out, int T, cudaStream_t stream)
{
    if (T <= 0) return cudaSuccess;
    const int grid = (T + kQuantTokensPerCta - 1) / kQuantTokensPerCta;
    quantize_rows_kernel<<<grid, kQuantThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                             static_cast<uint8_t*>(q), scale_out, T);
    return cudaGetLastError();
}

}  // namespace moe
