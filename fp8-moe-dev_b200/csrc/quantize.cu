// Quantise-on-entry: bf16 activations [T, 7168] -> e4m3 [T, 7168] plus one fp32 scale per
// (token, 128-column block), stored block-major [56, T] -- the producer of the layer's
// `hidden_states` / `hidden_states_scale` arguments (kernel/moe_fp8.cu:2665-2666 in the
// reference, which expects them already quantised).  The scheme is the 1x128 one the layer
// itself applies to the SwiGLU output (kernel/moe_fp8.cu:1823-1830): scale = amax / 448
// (1 where the block is all zero); the payload is e4m3_rn_satfinite(x / scale) with a true
// division, so that x ~= q * scale as the layer's GEMM1 assumes.
//
// HBM-bound: 2 B read + 1 B written per element, 4 B per block.  A CTA takes eight tokens
// (one warp each) times a quarter of the row (14 blocks), so that a batch makes many more
// CTAs than fit on the chip at once and the last wave is short; each half-warp owns every
// other 128-column block (16 lanes x 16 B = one block) and issues its seven 16-byte loads
// up front.  The scales of a CTA's eight tokens are staged in shared memory and written as
// 32-byte runs of the [56, T] array.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "layer.cuh"
#include "ptx.cuh"

namespace moe {

constexpr int kQuantTokensPerCta = 8;
constexpr int kQuantThreads = 32 * kQuantTokensPerCta;
constexpr int kQuantRowParts = 4;                                   // blockIdx.y: quarter of the row
constexpr int kQuantBlocksPerPart = kHiddenBlocks / kQuantRowParts; // 14
static_assert(kHiddenBlocks % (2 * kQuantRowParts) == 0, "a part must split evenly over two half-warps");

// One 128-column block of one row, spread over the 16 lanes of a half-warp (16 bytes of bf16 input each):
// returns the block's scale and this lane's eight e4m3 codes.
__device__ __forceinline__ float quantize_block_lane(const uint4& raw, uint32_t (&w)[2])
{
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    // block maximum on packed bf16 pairs, then over the 16 lanes of this half-warp
    // (xor offsets < 16 stay inside it)
    __nv_bfloat162 m2 = __hmax2(__habs2(h2[0]), __habs2(h2[1]));
    m2 = __hmax2(m2, __hmax2(__habs2(h2[2]), __habs2(h2[3])));
    float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // scale = RN(amax / 448) without the division subroutine: q = amax * RN(1/448) is
    // within an ulp, r = amax - 448 q is exact in an FMA, and q + r * RN(1/448) then rounds
    // to the correctly rounded quotient (one-step FMA correction with a correctly rounded
    // reciprocal; checked against the division for every bf16 maximum by the tests).  It
    // needs a normal result, so tiny and huge maxima divide.
    constexpr float kInv448 = 1.0f / 448.0f;
    const bool sane = amax >= 0x1p-90f && amax <= 0x1p100f;
    float scale;
    if (sane) {
        const float q0 = amax * kInv448;
        scale = fmaf(fmaf(-448.0f, q0, amax), kInv448, q0);
    } else {
        scale = amax > 0.0f ? amax / 448.0f : 1.0f;
    }
    // The payload is e4m3(x / scale) with the correctly rounded quotient, but an IEEE
    // division per element would make this kernel instruction-bound.  Instead bracket the
    // quotient: x * inv_lo <= x / scale <= x * inv_hi in magnitude, where inv_lo/hi are
    // an approximate 1 / scale (error <= 2^-23) pushed down / up by 2^-21 (the roundings
    // involved move a value by less than 2^-22).  Rounding to e4m3 is monotonic, so where
    // both ends give the same code that code is the answer; only lanes where they differ
    // (the quotient is within 2^-20 of a rounding boundary) and blocks with an extreme
    // scale divide.
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(scale));
    const float inv_lo = inv * (1.0f - 0x1p-21f), inv_hi = inv * (1.0f + 0x1p-21f);
    const float2 lo2 = make_float2(inv_lo, inv_lo), hi2 = make_float2(inv_hi, inv_hi);
    bool redo = !sane;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 fa = __bfloat1622float2(h2[2 * i]), fb = __bfloat1622float2(h2[2 * i + 1]);
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(__fmul2_rn(fa, lo2), __NV_SATFINITE, __NV_E4M3) |
                            ((uint32_t)__nv_cvt_float2_to_fp8x2(__fmul2_rn(fb, lo2), __NV_SATFINITE, __NV_E4M3) << 16);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(__fmul2_rn(fa, hi2), __NV_SATFINITE, __NV_E4M3) |
                            ((uint32_t)__nv_cvt_float2_to_fp8x2(__fmul2_rn(fb, hi2), __NV_SATFINITE, __NV_E4M3) << 16);
        w[i] = lo;
        redo |= lo != hi;
    }
    if (redo) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float2 fa = __bfloat1622float2(h2[2 * i]), fb = __bfloat1622float2(h2[2 * i + 1]);
            w[i] = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(fa.x, scale), __fdiv_rn(fa.y, scale)), __NV_SATFINITE, __NV_E4M3) |
                   ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(fb.x, scale), __fdiv_rn(fb.y, scale)), __NV_SATFINITE, __NV_E4M3) << 16);
        }
    }
    return scale;
}

__global__ void __launch_bounds__(kQuantThreads) quantize_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                      uint8_t* __restrict__ q,
                                                                      float* __restrict__ scale_out, int T)
{
    __shared__ float s_scale[kQuantBlocksPerPart][kQuantTokensPerCta];
    const int kb0 = blockIdx.y * kQuantBlocksPerPart;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int t0 = blockIdx.x * kQuantTokensPerCta;
    const int t = t0 + warp;
    pdl_launch_dependents();
    pdl_wait();
    if (t < T) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * kHidden);
        uint2* dst = reinterpret_cast<uint2*>(q + (size_t)t * kHidden);
        constexpr int kIters = kQuantBlocksPerPart / 2;   // 7 blocks per half-warp
        constexpr int kUnroll = kIters;
        for (int it0 = 0; it0 < kIters; it0 += kUnroll) {
            uint4 raw[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kb = kb0 + 2 * (it0 + u) + half;
                raw[u] = __ldg(src + kb * 16 + l16);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int kb = kb0 + 2 * (it0 + u) + half;
                uint32_t w[2];
                const float scale = quantize_block_lane(raw[u], w);
                dst[kb * 16 + l16] = make_uint2(w[0], w[1]);
                if (l16 == 0) s_scale[kb - kb0][warp] = scale;
            }
        }
    }
    __syncthreads();
    // [56, T]: for each block the CTA's eight tokens are consecutive
    for (int i = threadIdx.x; i < kQuantBlocksPerPart * kQuantTokensPerCta; i += kQuantThreads) {
        const int kb = i / kQuantTokensPerCta, w = i % kQuantTokensPerCta;
        if (t0 + w < T) scale_out[(size_t)(kb0 + kb) * T + t0 + w] = s_scale[kb][w];
    }
}

// Any row length that is a multiple of 128: one warp per token, its half-warps take alternate blocks.
__global__ void __launch_bounds__(kQuantThreads) quantize_rows_generic_kernel(const __nv_bfloat16* __restrict__ x,
                                                                              uint8_t* __restrict__ q,
                                                                              float* __restrict__ scale_out, int T, int K)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int t = blockIdx.x * kQuantTokensPerCta + warp;
    if (t >= T) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * K);
    uint2* dst = reinterpret_cast<uint2*>(q + (size_t)t * K);
    const int blocks = K / kBlock;
    for (int kb0 = 0; kb0 < blocks; kb0 += 2) {   // uniform trip count: the shuffles inside want whole warps
        const int kb = kb0 + half;
        const bool live = kb < blocks;
        const uint4 raw = live ? __ldg(src + kb * 16 + l16) : make_uint4(0u, 0u, 0u, 0u);
        uint32_t w[2];
        const float scale = quantize_block_lane(raw, w);
        if (live) {
            dst[kb * 16 + l16] = make_uint2(w[0], w[1]);
            if (l16 == 0) scale_out[(size_t)kb * T + t] = scale;
        }
    }
}

cudaError_t launch_quantize_rows(const void* x, void* q, float* scale_out, int T, int K, cudaStream_t stream)
{
    if (T <= 0) return cudaSuccess;
    if (K != kHidden) {
        const int g = (T + kQuantTokensPerCta - 1) / kQuantTokensPerCta;
        quantize_rows_generic_kernel<<<g, kQuantThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                      static_cast<uint8_t*>(q), scale_out, T, K);
        return cudaGetLastError();
    }
    const int grid = (T + kQuantTokensPerCta - 1) / kQuantTokensPerCta;
    quantize_rows_kernel<<<dim3(grid, kQuantRowParts), kQuantThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                             static_cast<uint8_t*>(q), scale_out, T);
    return cudaGetLastError();
}

}  // namespace moe
