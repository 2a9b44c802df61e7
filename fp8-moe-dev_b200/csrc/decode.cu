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
//     B tile.  The weights go from global memory straight into the A fragments (each weight
//     byte is used once; shared memory would only add a hop), the 16 warps split K, promote
//     per 128-K block with the two scales like the staged kernel, and meet in shared memory.
//     In the accumulator layout a thread owns the linear and the gated value of the same
//     (column, token), so SwiGLU needs no exchange.  v = silu(gate) * lin goes to a small
//     fp32 scratch (the 1x128 requantisation needs whole 128-column blocks, which span units);
//   * grid barrier; phase 2 (GEMM2): each CTA requantises the rows of its expert from the
//     scratch (same arithmetic as the staged epilogue), streams 16 rows of W2 per unit the
//     same way, and writes bf16 y rows; grid barrier; phase 3 is the weighted combine.
// The first weights of phase 2 are requested before the barrier, so the barrier and the
// requantisation hide behind their latency.  The two grid barriers are bounded waits.
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
constexpr int kDecMaxActive = kDecodeMaxTokens * kTopK;   // 64 (token, expert) pairs at most
constexpr int kHidStride = kHidden + 64;   // row strides that spread the eight token rows over the banks
constexpr int kA2Stride = kInter + 64;
constexpr int kG1Cols = 8;                              // SwiGLU columns of a phase-1 unit
constexpr int kG1Units = kInter / kG1Cols;              // 256 per expert
constexpr int kG2Cols = 16;                             // output columns of a phase-2 unit
constexpr int kG2Units = kHidden / kG2Cols;             // 448 per expert
constexpr int kG1Steps = (kHiddenBlocks + kDecWarps - 1) / kDecWarps;   // K blocks per warp (4, last may be absent)
static_assert(kInterBlocks == kDecWarps, "phase 2 gives each warp one K block");

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
    float scale[kDecodeMaxTokens][kHiddenBlocks];   // phase 1: [slot][kb] hidden scales; phase 2: [slot][kb < 16]
    float w2_scale[2][kInterBlocks];
    alignas(16) float red[2][kDecWarps][128];
    alignas(16) uint8_t stage[kDecodeMaxTokens * kHidStride];
};

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const unsigned* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Weights are read exactly once: streaming loads that do not linger in L1.
__device__ __forceinline__ uint4 ld_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 128-K block: rows r / r + 8 of the A tile in lo[2] / hi[2] (16 B at byte 16c and at byte
// 64 + 16c of the block, c = lane % 4), the token rows' same bytes in b[2].  Which 4 bytes feed
// which k index of the MMA is the same for A and B, and a dot product does not care about more.
__device__ __forceinline__ void mma_block(float (&c)[4], const uint4 (&lo)[2], const uint4 (&hi)[2], const uint4 (&b)[2]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mma_e4m3(c, lo[h].x, hi[h].x, lo[h].y, hi[h].y, b[h].x, b[h].y);
        mma_e4m3(c, lo[h].z, hi[h].z, lo[h].w, hi[h].w, b[h].z, b[h].w);
    }
}

// All CTAs of the (cooperative, co-resident) grid meet here.  Bounded: a CTA that waits longer
// than the limit records the failure and returns false; its peers run into the same limit.
__device__ __forceinline__ bool grid_barrier(Control* ctrl, DecodeShared* sh)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t phase = ld_acquire_gpu(&ctrl->dec_phase);
        const unsigned ticket = atomicAdd(&ctrl->dec_count, 1u);
        if (ticket == gridDim.x - 1) {
            ctrl->dec_count = 0;
            __threadfence();
            st_release_gpu(&ctrl->dec_phase, phase + 1);
        } else {
            const uint64_t t0 = global_timer_ns();
            uint32_t it = 0;
            while (ld_acquire_gpu(&ctrl->dec_phase) == phase) {
                if ((++it & 0x3fu) == 0u && global_timer_ns() - t0 > kWaitLimitNs) {
                    atomicCAS(&ctrl->status, kStatusOk, kStatusDecodeTimeout);
                    sh->abort = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return sh->abort == 0;
}

__global__ void __launch_bounds__(kDecThreads, 1) decode_layer_kernel(DecodeArgs a, Workspace ws)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    DecodeShared* sh = reinterpret_cast<DecodeShared*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, c = lane & 3;   // MMA fragment coordinates
    const int T = a.T, E = a.num_local_experts;

    // ------------------------------------------------------------------ routing (every CTA)
    if (tid < kMaxLocalExperts) sh->expert_slot[tid] = -1;
    if (tid == 0) sh->abort = 0;
    if (warp < T) {
        int idx[kTopK];
        float wn[kTopK];
        route_token_warp(a.logits + (size_t)warp * kNumExperts, a.bias, lane, idx, wn);
        if (blockIdx.x == 0 && lane < kTopK) {
            int my_idx = 0;
            float my_w = 0.0f;
#pragma unroll
            for (int k = 0; k < kTopK; ++k)
                if (k == lane) { my_idx = idx[k]; my_w = wn[k]; }
            ws.topk_idx[(size_t)warp * kTopK + lane] = my_idx;
            ws.topk_weight[(size_t)warp * kTopK + lane] = my_w;
        }
        if (lane == 0) {
            int n_pairs = 0;
            int p_le[kTopK];
            float p_w[kTopK];
#pragma unroll
            for (int i = 0; i < kTopK; ++i) { p_le[i] = 0; p_w[i] = 0.0f; }
            const int shards = E / kShardExperts;
            for (int s = 0; s < shards; ++s)
                dispatch_one_shard(idx, wn, s, a.local_expert_offset, a.pol, a.rsf, n_pairs, p_le, p_w);
            sh->pair_count[warp] = n_pairs;
#pragma unroll
            for (int i = 0; i < kTopK; ++i) { sh->pair_le[warp][i] = p_le[i]; sh->pair_w[warp][i] = p_w[i]; }
        }
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
    }
    __syncthreads();
    if (tid < T * kTopK) {
        const int t = tid / kTopK, p = tid % kTopK;
        if (p < sh->pair_count[t]) sh->pair_row[t][p] = sh->act_row0[sh->expert_slot[sh->pair_le[t][p]]] + sh->pair_slot[t][p];
    }
    if (blockIdx.x == 0) {   // the tables other entry points and the tests read
        if (tid == 0) { ws.ctrl->status = kStatusOk; ws.ctrl->status_detail = 0; }
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
    __syncthreads();
    const int n_active = sh->n_active;
    float* act = ws.splitk_partial;   // [rows, 2048] fp32 SwiGLU output (the split-K scratch is idle on this path)

    // ------------------------------------------------------------------ phase 1: GEMM1 + SwiGLU
    {
        const int units = n_active * kG1Units;
        const int u_begin = (int)((long long)units * blockIdx.x / gridDim.x);
        const int u_end = (int)((long long)units * (blockIdx.x + 1) / gridDim.x);
        uint4 wl[kG1Steps][2], wg[kG1Steps][2];
        auto load_unit = [&](int u, int i) {
            const int kb = warp + kDecWarps * i;
            if (kb < kHiddenBlocks) {
                const int e = sh->act_expert[u / kG1Units];
                const int n = (u % kG1Units) * kG1Cols + r;
                const uint8_t* lin = a.w1 + ((size_t)e * kGemm1Out + n) * kHidden + kb * kBlock + 16 * c;
                const uint8_t* gat = lin + (size_t)kInter * kHidden;
                wl[i][0] = ld_stream(lin);
                wl[i][1] = ld_stream(lin + 64);
                wg[i][0] = ld_stream(gat);
                wg[i][1] = ld_stream(gat + 64);
            }
        };
        if (u_begin < u_end) {
#pragma unroll
            for (int i = 0; i < kG1Steps; ++i) load_unit(u_begin, i);
        }
        int staged = -1;
        for (int u = u_begin; u < u_end; ++u) {
            const int ai = u / kG1Units, g = u % kG1Units;
            const int e = sh->act_expert[ai], m = sh->act_m[ai];
            if (ai != staged) {
                __syncthreads();   // every warp is done with the previous expert's rows
                for (int i = tid; i < m * (kHidden / 16); i += kDecThreads) {
                    const int slot = i / (kHidden / 16), off = i % (kHidden / 16);
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.hidden + (size_t)sh->act_tok[ai][slot] * kHidden) + off);
                    *reinterpret_cast<uint4*>(sh->stage + slot * kHidStride + off * 16) = v;
                }
                for (int i = tid; i < m * kHiddenBlocks; i += kDecThreads) {
                    const int slot = i / kHiddenBlocks, kb = i % kHiddenBlocks;
                    sh->scale[slot][kb] = __ldg(a.hscale + (size_t)kb * T + sh->act_tok[ai][slot]);
                }
                __syncthreads();
                staged = ai;
            }
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float* s1l = a.s1 + ((size_t)e * (kGemm1Out / kBlock) + g / (kBlock / kG1Cols)) * kHiddenBlocks;
            const float* s1g = s1l + (size_t)(kInter / kBlock) * kHiddenBlocks;
#pragma unroll
            for (int i = 0; i < kG1Steps; ++i) {
                const int kb = warp + kDecWarps * i;
                if (kb < kHiddenBlocks) {
                    const uint8_t* brow = sh->stage + r * kHidStride + kb * kBlock + 16 * c;
                    uint4 b[2];
                    b[0] = *reinterpret_cast<const uint4*>(brow);
                    b[1] = *reinterpret_cast<const uint4*>(brow + 64);
                    float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_block(raw, wl[i], wg[i], b);
                    const float sl = __ldg(s1l + kb), sg = __ldg(s1g + kb);
                    const float sa0 = sh->scale[2 * c][kb], sa1 = sh->scale[2 * c + 1][kb];
                    acc[0] = fmaf(raw[0], sa0 * sl, acc[0]);
                    acc[1] = fmaf(raw[1], sa1 * sl, acc[1]);
                    acc[2] = fmaf(raw[2], sa0 * sg, acc[2]);
                    acc[3] = fmaf(raw[3], sa1 * sg, acc[3]);
                }
                if (u + 1 < u_end) load_unit(u + 1, i);   // the next unit's bytes fly during the reduction
            }
            float* red = &sh->red[u & 1][0][0];
            *reinterpret_cast<float4*>(red + warp * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            __syncthreads();
            if (tid < 64) {
                const int l = tid & 31, j = tid >> 5;
                float lin = 0.0f, gate = 0.0f;
#pragma unroll
                for (int w = 0; w < kDecWarps; ++w) {
                    lin += red[w * 128 + l * 4 + j];
                    gate += red[w * 128 + l * 4 + 2 + j];
                }
                const int slot = 2 * (l & 3) + j, col = g * kG1Cols + (l >> 2);
                if (slot < m) {
                    const float x1 = round_bf16(lin), x2 = round_bf16(gate);
                    const float silu = a.silu_exact ? x2 / (1.0f + __expf(-x2))
                                                    : x2 * (0.5f * (x2 * rsqrtf(fmaf(x2, x2, 4.0f)) + 1.0f));
                    act[(size_t)(sh->act_row0[ai] + slot) * kInter + col] = silu * x1;
                }
            }
        }
    }

    // ------------------------------------------------------------------ phase 2: requant + GEMM2
    {
        const int units = n_active * kG2Units;
        const int u_begin = (int)((long long)units * blockIdx.x / gridDim.x);
        const int u_end = (int)((long long)units * (blockIdx.x + 1) / gridDim.x);
        uint4 wl[2], wg[2];
        auto load_unit = [&](int u) {
            const int e = sh->act_expert[u / kG2Units];
            const int hrow = (u % kG2Units) * kG2Cols + r;
            const uint8_t* p = a.w2 + ((size_t)e * kHidden + hrow) * kInter + warp * kBlock + 16 * c;
            wl[0] = ld_stream(p);
            wl[1] = ld_stream(p + 64);
            wg[0] = ld_stream(p + (size_t)8 * kInter);
            wg[1] = ld_stream(p + (size_t)8 * kInter + 64);
        };
        if (u_begin < u_end) load_unit(u_begin);   // in flight across the barrier
        __threadfence();
        if (!grid_barrier(ws.ctrl, sh)) return;
        int staged = -1;
        for (int u = u_begin; u < u_end; ++u) {
            const int ai = u / kG2Units, hg = u % kG2Units;
            const int e = sh->act_expert[ai], m = sh->act_m[ai];
            if (ai != staged) {
                __syncthreads();
                // 1x128 requantisation of the expert's rows, as in the staged GEMM1 epilogue:
                // scale = amax / 448 (1 if the block is zero), payload e4m3(v * (1 / scale))
                for (int item = warp; item < m * kInterBlocks; item += kDecWarps) {
                    const int slot = item / kInterBlocks, ib = item % kInterBlocks;
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(
                        act + (size_t)(sh->act_row0[ai] + slot) * kInter + ib * kBlock) + lane);
                    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    const float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
                    const float inv = 1.0f / scale;
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v.x * inv, v.y * inv), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v.z * inv, v.w * inv), __NV_SATFINITE, __NV_E4M3);
                    *reinterpret_cast<uint32_t*>(sh->stage + slot * kA2Stride + ib * kBlock + lane * 4) = lo | (hi << 16);
                    if (lane == 0) sh->scale[slot][ib] = scale;
                }
                staged = ai;
            }
            if (tid < kInterBlocks)
                sh->w2_scale[u & 1][tid] = __ldg(a.s2 + ((size_t)e * kHiddenBlocks + hg / (kBlock / kG2Cols)) * kInterBlocks + tid);
            __syncthreads();   // rows, scales and the previous unit's reduction are settled
            {
                const uint8_t* brow = sh->stage + r * kA2Stride + warp * kBlock + 16 * c;
                uint4 b[2];
                b[0] = *reinterpret_cast<const uint4*>(brow);
                b[1] = *reinterpret_cast<const uint4*>(brow + 64);
                float raw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                mma_block(raw, wl, wg, b);
                *reinterpret_cast<float4*>(&sh->red[0][warp][lane * 4]) = make_float4(raw[0], raw[1], raw[2], raw[3]);
            }
            if (u + 1 < u_end) load_unit(u + 1);
            __syncthreads();
            if (tid < 128) {
                // the K blocks are promoted in order with one FMA each, like the staged kernel
                const int l = tid >> 2, i = tid & 3;
                const int slot = 2 * (l & 3) + (i & 1), hrow = hg * kG2Cols + (l >> 2) + 8 * (i >> 1);
                float acc = 0.0f;
#pragma unroll
                for (int kb = 0; kb < kInterBlocks; ++kb)
                    acc = fmaf(sh->red[0][kb][l * 4 + i], sh->scale[slot][kb] * sh->w2_scale[u & 1][kb], acc);
                if (slot < m) ws.y[(size_t)(sh->act_row0[ai] + slot) * kHidden + hrow] = __float2bfloat16_rn(acc);
            }
        }
    }

    // ------------------------------------------------------------------ phase 3: weighted combine
    __threadfence();
    if (!grid_barrier(ws.ctrl, sh)) return;
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

cudaError_t launch_decode_layer(const DecodeArgs& args, const Workspace& ws, int num_ctas, cudaStream_t stream)
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
    return cudaLaunchKernelEx(&cfg, decode_layer_kernel, args, ws);
}

}  // namespace moe
