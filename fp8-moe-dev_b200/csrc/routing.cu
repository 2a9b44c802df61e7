// Stage 1-3 of the layer: DeepSeek-V3 no-aux routing fused with the per-shard dispatch
// policy (one warp per token), the expert-offset scan that turns the per-expert row
// counters into 128-row tiles, and the token-centric permute that gathers e4m3 rows and
// their 1x128 scales into expert-contiguous order.  Nothing here reads a device value on
// the host, so the whole chain can sit in a CUDA graph.
#include "layer.cuh"
#include "ptx.cuh"
#include "route_token.cuh"

namespace moe {

// ---------------------------------------------------------------------------------------
// Offsets and tiles, run by the LAST routing CTA to finish (256 threads).  Every expert's
// row count is rounded up to 128, an exclusive scan gives the first packed row of each
// expert, and each 128-row tile gets its expert and its number of valid rows; the counters
// are then cleared for the next call.  (The reference does the scan in a separate one-warp
// kernel and then reads the totals back on the host, kernel/moe_fp8.cu:838-870, 2816-2824.)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void scan_tiles_block(const Workspace& ws, int num_local_experts, const int* local_counts)
{
    __shared__ int s_warp_total[kMaxLocalExperts / 32];
    const int e = threadIdx.x;
    const int lane = e & 31, warp = e >> 5;
    // single-CTA launches count in shared memory (local_counts); otherwise the counters were
    // written by other CTAs' atomics and are read past the L1
    int m = 0;
    if (e < num_local_experts) m = local_counts ? local_counts[e] : __ldcg(&ws.ctrl->expert_count[e]);
    const int k = (m + kTileM - 1) / kTileM;
    int incl = k;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += y;
    }
    if (lane == 31) s_warp_total[warp] = incl;
    __syncthreads();
    int warp_base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kMaxLocalExperts / 32; ++w) {
        const int t = s_warp_total[w];
        if (w < warp) warp_base += t;
        total += t;
    }
    const int base = warp_base + incl - k;  // exclusive prefix, in tiles
    const bool overflow = total > ws.max_tiles || total * kTileM > ws.m_cap;
    if (overflow) total = 0;
    if (e < num_local_experts) {
        ws.expert_offset[e] = overflow ? 0 : base * kTileM;
        ws.ctrl->expert_rows[e] = m;
        if (!local_counts) ws.ctrl->expert_count[e] = 0;
    }
    if (e < 8) ws.ctrl->xch_time[e] = (e == 0 || e == 2) ? ~0ull : 0ull;
    if (e == 0) {
        ws.expert_offset[num_local_experts] = total * kTileM;
        ws.num_tiles[0] = total;
        ws.ctrl->blocks_done = 0;
        // the status word is sticky: the first failure stays until the host has read it
        if (overflow && atomicCAS(&ws.ctrl->status, kStatusOk, kStatusRowOverflow) == kStatusOk)
            ws.ctrl->status_detail = warp_base + incl;
    }
    if (!overflow && e < num_local_experts) {
        const int4 info = make_int4(e, base, k, m);
        for (int j = 0; j < k; ++j) ws.tile_info[base + j] = info;
    }
}

constexpr int kRouteWarps = 8;

// GENERIC_ROUTE: the routing constants come from the policy record (top_k, n_group, topk_group) instead of
// the reference's 8 / 8 / 4.
template <bool GENERIC_ROUTE>
__global__ void __launch_bounds__(kRouteWarps * 32) route_dispatch_kernel(
    const float* __restrict__ logits, const __nv_bfloat16* __restrict__ bias, Workspace ws, int T,
    int local_expert_offset, int num_local_experts, float rsf, DispatchPolicy pol, int do_scan)
{
    // Rows are counted per CTA in shared memory first; one global atomic per (CTA, expert)
    // then reserves a contiguous slot range (a single-CTA launch needs no global atomic).
    __shared__ int s_cnt[kMaxLocalExperts];
    __shared__ int s_base[kMaxLocalExperts];
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRouteWarps + (threadIdx.x >> 5);
    const bool single_cta = do_scan && gridDim.x == 1;
    s_cnt[threadIdx.x] = 0;
    pdl_launch_dependents();
    pdl_wait();  // the previous call's kernels still read the pair tables and offsets
    __syncthreads();
    // Dispatch is spread over the warp: lane s applies the policy to the token's experts that fall into
    // 32-expert shard s (the reference does one shard per call; a handle with 64..256 experts, or one with
    // a strided / table placement, has up to eight).  A lane's kept pairs follow those of the lanes before
    // it, so the token's pair list is in shard order, then in the policy's emission order, exactly as a
    // serial walk over the shards would leave it.
    int n_pairs = 0, pair_base = 0, total_pairs = 0;
    int p_le[kTopK], p_rank[kTopK];
    float p_w[kTopK];
#pragma unroll
    for (int i = 0; i < kTopK; ++i) { p_le[i] = 0; p_rank[i] = 0; p_w[i] = 0.0f; }
    if (t < T) {

    int idx[kTopK];
    float wn[kTopK];
    if (GENERIC_ROUTE)
        route_token_warp_generic(logits + (size_t)t * kNumExperts, bias, lane, idx, wn, pol.n_group, pol.topk_group, pol.top_k);
    else
        route_token_warp(logits + (size_t)t * kNumExperts, bias, lane, idx, wn);

    if (lane < kTopK) {
        int my_idx = 0;
        float my_w = 0.0f;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) {
            if (k == lane) { my_idx = idx[k]; my_w = wn[k]; }
        }
        ws.topk_idx[(size_t)t * kTopK + lane] = my_idx;
        ws.topk_weight[(size_t)t * kTopK + lane] = my_w;
    }

    const bool contiguous = pol.expert_stride == 0 || pol.expert_stride == 1;
    const int n_shards = contiguous ? num_local_experts / kShardExperts : kNumExperts / kShardExperts;
    if (lane < n_shards) {
        if (contiguous) {
            dispatch_one_shard(idx, wn, lane, local_expert_offset, pol, rsf, n_pairs, p_le, p_w);
        } else {
            // strided or table placement: the policy runs on a global shard, this rank keeps its experts
            int n_sh = 0;
            int g_le[kTopK];
            float g_w[kTopK];
#pragma unroll
            for (int i = 0; i < kTopK; ++i) { g_le[i] = 0; g_w[i] = 0.0f; }
            dispatch_one_shard(idx, wn, lane, 0, pol, rsf, n_sh, g_le, g_w);
#pragma unroll
            for (int i = 0; i < kTopK; ++i) {
                if (i < n_sh) {
                    const int local = pol.expert_stride > 1
                                          ? (g_le[i] % pol.expert_stride == pol.expert_phase ? g_le[i] / pol.expert_stride : -1)
                                          : __ldg(ws.expert_map + g_le[i]);
                    if (local >= 0) emit_pair(p_le, p_w, n_pairs, local, g_w[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kTopK; ++i) {
            if (i < n_pairs) p_rank[i] = atomicAdd(&s_cnt[p_le[i]], 1);
        }
    }
    // exclusive prefix of the lanes' pair counts (lanes at or above n_shards hold 0)
    int incl = n_pairs;
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += y;
    }
    pair_base = incl - n_pairs;
    total_pairs = __shfl_sync(0xffffffffu, incl, 7);
    }  // t < T

    __syncthreads();
    {
        const int e = threadIdx.x;
        int base = 0;
        if (!single_cta && e < num_local_experts) {
            const int c = s_cnt[e];
            if (c > 0) base = atomicAdd(&ws.ctrl->expert_count[e], c);
        }
        s_base[e] = base;
    }
    __syncthreads();
    if (t < T) {
#pragma unroll
        for (int i = 0; i < kTopK; ++i) {
            if (i < n_pairs) {
                const uint32_t slot = (uint32_t)(s_base[p_le[i]] + p_rank[i]);
                ws.pair_code[(size_t)t * kTopK + pair_base + i] = ((uint32_t)p_le[i] << 24) | slot;
                ws.pair_weight[(size_t)t * kTopK + pair_base + i] = p_w[i];
            }
        }
        if (lane == 0) ws.pair_count[t] = total_pairs;
    }

    if (!do_scan) return;
    if (single_cta) {
        scan_tiles_block(ws, num_local_experts, s_cnt);
        return;
    }
    // Last CTA to get here turns the counters into offsets and tiles.
    __shared__ int s_is_last;
    if (threadIdx.x == 0) {
        __threadfence();
        const int ticket = atomicAdd(&ws.ctrl->blocks_done, 1);
        s_is_last = (ticket == (int)gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_is_last) {
        __threadfence();
        scan_tiles_block(ws, num_local_experts, nullptr);
    }
}

// ---------------------------------------------------------------------------------------
// Permute.  One warp per token: the 7168-byte e4m3 row is read once (14 x 16 B per lane)
// and written to each packed row the token owns; the 56 scales move from the [56, T]
// input layout to the [56, M_cap] packed layout.  Same data movement as the reference's
// row-centric kernel/moe_fp8.cu:1064-1115, without an [E, T] token list.
// ---------------------------------------------------------------------------------------
constexpr int kPermuteWarps = 4;

__global__ void __launch_bounds__(kPermuteWarps * 32) permute_rows_kernel(
    const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale, Workspace ws, int T)
{
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kPermuteWarps + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T) return;
    const int n_pairs = (ws.num_tiles[0] == 0) ? 0 : ws.pair_count[t];
    if (lane < kTopK) {   // the token's packed rows, for the fused exchange
        int r = -1;
        if (lane < n_pairs) {
            const uint32_t code = ws.pair_code[(size_t)t * kTopK + lane];
            r = ws.expert_offset[code >> 24] + (int)(code & 0x00ffffffu);
        }
        ws.pair_row[(size_t)t * kTopK + lane] = r;
    }
    if (n_pairs == 0) return;

    constexpr int kVec = kHidden / 16 / 32;  // 14 uint4 per lane
    uint4 v[kVec];
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden);
#pragma unroll
    for (int i = 0; i < kVec; ++i) v[i] = __ldg(src + lane + 32 * i);
    const float sc0 = __ldg(hidden_scale + (size_t)lane * T + t);
    const float sc1 = (lane + 32 < kHiddenBlocks) ? __ldg(hidden_scale + (size_t)(lane + 32) * T + t) : 0.0f;

    for (int p = 0; p < n_pairs; ++p) {
        const uint32_t code = ws.pair_code[(size_t)t * kTopK + p];
        const int le = (int)(code >> 24);
        const int slot = (int)(code & 0x00ffffffu);
        const int row = ws.expert_offset[le] + slot;
        uint4* dst = reinterpret_cast<uint4*>(ws.a1 + (size_t)row * kHidden);
#pragma unroll
        for (int i = 0; i < kVec; ++i) dst[lane + 32 * i] = v[i];
        ws.sfa1[(size_t)lane * ws.m_cap + row] = sc0;
        if (lane + 32 < kHiddenBlocks) ws.sfa1[(size_t)(lane + 32) * ws.m_cap + row] = sc1;
        if (lane == 0) ws.row_token[row] = t;
    }
}

// The same movement for a run-time row length (Workspace::geo.hidden, a multiple of 256 bytes): the row
// is re-read per packed row it goes to (it sits in L1 after the first pass).
__global__ void __launch_bounds__(kPermuteWarps * 32) permute_rows_generic_kernel(
    const uint8_t* __restrict__ hidden, const float* __restrict__ hidden_scale, Workspace ws, int T)
{
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kPermuteWarps + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T) return;
    const int n_pairs = (ws.num_tiles[0] == 0) ? 0 : ws.pair_count[t];
    if (lane < kTopK) {
        int r = -1;
        if (lane < n_pairs) {
            const uint32_t code = ws.pair_code[(size_t)t * kTopK + lane];
            r = ws.expert_offset[code >> 24] + (int)(code & 0x00ffffffu);
        }
        ws.pair_row[(size_t)t * kTopK + lane] = r;
    }
    if (n_pairs == 0) return;
    const int H = ws.geo.hidden;
    const int vecs = H / 16, blocks = H / kBlock;   // <= 512 uint4, <= 64 scales
    const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * H);
    const float sc0 = (lane < blocks) ? __ldg(hidden_scale + (size_t)lane * T + t) : 0.0f;
    const float sc1 = (lane + 32 < blocks) ? __ldg(hidden_scale + (size_t)(lane + 32) * T + t) : 0.0f;
    for (int p = 0; p < n_pairs; ++p) {
        const uint32_t code = ws.pair_code[(size_t)t * kTopK + p];
        const int row = ws.expert_offset[code >> 24] + (int)(code & 0x00ffffffu);
        uint4* dst = reinterpret_cast<uint4*>(ws.a1 + (size_t)row * H);
        for (int i = lane; i < vecs; i += 32) dst[i] = __ldg(src + i);
        if (lane < blocks) ws.sfa1[(size_t)lane * ws.m_cap + row] = sc0;
        if (lane + 32 < blocks) ws.sfa1[(size_t)(lane + 32) * ws.m_cap + row] = sc1;
        if (lane == 0) ws.row_token[row] = t;
    }
}

// ---------------------------------------------------------------------------------------
// Combine.  out[t, :] = bf16( sum_p float(Y[row_p, :]) * w_p ) with the pairs taken in
// dispatch order and fp32 accumulation; tokens without a local expert get zeros.  Same
// arithmetic as kernel/moe_fp8.cu:2276-2321.
// ---------------------------------------------------------------------------------------
constexpr int kCombineThreads = 448;  // 448 threads x 2 x 8 columns = 7168

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(Workspace ws, __nv_bfloat16* __restrict__ out, int T)
{
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T) return;
    int n_pairs = ws.pair_count[t];
    if (ws.num_tiles[0] == 0) n_pairs = 0;
    float acc[2][8];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[c][j] = 0.0f;

    for (int p = 0; p < n_pairs; ++p) {
        const uint32_t code = ws.pair_code[(size_t)t * kTopK + p];
        const float w = ws.pair_weight[(size_t)t * kTopK + p];
        const int row = ws.expert_offset[code >> 24] + (int)(code & 0x00ffffffu);
        const uint4* src = reinterpret_cast<const uint4*>(ws.y + (size_t)row * kHidden);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint4 raw = __ldg(src + threadIdx.x + c * kCombineThreads);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h2[j]);
                acc[c][2 * j] += f.x * w;
                acc[c][2 * j + 1] += f.y * w;
            }
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * kHidden);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint4 packed;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(acc[c][2 * j], acc[c][2 * j + 1]);
        dst[threadIdx.x + c * kCombineThreads] = packed;
    }
}

// Run-time row length: a thread walks 8-column chunks, each summed over the pairs in the same order.
__global__ void __launch_bounds__(256) combine_generic_kernel(Workspace ws, __nv_bfloat16* __restrict__ out, int T)
{
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (t >= T) return;
    int n_pairs = ws.pair_count[t];
    if (ws.num_tiles[0] == 0) n_pairs = 0;
    const int H = ws.geo.hidden;
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)t * H);
    for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int p = 0; p < n_pairs; ++p) {
            const uint32_t code = ws.pair_code[(size_t)t * kTopK + p];
            const float w = ws.pair_weight[(size_t)t * kTopK + p];
            const int row = ws.expert_offset[code >> 24] + (int)(code & 0x00ffffffu);
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(ws.y + (size_t)row * H) + v);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h2[j]);
                acc[2 * j] += f.x * w;
                acc[2 * j + 1] += f.y * w;
            }
        }
        uint4 packed;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        dst[v] = packed;
    }
}

// ---------------------------------------------------------------------------------------
// Launchers (called by the C-ABI layer).  All launches carry the programmatic stream
// serialization attribute (see ptx.cuh).
// ---------------------------------------------------------------------------------------
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args)
{
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
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

cudaError_t launch_route_dispatch(const float* logits, const void* bias, const Workspace& ws, int T,
                                  int local_expert_offset, int num_local_experts, float rsf,
                                  const DispatchPolicy& pol, int do_scan, cudaStream_t stream)
{
    const int grid = (T + kRouteWarps - 1) / kRouteWarps;
    if (pol.top_k != 0)
        return launch_pdl(route_dispatch_kernel<true>, dim3(grid), dim3(kRouteWarps * 32), 0, stream, logits,
                          static_cast<const __nv_bfloat16*>(bias), ws, T, local_expert_offset, num_local_experts, rsf, pol,
                          do_scan);
    return launch_pdl(route_dispatch_kernel<false>, dim3(grid), dim3(kRouteWarps * 32), 0, stream, logits,
                      static_cast<const __nv_bfloat16*>(bias), ws, T, local_expert_offset, num_local_experts, rsf, pol,
                      do_scan);
}

cudaError_t launch_permute(const void* hidden, const float* hidden_scale, const Workspace& ws, int T,
                           cudaStream_t stream)
{
    const int grid = (T + kPermuteWarps - 1) / kPermuteWarps;
    if (!ws.geo.is_reference())
        return launch_pdl(permute_rows_generic_kernel, dim3(grid), dim3(kPermuteWarps * 32), 0, stream,
                          static_cast<const uint8_t*>(hidden), hidden_scale, ws, T);
    return launch_pdl(permute_rows_kernel, dim3(grid), dim3(kPermuteWarps * 32), 0, stream,
                      static_cast<const uint8_t*>(hidden), hidden_scale, ws, T);
}

cudaError_t launch_combine(const Workspace& ws, void* out, int T, cudaStream_t stream)
{
    if (!ws.geo.is_reference())
        return launch_pdl(combine_generic_kernel, dim3(T), dim3(256), 0, stream, ws, static_cast<__nv_bfloat16*>(out), T);
    return launch_pdl(combine_kernel, dim3(T), dim3(kCombineThreads), 0, stream, ws, static_cast<__nv_bfloat16*>(out),
                      T);
}


// ---------------------------------------------------------------------------------------
// Fused combine + reduce-scatter over NVLink (no counterpart in the reference, which has no
// multi-GPU code).  Instead of writing its partial [T, 7168] output locally and handing it to
// a collective, every rank writes each weighted row sum straight into the receive buffer of
// the rank that owns the token (plain peer stores; rows of tokens without a local expert are
// not sent at all, only a one-byte "absent" mark), then raises a per-source epoch flag on
// every peer.  The owner waits (bounded) for all sources' flags and adds the rows that are
// present, in rank order, in fp32.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Select without dynamic indexing: the view is a kernel parameter, and indexing its pointer
// array with a run-time value would make the compiler copy it to local memory.
__device__ __forceinline__ uint8_t* peer_ptr(const ExchangeView& ex, int i) {
    uint8_t* p = ex.peer[0];
#pragma unroll
    for (int k = 1; k < kMaxRanks; ++k)
        if (i == k) p = ex.peer[k];
    return p;
}

// A token's rows here and their weights: two 32-byte loads from the tables the permute kernel left behind
// (row -1 = no such pair), one round trip instead of the chain pair count -> pair code -> expert offset.
struct PairTable {
    int4 row[2];
    float4 weight[2];
};
__device__ __forceinline__ PairTable load_pair_table(const Workspace& ws, int t) {
    PairTable p;
    const int4* r = reinterpret_cast<const int4*>(ws.pair_row + (size_t)t * kTopK);
    const float4* w = reinterpret_cast<const float4*>(ws.pair_weight + (size_t)t * kTopK);
    p.row[0] = __ldg(r);
    p.row[1] = __ldg(r + 1);
    p.weight[0] = __ldg(w);
    p.weight[1] = __ldg(w + 1);
    return p;
}

__global__ void __launch_bounds__(kCombineThreads, 2) combine_push_kernel(Workspace ws, ExchangeView ex, int T)
{
    pdl_launch_dependents();
    pdl_wait();
    const int parity = (int)(ex.epoch & 1u);
    const bool any_tiles = ws.num_tiles[0] != 0;
    if (threadIdx.x == 0) atomicMin(&ws.ctrl->xch_time[0], global_timer_ns());
    // Persistent CTAs walk the tokens destination by destination in turn -- index i goes to rank
    // (rank + 1 + i mod world) -- so that stores to every peer and the local rows (which cost HBM, not
    // NVLink, bandwidth) are under way at the same time.  One system-scope fence per CTA, after its last
    // store, instead of one per token.
    const int span = ex.tokens_per_rank * ex.world;
    auto token_of = [&](int i) {
        const int dest = (ex.rank + 1 + i % ex.world) % ex.world;
        return dest * ex.tokens_per_rank + i / ex.world;
    };
    // the next token's table travels while this token's rows are summed and stored
    PairTable next;
    {
        const int t0 = token_of(blockIdx.x);
        if (t0 < T) next = load_pair_table(ws, t0);
    }
    for (int i = blockIdx.x; i < span; i += gridDim.x) {
        const int t = token_of(i);
        const PairTable cur = next;
        if (i + (int)gridDim.x < span) {
            const int tn = token_of(i + gridDim.x);
            if (tn < T) next = load_pair_table(ws, tn);
        }
        if (t >= T) continue;
        const int rows[kTopK] = {cur.row[0].x, cur.row[0].y, cur.row[0].z, cur.row[0].w,
                                 cur.row[1].x, cur.row[1].y, cur.row[1].z, cur.row[1].w};
        const float wts[kTopK] = {cur.weight[0].x, cur.weight[0].y, cur.weight[0].z, cur.weight[0].w,
                                  cur.weight[1].x, cur.weight[1].y, cur.weight[1].z, cur.weight[1].w};
        const bool has_rows = any_tiles && rows[0] >= 0;   // pairs are packed from entry 0
        const int owner = t / ex.tokens_per_rank;
        const int tl = t - owner * ex.tokens_per_rank;
        uint8_t* dst_base = peer_ptr(ex, owner) + ex.data_offset;
        if (has_rows) {
            float acc[2][8];
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[c][j] = 0.0f;
            // the rows of four pairs are requested together, then added in pair order
#pragma unroll
            for (int p0 = 0; p0 < kTopK; p0 += 4) {
                if (rows[p0] < 0) break;
                uint4 raw[4][2];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (rows[p0 + u] >= 0) {
                        const uint4* src = reinterpret_cast<const uint4*>(ws.y + (size_t)rows[p0 + u] * kHidden);
                        raw[u][0] = __ldg(src + threadIdx.x);
                        raw[u][1] = __ldg(src + threadIdx.x + kCombineThreads);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (rows[p0 + u] >= 0) {
                        const float w = wts[p0 + u];
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u][c]);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __bfloat1622float2(h2[j]);
                                acc[c][2 * j] += f.x * w;
                                acc[c][2 * j + 1] += f.y * w;
                            }
                        }
                    }
                }
            }
            uint4* dst = reinterpret_cast<uint4*>(dst_base + (size_t)parity * ex.rows_bytes_per_parity +
                                                  ((size_t)ex.rank * ex.slot_rows + tl) * (kHidden * 2));
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint4 packed;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(acc[c][2 * j], acc[c][2 * j + 1]);
                dst[threadIdx.x + c * kCombineThreads] = packed;
            }
        }
        if (threadIdx.x == 0) {
            uint8_t* present = dst_base + 2 * ex.rows_bytes_per_parity + (size_t)parity * ex.present_bytes_per_parity +
                               (size_t)ex.rank * ex.present_stride + tl;
            *present = has_rows ? 1 : 0;
        }
    }
    // All of this CTA's peer stores become visible system-wide before it takes its ticket; the
    // last CTA then publishes this rank's epoch on every peer.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&ws.ctrl->push_done, 1);
        if (ticket == (int)gridDim.x - 1) {
            ws.ctrl->push_done = 0;
            // one system-scope fence, then the flags as relaxed stores (fence + relaxed store is a release
            // pattern): they leave back to back instead of each waiting for the one before it
            __threadfence_system();
            for (int o = 0; o < ex.world; ++o) {
                uint32_t* flag = reinterpret_cast<uint32_t*>(peer_ptr(ex, o)) + ex.rank;
                st_relaxed_sys_u32(flag, ex.epoch);
            }
            ws.ctrl->xch_time[1] = global_timer_ns();
        }
    }
}

__global__ void __launch_bounds__(kCombineThreads) reduce_owned_kernel(Workspace ws, ExchangeView ex, int T,
                                                                       __nv_bfloat16* __restrict__ out)
{
    const int tl = blockIdx.x;   // token owned by this rank
    pdl_launch_dependents();
    pdl_wait();
    const int parity = (int)(ex.epoch & 1u);
    uint8_t* const mine_base = peer_ptr(ex, ex.rank);
    const uint8_t* mine = mine_base + ex.data_offset;
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        // bounded wait for every source's epoch flag (a peer that never arrives must not hang us)
        const uint32_t* flags = reinterpret_cast<const uint32_t*>(mine_base);
        int ok = 1;
        const uint64_t t0 = global_timer_ns();
        atomicMin(&ws.ctrl->xch_time[2], (unsigned long long)t0);
        const uint64_t limit_ns = (uint64_t)ex.wait_limit_us * 1000ull;
        for (int src = 0; src < ex.world; ++src) {
            uint32_t it = 0;
            // epochs only grow; the signed difference also survives wrap-around
            while ((int32_t)(ld_acquire_sys_u32(flags + src) - ex.epoch) < 0) {
                if ((++it & 0x3fu) == 0u && global_timer_ns() - t0 > limit_ns) { ok = 0; break; }
            }
            if (!ok) break;
        }
        if (!ok) atomicCAS(&ws.ctrl->status, kStatusOk, kStatusExchangeTimeout);
        atomicMax(&ws.ctrl->xch_time[3], (unsigned long long)global_timer_ns());
        s_ok = ok;
    }
    __syncthreads();
    const int t = ex.rank * ex.tokens_per_rank + tl;
    if (t >= T) return;
    float acc[2][8];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[c][j] = 0.0f;
    if (s_ok) {
        const uint8_t* present = mine + 2 * ex.rows_bytes_per_parity + (size_t)parity * ex.present_bytes_per_parity + tl;
        for (int src = 0; src < ex.world; ++src) {
            if (present[(size_t)src * ex.present_stride] == 0) continue;
            const uint4* row = reinterpret_cast<const uint4*>(mine + (size_t)parity * ex.rows_bytes_per_parity +
                                                              ((size_t)src * ex.slot_rows + tl) * (kHidden * 2));
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 raw = row[threadIdx.x + c * kCombineThreads];
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h2[j]);
                    acc[c][2 * j] += f.x;
                    acc[c][2 * j + 1] += f.y;
                }
            }
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)tl * kHidden);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        uint4 packed;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(acc[c][2 * j], acc[c][2 * j + 1]);
        dst[threadIdx.x + c * kCombineThreads] = packed;
    }
    if (threadIdx.x == 0) atomicMax(&ws.ctrl->xch_time[4], (unsigned long long)global_timer_ns());
}

// ---------------------------------------------------------------------------------------
// Hand-shake for staging buffers that the ranks fill in each other's memory with copy engines (the
// host-resident form of the layer: every rank brings its token slice over PCIe and stores it into every
// peer's input staging over NVLink, no SM involved).  signal: this rank's word of every peer's flag
// array takes `value` (release, system scope; the copies before it in the stream have completed).  wait:
// bounded spin until every rank's word in the LOCAL array has reached `value`; a peer that does not
// arrive leaves kStatusExchangeTimeout in the status word, not a hung GPU.
// ---------------------------------------------------------------------------------------
__global__ void signal_peers_kernel(ExchangeView ex, size_t flag_offset, uint32_t value)
{
    if (threadIdx.x < (unsigned)ex.world) {
        __threadfence_system();
        uint32_t* flag = reinterpret_cast<uint32_t*>(peer_ptr(ex, threadIdx.x) + flag_offset) + ex.rank;
        st_release_sys_u32(flag, value);
    }
}

__global__ void wait_peers_kernel(ExchangeView ex, size_t flag_offset, uint32_t value, Control* ctrl)
{
    if (threadIdx.x < (unsigned)ex.world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(peer_ptr(ex, ex.rank) + flag_offset) + threadIdx.x;
        const uint64_t t0 = global_timer_ns();
        const uint64_t limit_ns = (uint64_t)ex.wait_limit_us * 1000ull;
        uint32_t it = 0;
        while ((int32_t)(ld_acquire_sys_u32(flag) - value) < 0) {
            if ((++it & 0x3fu) == 0u && global_timer_ns() - t0 > limit_ns) {
                atomicCAS(&ctrl->status, kStatusOk, kStatusExchangeTimeout);
                break;
            }
        }
    }
}

cudaError_t launch_signal_peers(const ExchangeView& ex, size_t flag_offset, uint32_t value, cudaStream_t stream)
{
    signal_peers_kernel<<<1, 32, 0, stream>>>(ex, flag_offset, value);
    return cudaGetLastError();
}
cudaError_t launch_wait_peers(const ExchangeView& ex, size_t flag_offset, uint32_t value, Control* ctrl, cudaStream_t stream)
{
    wait_peers_kernel<<<1, 32, 0, stream>>>(ex, flag_offset, value, ctrl);
    return cudaGetLastError();
}

cudaError_t launch_combine_push(const Workspace& ws, const ExchangeView& ex, int T, cudaStream_t stream)
{
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    const int span = ex.tokens_per_rank * ex.world;
    const int grid = span < sms * 2 ? span : sms * 2;   // two resident CTAs per SM
    return launch_pdl(combine_push_kernel, dim3(grid), dim3(kCombineThreads), 0, stream, ws, ex, T);
}
cudaError_t launch_reduce_owned(const Workspace& ws, const ExchangeView& ex, int T, void* out, cudaStream_t stream)
{
    return launch_pdl(reduce_owned_kernel, dim3(ex.tokens_per_rank), dim3(kCombineThreads), 0, stream, ws, ex, T,
                      static_cast<__nv_bfloat16*>(out));
}
}  // namespace moe
