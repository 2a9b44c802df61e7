// Per-token routing and the per-shard dispatch policy as device functions, shared by the
// routing kernel of the staged chain and by the single-kernel decode path.
#pragma once
#include "layer.cuh"

namespace moe {

// ---------------------------------------------------------------------------------------
// Routing.  Restates kernel/moe_fp8.cu:359-448 of the reference (sigmoid, +bias, group
// score = two largest of 32, 4 groups kept, 8 argmax rounds, weights from the unbiased
// sigmoid normalised by 1e-20 + their sum taken in selection order) so that indices and
// weights come out bit-identical.  The reference runs 256 threads per token with shared
// memory round trips; here lane l of one warp owns experts {32 w + l : w = 0..7} in
// registers and every reduction is a redux.sync over an order-preserving integer key.
//
// Tie order of the reference: inside a 32-expert warp its xor-butterfly with a strict
// `>` keeps the candidate whose lane index is smallest after 5-bit reversal
// (kernel/moe_fp8.cu:416-420), across warps the lowest warp wins
// (kernel/moe_fp8.cu:427-431).  `rank = w * 32 + bitrev5(lane)` reproduces that order.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t k) {
    const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

constexpr float kNegSentinel = -1e30f;

// Appends one kept (local expert, weight) pair to the token's list (static indexing keeps
// the lists in registers).
__device__ __forceinline__ void emit_pair(int (&p_le)[kTopK], float (&p_w)[kTopK], int& n, int le, float w) {
#pragma unroll
    for (int i = 0; i < kTopK; ++i) {
        if (i == n) { p_le[i] = le; p_w[i] = w; }
    }
    ++n;
}

// Applies the dispatch policy to the experts of token `t` that fall into shard `s`
// (local experts [32 s, 32 s + 32)) and appends the kept pairs.  Run by one lane.
__device__ __forceinline__ void dispatch_one_shard(
    const int (&idx)[kTopK], const float (&wn)[kTopK], int s, int local_expert_offset,
    const DispatchPolicy& pol, float rsf, int& n_pairs, int (&p_le)[kTopK], float (&p_w)[kTopK])
{
    const int lo = s * kShardExperts;
    if (!pol.prune) {
#pragma unroll
        for (int k = 0; k < kTopK; ++k) {
            const int le = idx[k] - local_expert_offset;
            if ((unsigned)(le - lo) < (unsigned)kShardExperts) {
                const float wk = wn[k];
                if (pol.skip_zero_weight && wk == 0.0f) continue;
                emit_pair(p_le, p_w, n_pairs, le, wk * rsf);
            }
        }
        return;
    }

    // Pruning dispatch: the three largest local weights in descending order by strict
    // insertion (kernel/moe_fp8.cu:477-507), then the drop rules (:508-577), the
    // renormalisation (:579-591) and emission in descending-weight order (:592-606).
    constexpr int kKeep = 3;
    int keep_le[kKeep];
    float keep_w[kKeep];
#pragma unroll
    for (int i = 0; i < kKeep; ++i) { keep_le[i] = -1; keep_w[i] = -1.0f; }
    int local_count = 0;
    float local_w_sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
        const int le = idx[k] - local_expert_offset;
        if ((unsigned)(le - lo) < (unsigned)kShardExperts) {
            const float wk = wn[k];
            ++local_count;
            local_w_sum += wk;
#pragma unroll
            for (int i = 0; i < kKeep; ++i) {
                if (wk > keep_w[i]) {
#pragma unroll
                    for (int j = kKeep - 1; j > i; --j) {
                        keep_w[j] = keep_w[j - 1];
                        keep_le[j] = keep_le[j - 1];
                    }
                    keep_w[i] = wk;
                    keep_le[i] = le;
                    break;
                }
            }
        }
    }
    if (local_count == 0) return;
    int max_keep = pol.keep_limit < kKeep ? pol.keep_limit : kKeep;
    if (pol.keep_limit >= 3 && local_count >= 3 && keep_le[2] >= 0 && local_w_sum > 0.0f) {
        if (pol.drop_third && keep_w[2] <= pol.drop_third_frac * local_w_sum) max_keep = 2;
    }
    if (pol.keep_limit >= 3 && local_count >= 2 && keep_le[1] >= 0 && local_w_sum > 0.0f) {
        const float frac = (local_count >= 3) ? pol.drop_second_frac_ge3 : pol.drop_second_frac_2;
        if (frac > 0.0f && keep_w[1] <= frac * local_w_sum) max_keep = 1;
    }
    float renorm = 1.0f;
    if (pol.renorm && local_count > max_keep) {
        float kept_w_sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            if (i < max_keep && keep_le[i] >= 0) kept_w_sum += keep_w[i];
        }
        if (kept_w_sum > 0.0f) renorm = local_w_sum / kept_w_sum;
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
        const int le = keep_le[i];
        if (i < max_keep && le >= 0) {
            emit_pair(p_le, p_w, n_pairs, le, keep_w[i] * renorm * rsf);
        }
    }
}

// Routes one token with one warp (all 32 lanes call it together): on return every lane holds
// the eight selected global expert ids in selection order and their normalised weights.
__device__ __forceinline__ void route_token_warp(const float* __restrict__ logits_row,
                                                 const __nv_bfloat16* __restrict__ bias, int lane,
                                                 int (&idx)[kTopK], float (&wn)[kTopK])
{
    constexpr uint32_t kFull = 0xffffffffu;
    float s[kNumGroups];   // unbiased sigmoid of expert 32 w + lane
    float sb[kNumGroups];  // biased score, later masked
#pragma unroll
    for (int w = 0; w < kNumGroups; ++w) {
        const float l = logits_row[w * 32 + lane];
        const float sig = 1.0f / (1.0f + __expf(-l));
        s[w] = sig;
        sb[w] = sig + __bfloat162float(bias[w * 32 + lane]);
    }

    // Group score: sum of the two largest biased scores of the group (duplicates count).
    float gscore[kNumGroups];
#pragma unroll
    for (int w = 0; w < kNumGroups; ++w) {
        const uint32_t key = float_to_ordered(sb[w]);
        const uint32_t k1 = __reduce_max_sync(kFull, key);
        const uint32_t holders = __ballot_sync(kFull, key == k1);
        uint32_t k2;
        if (__popc(holders) >= 2) {
            k2 = k1;
        } else {
            const uint32_t masked = (key == k1) ? 0u : key;
            k2 = __reduce_max_sync(kFull, masked);
        }
        gscore[w] = ordered_to_float(k1) + ordered_to_float(k2);
    }

    // Four best groups, lowest index first on ties (kernel/moe_fp8.cu:380-389).
    uint32_t kept_mask = 0;
#pragma unroll
    for (int k = 0; k < kTopKGroup; ++k) {
        float best = kNegSentinel;
        int best_i = -1;
#pragma unroll
        for (int i = 0; i < kNumGroups; ++i) {
            if (!((kept_mask >> i) & 1u) && gscore[i] > best) { best = gscore[i]; best_i = i; }
        }
        if (best_i >= 0) kept_mask |= 1u << best_i;
    }
#pragma unroll
    for (int w = 0; w < kNumGroups; ++w) {
        if (!((kept_mask >> w) & 1u)) sb[w] = kNegSentinel;
    }

    // Eight argmax rounds over the 256 masked scores.
    const uint32_t lane_rev = __brev((uint32_t)lane) >> 27;
    float sel[kTopK];
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
        float bv = sb[0];
        int bw = 0;
#pragma unroll
        for (int w = 1; w < kNumGroups; ++w) {
            if (sb[w] > bv) { bv = sb[w]; bw = w; }
        }
        const uint32_t key = float_to_ordered(bv);
        const uint32_t kmax = __reduce_max_sync(kFull, key);
        const uint32_t my_rank = (key == kmax) ? ((uint32_t)bw * 32u + lane_rev) : 0xffffffffu;
        const uint32_t win_rank = __reduce_min_sync(kFull, my_rank);
        const int win_w = (int)(win_rank >> 5);
        const int win_lane = (int)(__brev(win_rank & 31u) >> 27);
        float s_mine = 0.0f;
#pragma unroll
        for (int w = 0; w < kNumGroups; ++w) {
            if (w == win_w) {
                s_mine = s[w];
                if (lane == win_lane) sb[w] = kNegSentinel;
            }
        }
        sel[k] = __shfl_sync(kFull, s_mine, win_lane);
        idx[k] = win_w * 32 + win_lane;
    }

    float sumw = 1e-20f;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) sumw += sel[k];
    const float inv = 1.0f / sumw;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) wn[k] = sel[k] * inv;

}

// The same selection for other routing constants (FlashInfer's definition of the layer carries top_k,
// n_group and topk_group as axes; the reference compiles 8 / 8 / 4 in): n_group in {1, 2, 4, 8} groups of
// 256 / n_group experts -- a group is 8 / n_group of the warp's 32-expert slices -- scored by the sum of
// their two largest biased scores, topk_group groups kept, top_k <= 8 argmax rounds with the tie order of
// the routine above, weights normalised over the top_k picks.  Entries past top_k come back as expert -1
// with weight 0, which no dispatch takes for a local expert.
__device__ __forceinline__ void route_token_warp_generic(const float* __restrict__ logits_row,
                                                         const __nv_bfloat16* __restrict__ bias, int lane,
                                                         int (&idx)[kTopK], float (&wn)[kTopK], int n_group,
                                                         int topk_group, int top_k)
{
    constexpr uint32_t kFull = 0xffffffffu;
    float s[kNumGroups], sb[kNumGroups];
    uint32_t k1[kNumGroups], k2[kNumGroups];   // the two largest keys of each 32-expert slice (duplicates count)
#pragma unroll
    for (int w = 0; w < kNumGroups; ++w) {
        const float l = logits_row[w * 32 + lane];
        const float sig = 1.0f / (1.0f + __expf(-l));
        s[w] = sig;
        sb[w] = sig + __bfloat162float(bias[w * 32 + lane]);
        const uint32_t key = float_to_ordered(sb[w]);
        k1[w] = __reduce_max_sync(kFull, key);
        const uint32_t holders = __ballot_sync(kFull, key == k1[w]);
        k2[w] = (__popc(holders) >= 2) ? k1[w] : __reduce_max_sync(kFull, (key == k1[w]) ? 0u : key);
    }
    const int per = kNumGroups / n_group;   // slices per group
    float gscore[kNumGroups];
#pragma unroll
    for (int g = 0; g < kNumGroups; ++g) {
        uint32_t a = 0u, b = 0u;
#pragma unroll
        for (int w = 0; w < kNumGroups; ++w) {
            if (g < n_group && w / per == g) {
                const uint32_t t1 = a >= k1[w] ? a : k1[w];
                const uint32_t t2 = a >= k1[w] ? (b >= k1[w] ? b : k1[w]) : (a >= k2[w] ? a : k2[w]);
                a = t1;
                b = t2;
            }
        }
        gscore[g] = (g < n_group) ? ordered_to_float(a) + ordered_to_float(b) : kNegSentinel;
    }
    uint32_t kept_mask = 0;
    for (int k = 0; k < topk_group; ++k) {
        float best = kNegSentinel;
        int best_i = -1;
#pragma unroll
        for (int i = 0; i < kNumGroups; ++i) {
            if (i < n_group && !((kept_mask >> i) & 1u) && gscore[i] > best) { best = gscore[i]; best_i = i; }
        }
        if (best_i >= 0) kept_mask |= 1u << best_i;
    }
#pragma unroll
    for (int w = 0; w < kNumGroups; ++w) {
        if (!((kept_mask >> (w / per)) & 1u)) sb[w] = kNegSentinel;
    }
    const uint32_t lane_rev = __brev((uint32_t)lane) >> 27;
    float sel[kTopK];
#pragma unroll
    for (int k = 0; k < kTopK; ++k) {
        if (k < top_k) {
            float bv = sb[0];
            int bw = 0;
#pragma unroll
            for (int w = 1; w < kNumGroups; ++w) {
                if (sb[w] > bv) { bv = sb[w]; bw = w; }
            }
            const uint32_t key = float_to_ordered(bv);
            const uint32_t kmax = __reduce_max_sync(kFull, key);
            const uint32_t my_rank = (key == kmax) ? ((uint32_t)bw * 32u + lane_rev) : 0xffffffffu;
            const uint32_t win_rank = __reduce_min_sync(kFull, my_rank);
            const int win_w = (int)(win_rank >> 5);
            const int win_lane = (int)(__brev(win_rank & 31u) >> 27);
            float s_mine = 0.0f;
#pragma unroll
            for (int w = 0; w < kNumGroups; ++w) {
                if (w == win_w) {
                    s_mine = s[w];
                    if (lane == win_lane) sb[w] = kNegSentinel;
                }
            }
            sel[k] = __shfl_sync(kFull, s_mine, win_lane);
            idx[k] = win_w * 32 + win_lane;
        } else {
            sel[k] = 0.0f;
            idx[k] = -1;
        }
    }
    float sumw = 1e-20f;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) sumw += sel[k];
    const float inv = 1.0f / sumw;
#pragma unroll
    for (int k = 0; k < kTopK; ++k) wn[k] = sel[k] * inv;
}

}  // namespace moe
