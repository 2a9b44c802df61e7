// C ABI of the layer (declared in include/moe_fp8_b200.h): handle + workspace, argument
// validation, the reference's T-keyed dispatch policy resolved on the host, and the
// stage chain enqueued on the caller's stream.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "../../include/moe_fp8_b200.h"
#include "decode.cuh"
#include "layer.cuh"

namespace moe {
cudaError_t launch_route_dispatch(const float*, const void*, const Workspace&, int, int, int, float,
                                  const DispatchPolicy&, int, cudaStream_t);
cudaError_t launch_permute(const void*, const float*, const Workspace&, int, cudaStream_t);
cudaError_t launch_combine(const Workspace&, void*, int, cudaStream_t);
cudaError_t launch_quantize_rows(const void*, void*, float*, int, int, cudaStream_t);
cudaError_t launch_combine_push(const Workspace&, const ExchangeView&, int, cudaStream_t);
cudaError_t launch_reduce_owned(const Workspace&, const ExchangeView&, int, void*, cudaStream_t);
cudaError_t launch_signal_peers(const ExchangeView&, size_t, uint32_t, cudaStream_t);
cudaError_t launch_wait_peers(const ExchangeView&, size_t, uint32_t, Control*, cudaStream_t);
int encode_kmajor_u8_map(void*, const void*, uint64_t, uint64_t, uint64_t, uint32_t);
int encode_rows_1k_map(void*, const void*, uint64_t, uint64_t, uint32_t);
int encode_out_bf16_map(void*, void*, uint64_t, uint64_t);
size_t tensor_map_bytes();
cudaError_t configure_gemm_kernels();
cudaError_t launch_grouped_gemm(int, const void*, const void*, const void*, const Workspace&, const float*, int, int, int, int,
                                cudaStream_t);
int gemm_tiles_n(int mode, const Geometry& geo);
size_t packed_scale_floats(int mode, int num_experts, const Geometry& geo);
cudaError_t launch_repack_weight_scales(const float*, const float*, float*, float*, int, const Geometry&, cudaStream_t);
cudaError_t launch_tile_weights(int, const void*, void*, int, const Geometry&, int, cudaStream_t);
}  // namespace moe

using namespace moe;

namespace {

constexpr int kVersion = (0 << 16) | 1;
thread_local std::string g_create_error;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int row_capacity(int max_tokens, int num_local_experts)
{
    const long long pairs = 8LL * max_tokens;
    const long long nonempty = pairs < num_local_experts ? pairs : num_local_experts;
    long long cap = pairs + 127LL * nonempty;
    cap = (cap + kTileM - 1) / kTileM * kTileM;
    if (cap < kTileM) cap = kTileM;
    return (int)cap;
}

struct Carve {
    size_t off = 0;
    size_t take(size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 1024);
        return o;
    }
};

struct Layout {
    size_t ctrl, expert_offset, tile_info, num_tiles, expert_map, topk_idx, topk_weight, pair_count, pair_code,
        pair_weight, pair_row, row_token, a1, sfa1, a2, sfa2, y, splitk, sw1_packed, sw2_packed, total;
    int m_cap, max_tiles;
};

constexpr Geometry kReferenceGeometry = {kHidden, kInter};

Layout make_layout(int T, int E, const Geometry& geo = kReferenceGeometry)
{
    const size_t hidden = (size_t)geo.hidden, inter = (size_t)geo.inter;
    Layout L;
    L.m_cap = row_capacity(T, E);
    L.max_tiles = L.m_cap / kTileM;
    Carve c;
    L.ctrl = c.take(sizeof(Control));
    L.expert_offset = c.take(sizeof(int) * (kMaxLocalExperts + 1));
    L.tile_info = c.take(sizeof(int4) * L.max_tiles);
    L.num_tiles = c.take(sizeof(int) * 4);
    L.expert_map = c.take(sizeof(int) * kNumExperts);
    L.topk_idx = c.take(sizeof(int) * (size_t)T * kTopK);
    L.topk_weight = c.take(sizeof(float) * (size_t)T * kTopK);
    L.pair_count = c.take(sizeof(int) * (size_t)T);
    L.pair_code = c.take(sizeof(uint32_t) * (size_t)T * kTopK);
    L.pair_weight = c.take(sizeof(float) * (size_t)T * kTopK);
    L.pair_row = c.take(sizeof(int) * (size_t)T * kTopK);
    L.row_token = c.take(sizeof(int) * (size_t)L.m_cap);
    L.a1 = c.take((size_t)L.m_cap * hidden);
    L.sfa1 = c.take(sizeof(float) * (hidden / kBlock) * L.m_cap);
    L.a2 = c.take((size_t)L.m_cap * inter);
    L.sfa2 = c.take(sizeof(float) * (inter / kBlock) * L.m_cap);
    L.y = c.take(sizeof(__nv_bfloat16) * (size_t)L.m_cap * hidden);
    L.splitk = c.take(sizeof(float) * (size_t)kSplitKSlots * 4 * 256);  // kSplitKMaxRows rows of 256 floats per unit
    L.sw1_packed = c.take(sizeof(float) * packed_scale_floats(1, E, geo));
    L.sw2_packed = c.take(sizeof(float) * packed_scale_floats(2, E, geo));
    L.total = c.off;
    return L;
}

}  // namespace

struct moe_fp8_b200_ctx {
    int device = 0;
    int max_tokens = 0;
    int num_local_experts = 0;
    int num_sms = 0;
    Geometry geo = {kHidden, kInter};
    int top_k = kTopK, n_group = kNumGroups, topk_group = kTopKGroup;
    bool reference_routing() const { return top_k == kTopK && n_group == kNumGroups && topk_group == kTopKGroup; }
    int opt_reference_pruning = 1;
    int opt_exact_silu = 0;
    bool counters_dirty = false;
    int opt_stop_after = 0;   // diagnostics: enqueue only the first N stages (0 = all)
    int opt_decode = 1;       // single-kernel path for batches of at most kDecodeMaxTokens tokens
    int opt_expert_stride = 1;   // > 1: strided expert placement (multi-GPU wrapper)
    bool expert_map_set = false; // table placement (set_expert_map) overrides the stride while set
    int opt_wait_limit_us = 1000000;   // bound of the exchange's wait for peer flags
    int decode_ctas_per_sm = 0;
    uint8_t* base = nullptr;
    Layout layout{};
    Workspace ws{};
    alignas(64) unsigned char tmap_a1[128];
    alignas(64) unsigned char tmap_a2[128];
    alignas(64) unsigned char tmap_a1_small[128];   // the same tensors with a 64-row box (batches of at most 64 tokens)
    alignas(64) unsigned char tmap_a2_small[128];
    int opt_small_batch_ring = 1;
    alignas(64) unsigned char tmap_y[128];    // GEMM2's staged output stores
    alignas(64) unsigned char tmap_w1[128];
    alignas(64) unsigned char tmap_w2[128];
    alignas(64) unsigned char tmap_dec_w1[128];   // the decode kernel's views of the same weights
    alignas(64) unsigned char tmap_dec_w2[128];
    const void* cached_w1 = nullptr;
    const void* cached_w2 = nullptr;
    // tile-ordered copies of the weights for the chain's GEMMs (MOE_FP8_B200_OPT_WEIGHT_PRELAYOUT):
    // allocated when the option is switched on, filled once per weight pointer
    int opt_weight_prelayout = 0;
    uint8_t* w1_tiled = nullptr;
    uint8_t* w2_tiled = nullptr;
    const void* tiled_src1 = nullptr;
    const void* tiled_src2 = nullptr;
    alignas(64) unsigned char tmap_w1_tiled[128];
    alignas(64) unsigned char tmap_w2_tiled[128];
    // weight scales in the promotion's order (made once per pair of scale tensors, remembered by address)
    float* sw1_packed = nullptr;
    float* sw2_packed = nullptr;
    const float* cached_s1 = nullptr;
    const float* cached_s2 = nullptr;
    // optional per-stage timing: events around each stage of the last kTimedRuns runs
    int opt_stage_timing = 0;
    static constexpr int kTimedRuns = 64;
    static constexpr int kStageEvents = 7;
    cudaEvent_t events[kTimedRuns][kStageEvents] = {};
    bool events_created = false;
    int timed_runs = 0;
    // staging for run_host (allocated on its first use)
    uint8_t* stage = nullptr;
    size_t stage_bytes = 0;
    // pipelined host path: two staging sets, copy streams, per-set events
    uint8_t* pipe_stage[2] = {nullptr, nullptr};
    size_t pipe_bytes = 0;
    cudaStream_t pipe_in = nullptr, pipe_out = nullptr;
    cudaEvent_t pipe_in_done[2] = {nullptr, nullptr}, pipe_compute_done[2] = {nullptr, nullptr},
                pipe_out_done[2] = {nullptr, nullptr};
    int64_t pipe_seq = 0;
    std::string error;
};

namespace {

int fail(moe_fp8_b200_handle h, int code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (h) h->error = buf; else g_create_error = buf;
    return code;
}

void resolve_reference_policy(int T, DispatchPolicy& p)
{
    std::memset(&p, 0, sizeof(p));
    p.keep_limit = 3;
    if (T <= 1) return;  // fused exact dispatch
    const bool prune = T >= 32 || T == 15;
    if (!prune) { p.skip_zero_weight = 1; return; }
    p.prune = 1;
    float frac = 0.30f;
    if (T >= 10000 && T < 13000) frac = 0.34f;
    const bool low_t = T == 32 || T == 57 || T == 58 || T == 62 || T == 80 || T == 901;
    if (low_t) frac = 0.20f;
    if (T == 14107) frac = 0.30f;
    else if (T == 32) frac = 0.25f;
    else if (T == 53) frac = 0.20f;
    else if (T == 80) frac = 0.20f;
    else if (T == 901) frac = 0.24f;
    p.drop_third_frac = frac;
    p.drop_third = (T >= 10000 || T == 54 || T == 56 || T == 59 || T == 53 || low_t) ? 1 : 0;
    if (T == 14107) { p.drop_second_frac_2 = 0.302f; p.drop_second_frac_ge3 = 0.303f; }
    else if (T == 901) { p.drop_second_frac_2 = p.drop_second_frac_ge3 = 0.245f; }
    else if (T == 80) { p.drop_second_frac_2 = p.drop_second_frac_ge3 = 0.20f; }
    else if (T == 53) { p.drop_second_frac_2 = p.drop_second_frac_ge3 = 0.30f; }
    p.renorm = (T == 14107) ? 0 : 1;
}

int enqueue_layer(moe_fp8_b200_handle h, const moe_fp8_b200_args& a, cudaStream_t stream,
                  const ExchangeView* ex = nullptr, bool finalize = true)
{
    const int T = a.num_tokens;
    const int E = h->num_local_experts;
    DispatchPolicy pol;
    if (h->opt_reference_pruning) {
        resolve_reference_policy(T, pol);
    } else {
        std::memset(&pol, 0, sizeof(pol));
        pol.keep_limit = 3;
    }
    const int placement = h->expert_map_set ? -1 : h->opt_expert_stride;   // -1 table, 1 contiguous, S strided
    pol.expert_stride = placement;
    pol.expert_phase = placement < 0 ? 0 : (int)a.local_expert_offset;
    if (!h->reference_routing()) { pol.top_k = h->top_k; pol.n_group = h->n_group; pol.topk_group = h->topk_group; }
    const bool ref_geo = h->geo.is_reference();
    const uint64_t hidden = (uint64_t)h->geo.hidden, inter = (uint64_t)h->geo.inter;
    if (ex && !ref_geo)
        return fail(h, MOE_FP8_B200_ERR_UNSUPPORTED, "the fused combine + reduce-scatter exists for hidden 7168 only (handle has %d)",
                    h->geo.hidden);
    if (a.gemm1_weights != h->cached_w1) {
        const int r = encode_kmajor_u8_map(h->tmap_w1, a.gemm1_weights, hidden, 2 * inter, E, 128);
        if (r != 0) return fail(h, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(W1) failed: %d", r);
        if (ref_geo) {
            const int r2 = encode_rows_1k_map(h->tmap_dec_w1, a.gemm1_weights, kHidden, (uint64_t)E * kGemm1Out, 8);
            if (r2 != 0) return fail(h, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(W1, decode view) failed: %d", r2);
        }
        h->cached_w1 = a.gemm1_weights;
    }
    if (a.gemm2_weights != h->cached_w2) {
        const int r = encode_kmajor_u8_map(h->tmap_w2, a.gemm2_weights, inter, hidden, E, 256);
        if (r != 0) return fail(h, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(W2) failed: %d", r);
        if (ref_geo) {
            const int r2 = encode_rows_1k_map(h->tmap_dec_w2, a.gemm2_weights, kInter, (uint64_t)E * kHidden, 16);
            if (r2 != 0) return fail(h, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(W2, decode view) failed: %d", r2);
        }
        h->cached_w2 = a.gemm2_weights;
    }
    cudaEvent_t* ev = nullptr;
    if (h->opt_stage_timing) {
        if (!h->events_created) {
            for (auto& run : h->events)
                for (auto& x : run)
                    if (cudaEventCreate(&x) != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "cudaEventCreate failed");
            h->events_created = true;
        }
        ev = h->events[h->timed_runs % moe_fp8_b200_ctx::kTimedRuns];
        ++h->timed_runs;
    }
    auto mark = [&](int i) { if (ev) cudaEventRecord(ev[i], stream); };
    // The routing kernel's last CTA leaves the counters at zero for the next call; only after
    // a failed launch (chain cut short) are they cleared explicitly.
    cudaError_t e = cudaSuccess;
    if (h->counters_dirty) {
        e = cudaMemsetAsync(h->ws.ctrl, 0, sizeof(Control), stream);
        h->counters_dirty = false;
    }
    if (h->opt_decode && h->decode_ctas_per_sm > 0 && T <= kDecodeMaxTokens && finalize && !ex && placement == 1 &&
        h->opt_stop_after == 0 && ref_geo && h->reference_routing()) {
        // the whole layer as one cooperative kernel, one CTA per SM
        DecodeArgs d;
        d.logits = a.routing_logits;
        d.bias = static_cast<const __nv_bfloat16*>(a.routing_bias);
        d.hidden = static_cast<const uint8_t*>(a.hidden_states);
        d.hscale = a.hidden_states_scale;
        d.w1 = static_cast<const uint8_t*>(a.gemm1_weights);
        d.s1 = a.gemm1_weights_scale;
        d.w2 = static_cast<const uint8_t*>(a.gemm2_weights);
        d.s2 = a.gemm2_weights_scale;
        d.out = static_cast<__nv_bfloat16*>(a.output);
        d.T = T;
        d.local_expert_offset = (int)a.local_expert_offset;
        d.num_local_experts = E;
        d.rsf = (float)a.routed_scaling_factor;
        d.silu_exact = h->opt_exact_silu;
        d.pol = pol;
        mark(0);
        if (e == cudaSuccess) e = launch_decode_layer(d, h->tmap_dec_w1, h->tmap_dec_w2, h->ws, h->num_sms, stream);
        if (e == cudaErrorCooperativeLaunchTooLarge) {
            // fewer SMs than the device reports are available to this context (partitioned GPU):
            // the grid cannot be co-resident, so this handle uses the chain from now on
            cudaGetLastError();
            h->decode_ctas_per_sm = 0;
            e = cudaSuccess;
        } else {
            for (int i = 1; i <= 6; ++i) mark(i);
            if (e != cudaSuccess) {
                h->counters_dirty = true;
                return fail(h, MOE_FP8_B200_ERR_CUDA, "decode launch failed: %s", cudaGetErrorString(e));
            }
            return MOE_FP8_B200_OK;
        }
    }
    if (e == cudaSuccess && (a.gemm1_weights_scale != h->cached_s1 || a.gemm2_weights_scale != h->cached_s2)) {
        // new scale tensors: lay them out for the GEMMs' promotion (stream-ordered in front of the chain)
        e = launch_repack_weight_scales(a.gemm1_weights_scale, a.gemm2_weights_scale, h->sw1_packed, h->sw2_packed, E, h->geo,
                                        stream);
        if (e == cudaSuccess) { h->cached_s1 = a.gemm1_weights_scale; h->cached_s2 = a.gemm2_weights_scale; }
    }
    const bool tiled = h->opt_weight_prelayout != 0;
    if (e == cudaSuccess && tiled && a.gemm1_weights != h->tiled_src1) {
        e = launch_tile_weights(1, a.gemm1_weights, h->w1_tiled, E, h->geo, h->num_sms, stream);
        if (e == cudaSuccess) h->tiled_src1 = a.gemm1_weights;
    }
    if (e == cudaSuccess && tiled && a.gemm2_weights != h->tiled_src2) {
        e = launch_tile_weights(2, a.gemm2_weights, h->w2_tiled, E, h->geo, h->num_sms, stream);
        if (e == cudaSuccess) h->tiled_src2 = a.gemm2_weights;
    }
    Workspace gemm_ws = h->ws;
    gemm_ws.w_tiled = tiled ? 1 : 0;
    mark(0);
    if (e == cudaSuccess)
        e = launch_route_dispatch(a.routing_logits, a.routing_bias, h->ws, T, (int)a.local_expert_offset, E,
                                  (float)a.routed_scaling_factor, pol, /*do_scan=*/1, stream);
    mark(1);
    mark(2);
    const int stop = h->opt_stop_after > 0 ? h->opt_stop_after : 99;
    // decode-sized batches may leave most SMs without a tile: there the split-K instantiation
    // (chosen here from T alone, it decides on the device whether to split) spreads the K range
    const int split_k = (T <= 4 && ref_geo) ? 1 : 0;   // 4 = kSplitKMaxRows of the GEMM kernel
    // at most 64 tokens (an expert then has at most 64 rows): 64-row activation boxes and a fourth operand stage
    const int small_a = (h->opt_small_batch_ring && T > 4 && T <= 64 && ref_geo) ? 1 : 0;
    // one persistent CTA per SM; CTAs without work leave at once, spare ones take split-K units
    auto ctas = [&](int) { return h->num_sms; };
    if (e == cudaSuccess && stop >= 2) e = launch_permute(a.hidden_states, a.hidden_states_scale, h->ws, T, stream);
    mark(3);
    if (e == cudaSuccess && stop >= 3)
        e = launch_grouped_gemm(1, small_a ? h->tmap_a1_small : h->tmap_a1, tiled ? h->tmap_w1_tiled : h->tmap_w1, h->tmap_y,
                                gemm_ws, h->sw1_packed, h->opt_exact_silu, ctas(1), split_k, small_a, stream);
    mark(4);
    if (e == cudaSuccess && stop >= 4)
        e = launch_grouped_gemm(2, small_a ? h->tmap_a2_small : h->tmap_a2, tiled ? h->tmap_w2_tiled : h->tmap_w2, h->tmap_y,
                                gemm_ws, h->sw2_packed, 0, ctas(2), split_k, small_a, stream);
    mark(5);
    if (e == cudaSuccess && stop >= 5 && finalize) {
        if (ex) {
            e = launch_combine_push(h->ws, *ex, T, stream);
            if (e == cudaSuccess) e = launch_reduce_owned(h->ws, *ex, T, a.output, stream);
        } else {
            e = launch_combine(h->ws, a.output, T, stream);
        }
    }
    mark(6);
    if (e != cudaSuccess) {
        h->counters_dirty = true;
        return fail(h, MOE_FP8_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    }
    return MOE_FP8_B200_OK;
}

int validate(moe_fp8_b200_handle h, const moe_fp8_b200_args* a, bool need_output = true)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (!a) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "args is NULL");
    if (a->num_tokens < 0) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "num_tokens %d < 0", a->num_tokens);
    if (a->num_tokens > h->max_tokens)
        return fail(h, MOE_FP8_B200_ERR_CAPACITY, "num_tokens %d exceeds the handle's max_tokens %d", a->num_tokens,
                    h->max_tokens);
    if (a->num_tokens == 0) return MOE_FP8_B200_OK;
    if (!a->routing_logits || !a->routing_bias || !a->hidden_states || !a->hidden_states_scale ||
        !a->gemm1_weights || !a->gemm1_weights_scale || !a->gemm2_weights || !a->gemm2_weights_scale ||
        (need_output && !a->output))
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "a tensor pointer is NULL");
    // Contiguous placement: the handle's experts are whole 32-expert shards of the reference
    // (kernel/moe_fp8.cu:462-463 filters [offset, offset + 32)), so the offset is a multiple of 32 and the
    // block ends inside the 256 experts.  Strided placement: the offset is the phase.  Table: ignored.
    if (h->expert_map_set) {
        // table placement: the offset plays no part
    } else if (h->opt_expert_stride > 1) {
        if (a->local_expert_offset < 0 || a->local_expert_offset >= h->opt_expert_stride)
            return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT,
                        "with expert stride %d local_expert_offset is the phase and must be in [0, %d)",
                        h->opt_expert_stride, h->opt_expert_stride);
    } else if (a->local_expert_offset < 0 || a->local_expert_offset % kShardExperts != 0 ||
               a->local_expert_offset + h->num_local_experts > kNumExperts) {
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT,
                    "local_expert_offset %lld must be a multiple of 32 with offset + %d local experts <= 256",
                    (long long)a->local_expert_offset, h->num_local_experts);
    }
    if (((uintptr_t)a->hidden_states & 15u) || ((uintptr_t)a->gemm1_weights & 15u) ||
        ((uintptr_t)a->gemm2_weights & 15u) || ((uintptr_t)a->output & 15u))
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "hidden_states, weights and output must be 16-byte aligned");
    return MOE_FP8_B200_OK;
}

}  // namespace

extern "C" {

int moe_fp8_b200_version(void) { return kVersion; }

int moe_fp8_b200_row_capacity(int max_tokens, int num_local_experts)
{
    if (max_tokens <= 0 || num_local_experts <= 0 || num_local_experts > kMaxLocalExperts) return 0;
    return row_capacity(max_tokens, num_local_experts);
}

size_t moe_fp8_b200_workspace_bytes(int max_tokens, int num_local_experts)
{
    if (max_tokens <= 0 || num_local_experts <= 0 || num_local_experts > kMaxLocalExperts) return 0;
    return make_layout(max_tokens, num_local_experts).total;
}

int moe_fp8_b200_reference_policy(int num_tokens, int32_t out_flags[5], float out_fracs[3])
{
    if (!out_flags || !out_fracs) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    DispatchPolicy p;
    resolve_reference_policy(num_tokens, p);
    out_flags[0] = p.prune; out_flags[1] = p.skip_zero_weight; out_flags[2] = p.keep_limit;
    out_flags[3] = p.drop_third; out_flags[4] = p.renorm;
    out_fracs[0] = p.drop_third_frac; out_fracs[1] = p.drop_second_frac_2; out_fracs[2] = p.drop_second_frac_ge3;
    return MOE_FP8_B200_OK;
}

namespace {
// NULL = the reference's shape.  Returns NULL when the shape is usable, else what is wrong with it.
const char* check_shape(const moe_fp8_b200_shape* sh, moe_fp8_b200_shape& out)
{
    out = {kHidden, kInter, kTopK, kNumGroups, kTopKGroup};
    if (!sh) return nullptr;
    out = *sh;
    if (out.hidden < 256 || out.hidden > 8192 || out.hidden % 256 != 0) return "hidden must be a multiple of 256 in [256, 8192]";
    if (out.intermediate < 128 || out.intermediate > 8192 || out.intermediate % 128 != 0)
        return "intermediate must be a multiple of 128 in [128, 8192]";
    if (out.top_k < 1 || out.top_k > kTopK) return "top_k must be in [1, 8]";
    if (out.n_group != 1 && out.n_group != 2 && out.n_group != 4 && out.n_group != 8) return "n_group must be 1, 2, 4 or 8";
    if (out.topk_group < 1 || out.topk_group > out.n_group) return "topk_group must be in [1, n_group]";
    if (out.topk_group * (kNumExperts / out.n_group) < out.top_k) return "the kept groups hold fewer than top_k experts";
    return nullptr;
}
}  // namespace

size_t moe_fp8_b200_workspace_bytes_shaped(int max_tokens, int num_local_experts, const moe_fp8_b200_shape* shape)
{
    moe_fp8_b200_shape sh;
    if (max_tokens <= 0 || num_local_experts <= 0 || num_local_experts > kMaxLocalExperts || check_shape(shape, sh)) return 0;
    return make_layout(max_tokens, num_local_experts, Geometry{sh.hidden, sh.intermediate}).total;
}

int moe_fp8_b200_get_shape(moe_fp8_b200_handle h, moe_fp8_b200_shape* out)
{
    if (!h || !out) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    *out = {h->geo.hidden, h->geo.inter, h->top_k, h->n_group, h->topk_group};
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_create(moe_fp8_b200_handle* out, int device, int max_tokens, int num_local_experts)
{
    return moe_fp8_b200_create_shaped(out, device, max_tokens, num_local_experts, nullptr);
}

int moe_fp8_b200_create_shaped(moe_fp8_b200_handle* out, int device, int max_tokens, int num_local_experts,
                               const moe_fp8_b200_shape* shape)
{
    if (!out) return fail(nullptr, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "out is NULL");
    *out = nullptr;
    if (max_tokens <= 0) return fail(nullptr, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "max_tokens must be positive");
    if (num_local_experts != 32 && num_local_experts != 64 && num_local_experts != 128 && num_local_experts != 256)
        return fail(nullptr, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "num_local_experts must be 32, 64, 128 or 256");
    moe_fp8_b200_shape sh;
    if (const char* why = check_shape(shape, sh)) return fail(nullptr, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "shape: %s", why);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess)
        return fail(nullptr, MOE_FP8_B200_ERR_CUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(nullptr, MOE_FP8_B200_ERR_CUDA, "device properties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
        return fail(nullptr, MOE_FP8_B200_ERR_UNSUPPORTED,
                    "device %d is sm_%d%d; this library holds sm_100a code only (no fallback path)", device,
                    prop.major, prop.minor);
    moe_fp8_b200_ctx* h = new (std::nothrow) moe_fp8_b200_ctx();
    if (!h) return fail(nullptr, MOE_FP8_B200_ERR_CUDA, "out of host memory");
    h->device = device;
    h->max_tokens = max_tokens;
    h->num_local_experts = num_local_experts;
    h->num_sms = prop.multiProcessorCount;
    h->decode_ctas_per_sm = decode_max_ctas_per_sm();
    h->geo = Geometry{sh.hidden, sh.intermediate};
    h->top_k = sh.top_k;
    h->n_group = sh.n_group;
    h->topk_group = sh.topk_group;
    h->layout = make_layout(max_tokens, num_local_experts, h->geo);
    e = cudaMalloc(&h->base, h->layout.total);
    if (e != cudaSuccess) {
        const int rc = fail(nullptr, MOE_FP8_B200_ERR_CUDA, "cudaMalloc(%zu): %s", h->layout.total, cudaGetErrorString(e));
        delete h;
        return rc;
    }
    const Layout& L = h->layout;
    Workspace& w = h->ws;
    w.ctrl = reinterpret_cast<Control*>(h->base + L.ctrl);
    w.expert_offset = reinterpret_cast<int*>(h->base + L.expert_offset);
    w.tile_info = reinterpret_cast<int4*>(h->base + L.tile_info);
    w.num_tiles = reinterpret_cast<int*>(h->base + L.num_tiles);
    w.topk_idx = reinterpret_cast<int*>(h->base + L.topk_idx);
    w.topk_weight = reinterpret_cast<float*>(h->base + L.topk_weight);
    w.pair_count = reinterpret_cast<int*>(h->base + L.pair_count);
    w.pair_code = reinterpret_cast<uint32_t*>(h->base + L.pair_code);
    w.pair_weight = reinterpret_cast<float*>(h->base + L.pair_weight);
    w.pair_row = reinterpret_cast<int*>(h->base + L.pair_row);
    w.row_token = reinterpret_cast<int*>(h->base + L.row_token);
    w.a1 = h->base + L.a1;
    w.sfa1 = reinterpret_cast<float*>(h->base + L.sfa1);
    w.a2 = h->base + L.a2;
    w.sfa2 = reinterpret_cast<float*>(h->base + L.sfa2);
    w.y = reinterpret_cast<__nv_bfloat16*>(h->base + L.y);
    w.splitk_partial = reinterpret_cast<float*>(h->base + L.splitk);
    w.expert_map = reinterpret_cast<int*>(h->base + L.expert_map);
    h->sw1_packed = reinterpret_cast<float*>(h->base + L.sw1_packed);
    h->sw2_packed = reinterpret_cast<float*>(h->base + L.sw2_packed);
    w.m_cap = L.m_cap;
    w.max_tiles = L.max_tiles;
    w.geo = h->geo;
    // Small control arrays start defined; the large row buffers are written before use.
    e = cudaMemset(h->base, 0, L.topk_idx);
    if (e == cudaSuccess) e = cudaMemset(w.row_token, 0xff, sizeof(int) * (size_t)L.m_cap);
    if (e == cudaSuccess) e = configure_gemm_kernels();
    int mr = 0;
    if (e == cudaSuccess) {
        if (tensor_map_bytes() > sizeof(h->tmap_a1)) mr = -100;
        if (mr == 0) mr = encode_kmajor_u8_map(h->tmap_a1, w.a1, h->geo.hidden, L.m_cap, 0, kTileM);
        if (mr == 0) mr = encode_kmajor_u8_map(h->tmap_a2, w.a2, h->geo.inter, L.m_cap, 0, kTileM);
        if (mr == 0) mr = encode_kmajor_u8_map(h->tmap_a1_small, w.a1, h->geo.hidden, L.m_cap, 0, kTileM / 2);
        if (mr == 0) mr = encode_kmajor_u8_map(h->tmap_a2_small, w.a2, h->geo.inter, L.m_cap, 0, kTileM / 2);
        if (mr == 0) mr = encode_out_bf16_map(h->tmap_y, w.y, h->geo.hidden, L.m_cap);
    }
    if (e != cudaSuccess || mr != 0) {
        const int rc = (e != cudaSuccess)
                           ? fail(nullptr, MOE_FP8_B200_ERR_CUDA, "workspace set-up: %s", cudaGetErrorString(e))
                           : fail(nullptr, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(workspace) failed: %d", mr);
        cudaFree(h->base);
        delete h;
        return rc;
    }
    *out = h;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_destroy(moe_fp8_b200_handle h)
{
    if (!h) return MOE_FP8_B200_OK;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    if (h->events_created)
        for (auto& run : h->events)
            for (auto& x : run) cudaEventDestroy(x);
    if (h->stage) cudaFree(h->stage);
    for (int i = 0; i < 2; ++i) {
        if (h->pipe_stage[i]) cudaFree(h->pipe_stage[i]);
        if (h->pipe_in_done[i]) cudaEventDestroy(h->pipe_in_done[i]);
        if (h->pipe_compute_done[i]) cudaEventDestroy(h->pipe_compute_done[i]);
        if (h->pipe_out_done[i]) cudaEventDestroy(h->pipe_out_done[i]);
    }
    if (h->pipe_in) cudaStreamDestroy(h->pipe_in);
    if (h->pipe_out) cudaStreamDestroy(h->pipe_out);
    if (h->w1_tiled) cudaFree(h->w1_tiled);
    if (h->w2_tiled) cudaFree(h->w2_tiled);
    if (h->base) cudaFree(h->base);
    delete h;
    return MOE_FP8_B200_OK;
}

const char* moe_fp8_b200_last_error(moe_fp8_b200_handle h) { return h ? h->error.c_str() : g_create_error.c_str(); }

int moe_fp8_b200_set_option(moe_fp8_b200_handle h, int option, int value)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    switch (option) {
        case MOE_FP8_B200_OPT_REFERENCE_PRUNING: h->opt_reference_pruning = value ? 1 : 0; return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_EXACT_SILU: h->opt_exact_silu = value ? 1 : 0; return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_STOP_AFTER_STAGE: h->opt_stop_after = value; return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_DECODE_KERNEL: h->opt_decode = value ? 1 : 0; return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_EXPERT_STRIDE:
            if (value != 1 && !((value == 2 || value == 4 || value == 8) && h->num_local_experts * value == kNumExperts))
                return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT,
                            "expert stride %d needs 2, 4 or 8 and num_local_experts * stride == 256 (handle has %d)", value,
                            h->num_local_experts);
            h->opt_expert_stride = value;
            return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_WAIT_LIMIT_US:
            if (value < 1) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "wait limit must be at least 1 us");
            h->opt_wait_limit_us = value;
            return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_SMALL_BATCH_RING: h->opt_small_batch_ring = value ? 1 : 0; return MOE_FP8_B200_OK;
        case MOE_FP8_B200_OPT_WEIGHT_PRELAYOUT: {
            const int on = value ? 1 : 0;
            if (on == h->opt_weight_prelayout) return MOE_FP8_B200_OK;
            int prev_device = 0;
            cudaGetDevice(&prev_device);
            cudaSetDevice(h->device);
            struct Restore { int d; ~Restore() { cudaSetDevice(d); } } restore{prev_device};
            if (!on) {
                // kernels of earlier runs may still read the copies
                cudaDeviceSynchronize();
                cudaFree(h->w1_tiled);
                cudaFree(h->w2_tiled);
                h->w1_tiled = h->w2_tiled = nullptr;
                h->tiled_src1 = h->tiled_src2 = nullptr;
                h->opt_weight_prelayout = 0;
                return MOE_FP8_B200_OK;
            }
            const size_t E = (size_t)h->num_local_experts;
            const size_t bytes1 = E * 2 * h->geo.inter * h->geo.hidden, bytes2 = E * h->geo.hidden * h->geo.inter;
            cudaError_t ce = cudaMalloc(&h->w1_tiled, bytes1);
            if (ce == cudaSuccess) ce = cudaMalloc(&h->w2_tiled, bytes2);
            int mr = 0;
            if (ce == cudaSuccess) mr = encode_kmajor_u8_map(h->tmap_w1_tiled, h->w1_tiled, 128, bytes1 / 128, 0, 256);
            if (ce == cudaSuccess && mr == 0) mr = encode_kmajor_u8_map(h->tmap_w2_tiled, h->w2_tiled, 128, bytes2 / 128, 0, 256);
            if (ce != cudaSuccess || mr != 0) {
                cudaGetLastError();
                cudaFree(h->w1_tiled);
                cudaFree(h->w2_tiled);
                h->w1_tiled = h->w2_tiled = nullptr;
                if (ce != cudaSuccess)
                    return fail(h, MOE_FP8_B200_ERR_CUDA, "no room for the tile-ordered weight copies (%zu bytes): %s", bytes1 + bytes2,
                                cudaGetErrorString(ce));
                return fail(h, MOE_FP8_B200_ERR_CUDA, "cuTensorMapEncodeTiled(tile-ordered weights) failed: %d", mr);
            }
            h->tiled_src1 = h->tiled_src2 = nullptr;
            h->opt_weight_prelayout = 1;
            return MOE_FP8_B200_OK;
        }
        case MOE_FP8_B200_OPT_STAGE_TIMING:
            h->opt_stage_timing = value ? 1 : 0;
            h->timed_runs = 0;
            return MOE_FP8_B200_OK;
        default: return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "unknown option %d", option);
    }
}

int moe_fp8_b200_run(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream)
{
    const int v = validate(h, args);
    if (v != MOE_FP8_B200_OK) return v;
    if (args->num_tokens == 0) return MOE_FP8_B200_OK;
    return enqueue_layer(h, *args, static_cast<cudaStream_t>(stream));
}

namespace {
constexpr size_t kExchangeFlagBytes = 256;
// Layout of a receive buffer for up to `capacity` tokens per call; depends on (capacity, world) only.
void exchange_layout(int capacity, int world, ExchangeView& v)
{
    v.world = world;
    v.slot_rows = (capacity + world - 1) / world;
    v.present_stride = (v.slot_rows + 15) / 16 * 16;
    v.data_offset = kExchangeFlagBytes;
    v.rows_bytes_per_parity = (size_t)world * v.slot_rows * kHidden * sizeof(__nv_bfloat16);
    v.present_bytes_per_parity = align_up((size_t)world * v.present_stride, 256);
}
}  // namespace

size_t moe_fp8_b200_exchange_bytes(int num_tokens, int world)
{
    if (num_tokens < 0 || (world != 1 && world != 2 && world != 4 && world != 8)) return 0;
    ExchangeView v;
    exchange_layout(num_tokens, world, v);
    return v.data_offset + 2 * v.rows_bytes_per_parity + 2 * v.present_bytes_per_parity;
}

int moe_fp8_b200_exchange_regions(int capacity_tokens, int world, size_t out_offsets[4], size_t out_sizes[2])
{
    if (capacity_tokens < 0 || (world != 1 && world != 2 && world != 4 && world != 8) || !out_offsets || !out_sizes)
        return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    ExchangeView v;
    exchange_layout(capacity_tokens, world, v);
    out_offsets[0] = v.data_offset;
    out_offsets[1] = v.data_offset + v.rows_bytes_per_parity;
    out_offsets[2] = v.data_offset + 2 * v.rows_bytes_per_parity;
    out_offsets[3] = out_offsets[2] + v.present_bytes_per_parity;
    out_sizes[0] = v.rows_bytes_per_parity;
    out_sizes[1] = v.present_bytes_per_parity;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_run_reduce_scatter(moe_fp8_b200_handle h, const moe_fp8_b200_args* args,
                                    const moe_fp8_b200_exchange* x, void* stream)
{
    const int v = validate(h, args);
    if (v != MOE_FP8_B200_OK) return v;
    if (!x) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "exchange is NULL");
    if (x->world != 1 && x->world != 2 && x->world != 4 && x->world != 8)
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "world %d is not 1, 2, 4 or 8", x->world);
    if (x->rank < 0 || x->rank >= x->world)
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "rank %d outside [0, %d)", x->rank, x->world);
    if (x->epoch == 0) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "epoch must start at 1");
    if (args->num_tokens == 0) return MOE_FP8_B200_OK;
    const int capacity = x->capacity_tokens > 0 ? x->capacity_tokens : h->max_tokens;
    if (args->num_tokens > capacity)
        return fail(h, MOE_FP8_B200_ERR_CAPACITY, "num_tokens %d exceeds the exchange buffers' capacity of %d tokens",
                    args->num_tokens, capacity);
    ExchangeView view;
    exchange_layout(capacity, x->world, view);
    view.tokens_per_rank = (args->num_tokens + x->world - 1) / x->world;
    view.wait_limit_us = (uint32_t)h->opt_wait_limit_us;
    const size_t need = moe_fp8_b200_exchange_bytes(capacity, x->world);
    if (x->buffer_bytes < need)
        return fail(h, MOE_FP8_B200_ERR_CAPACITY, "exchange buffers hold %zu bytes, a capacity of %d tokens on %d ranks needs %zu",
                    x->buffer_bytes, capacity, x->world, need);
    for (int i = 0; i < kMaxRanks; ++i) {
        view.peer[i] = i < x->world ? static_cast<uint8_t*>(x->peer_buffers[i]) : nullptr;
        if (i < x->world && (!view.peer[i] || ((uintptr_t)view.peer[i] & 255u)))
            return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "peer_buffers[%d] is NULL or not 256-byte aligned", i);
    }
    view.rank = x->rank;
    view.epoch = x->epoch;
    return enqueue_layer(h, *args, static_cast<cudaStream_t>(stream), &view);
}

int moe_fp8_b200_quantize_hidden(moe_fp8_b200_handle h, const void* x, int num_tokens, void* q, float* scale,
                                 void* stream)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (num_tokens < 0) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "num_tokens %d < 0", num_tokens);
    if (num_tokens == 0) return MOE_FP8_B200_OK;
    if (!x || !q || !scale) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "a tensor pointer is NULL");
    if (((uintptr_t)x & 15u) || ((uintptr_t)q & 15u) || ((uintptr_t)scale & 3u))
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "x and q must be 16-byte aligned");
    const cudaError_t e = launch_quantize_rows(x, q, scale, num_tokens, h->geo.hidden, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "quantize launch failed: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_run_unfinalized(moe_fp8_b200_handle h, const moe_fp8_b200_args* args,
                                 moe_fp8_b200_unfinalized* views, void* stream)
{
    const int v = validate(h, args, /*need_output=*/false);
    if (v != MOE_FP8_B200_OK) return v;
    if (!views) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "views is NULL");
    views->y = h->ws.y;
    views->expert_offset = h->ws.expert_offset;
    views->pair_count = h->ws.pair_count;
    views->pair_code = h->ws.pair_code;
    views->pair_weight = h->ws.pair_weight;
    views->row_capacity = h->ws.m_cap;
    if (args->num_tokens == 0) return MOE_FP8_B200_OK;
    return enqueue_layer(h, *args, static_cast<cudaStream_t>(stream), nullptr, /*finalize=*/false);
}

int moe_fp8_b200_finalize(moe_fp8_b200_handle h, int num_tokens, void* output, void* stream)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (num_tokens < 0 || num_tokens > h->max_tokens)
        return fail(h, MOE_FP8_B200_ERR_CAPACITY, "num_tokens %d outside [0, %d]", num_tokens, h->max_tokens);
    if (num_tokens == 0) return MOE_FP8_B200_OK;
    if (!output || ((uintptr_t)output & 15u))
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "output is NULL or not 16-byte aligned");
    const cudaError_t e = launch_combine(h->ws, output, num_tokens, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "combine launch failed: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_invalidate_weights(moe_fp8_b200_handle h)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    h->cached_w1 = h->cached_w2 = nullptr;
    h->cached_s1 = h->cached_s2 = nullptr;
    h->tiled_src1 = h->tiled_src2 = nullptr;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_set_expert_map(moe_fp8_b200_handle h, const int32_t* local_slot)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (!local_slot) {   // back to what MOE_FP8_B200_OPT_EXPERT_STRIDE says (contiguous unless set otherwise)
        h->expert_map_set = false;
        return MOE_FP8_B200_OK;
    }
    int seen[kMaxLocalExperts] = {0};
    for (int g = 0; g < kNumExperts; ++g) {
        const int s = local_slot[g];
        if (s < -1 || s >= h->num_local_experts || (s >= 0 && seen[s]++))
            return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "expert map: slot %d of global expert %d is out of range or used twice", s, g);
    }
    for (int s = 0; s < h->num_local_experts; ++s)
        if (!seen[s]) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "expert map: local slot %d has no expert", s);
    cudaError_t e = cudaSetDevice(h->device);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(h->ws.expert_map, local_slot, sizeof(int) * kNumExperts, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "expert map upload: %s", cudaGetErrorString(e));
    h->expert_map_set = true;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_run_host(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream_v)
{
    const int v = validate(h, args);
    if (v != MOE_FP8_B200_OK) return v;
    const int T = args->num_tokens;
    if (T == 0) return MOE_FP8_B200_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // staging sized once, on the first call, for the handle's max_tokens: no later call allocates or frees
    const size_t Tm = (size_t)h->max_tokens;
    const size_t b_logits = align_up(sizeof(float) * Tm * kNumExperts, 256);
    const size_t hidden = (size_t)h->geo.hidden, hidden_blocks = hidden / kBlock;
    const size_t b_hidden = align_up(Tm * hidden, 256);
    const size_t b_scale = align_up(sizeof(float) * hidden_blocks * Tm, 256);
    const size_t b_out = align_up(sizeof(__nv_bfloat16) * Tm * hidden, 256);
    if (!h->stage) {
        const size_t need = b_logits + b_hidden + b_scale + b_out;
        const cudaError_t e = cudaMalloc(&h->stage, need);
        if (e != cudaSuccess) {
            h->stage = nullptr;
            return fail(h, MOE_FP8_B200_ERR_CUDA, "cudaMalloc(staging %zu): %s", need, cudaGetErrorString(e));
        }
        h->stage_bytes = need;
    }
    uint8_t* d_logits = h->stage;
    uint8_t* d_hidden = d_logits + b_logits;
    uint8_t* d_scale = d_hidden + b_hidden;
    uint8_t* d_out = d_scale + b_scale;
    cudaError_t e = cudaMemcpyAsync(d_logits, args->routing_logits, sizeof(float) * (size_t)T * kNumExperts,
                                    cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_hidden, args->hidden_states, (size_t)T * hidden, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_scale, args->hidden_states_scale, sizeof(float) * hidden_blocks * T,
                            cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "host-to-device copy: %s", cudaGetErrorString(e));
    moe_fp8_b200_args dev = *args;
    dev.routing_logits = reinterpret_cast<const float*>(d_logits);
    dev.hidden_states = d_hidden;
    dev.hidden_states_scale = reinterpret_cast<const float*>(d_scale);
    dev.output = d_out;
    const int rc = enqueue_layer(h, dev, stream);
    if (rc != MOE_FP8_B200_OK) return rc;
    e = cudaMemcpyAsync(args->output, d_out, sizeof(__nv_bfloat16) * (size_t)T * hidden, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "device-to-host copy: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_run_host_async(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream_v, int64_t* ticket)
{
    const int v = validate(h, args);
    if (v != MOE_FP8_B200_OK) return v;
    if (!ticket) return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "ticket is NULL");
    const int T = args->num_tokens;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cudaError_t e = cudaSuccess;
    if (!h->pipe_in) {
        e = cudaStreamCreateWithFlags(&h->pipe_in, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->pipe_out, cudaStreamNonBlocking);
        for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
            e = cudaEventCreateWithFlags(&h->pipe_in_done[i], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->pipe_compute_done[i], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->pipe_out_done[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "pipeline set-up: %s", cudaGetErrorString(e));
    }
    const size_t Tm = (size_t)h->max_tokens;
    const size_t b_logits = align_up(sizeof(float) * Tm * kNumExperts, 256);
    const size_t hidden = (size_t)h->geo.hidden, hidden_blocks = hidden / kBlock;
    const size_t b_hidden = align_up(Tm * hidden, 256);
    const size_t b_scale = align_up(sizeof(float) * hidden_blocks * Tm, 256);
    const size_t b_out = align_up(sizeof(__nv_bfloat16) * Tm * hidden, 256);
    if (!h->pipe_stage[0]) {   // sized once for max_tokens: no allocation between pipelined calls
        const size_t need = b_logits + b_hidden + b_scale + b_out;
        for (int i = 0; i < 2 && e == cudaSuccess; ++i) e = cudaMalloc(&h->pipe_stage[i], need);
        if (e != cudaSuccess) {   // all or nothing: a half-made pair would be taken for a whole one next time
            for (int i = 0; i < 2; ++i) {
                if (h->pipe_stage[i]) cudaFree(h->pipe_stage[i]);
                h->pipe_stage[i] = nullptr;
            }
            return fail(h, MOE_FP8_B200_ERR_CUDA, "cudaMalloc(pipeline staging 2 x %zu): %s", need, cudaGetErrorString(e));
        }
        h->pipe_bytes = need;
    }
    // The ticket is handed out (and the sequence advanced) only once the whole call has been enqueued:
    // a call that fails on the way leaves no ticket behind.
    const int64_t seq = h->pipe_seq;
    const int set = (int)(seq & 1);
    if (T == 0) {   // nothing to move; keep the set's events meaningful for host_wait
        e = cudaEventRecord(h->pipe_out_done[set], h->pipe_out);
        if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "event record: %s", cudaGetErrorString(e));
        *ticket = seq;
        h->pipe_seq = seq + 1;
        return MOE_FP8_B200_OK;
    }
    uint8_t* d_logits = h->pipe_stage[set];
    uint8_t* d_hidden = d_logits + b_logits;
    uint8_t* d_scale = d_hidden + b_hidden;
    uint8_t* d_out = d_scale + b_scale;
    // copy-in: the set's inputs were last read by the compute of two calls ago
    if (seq >= 2) e = cudaStreamWaitEvent(h->pipe_in, h->pipe_compute_done[set], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_logits, args->routing_logits, sizeof(float) * (size_t)T * kNumExperts, cudaMemcpyHostToDevice, h->pipe_in);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_hidden, args->hidden_states, (size_t)T * hidden, cudaMemcpyHostToDevice, h->pipe_in);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(d_scale, args->hidden_states_scale, sizeof(float) * hidden_blocks * T, cudaMemcpyHostToDevice, h->pipe_in);
    if (e == cudaSuccess) e = cudaEventRecord(h->pipe_in_done[set], h->pipe_in);
    // compute: needs the inputs, and the set's output buffer must have been copied out (two calls ago)
    if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, h->pipe_in_done[set], 0);
    if (e == cudaSuccess && seq >= 2) e = cudaStreamWaitEvent(stream, h->pipe_out_done[set], 0);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "pipeline copy-in: %s", cudaGetErrorString(e));
    moe_fp8_b200_args dev = *args;
    dev.routing_logits = reinterpret_cast<const float*>(d_logits);
    dev.hidden_states = d_hidden;
    dev.hidden_states_scale = reinterpret_cast<const float*>(d_scale);
    dev.output = d_out;
    const int rc = enqueue_layer(h, dev, stream);
    if (rc != MOE_FP8_B200_OK) return rc;
    e = cudaEventRecord(h->pipe_compute_done[set], stream);
    // copy-out
    if (e == cudaSuccess) e = cudaStreamWaitEvent(h->pipe_out, h->pipe_compute_done[set], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(args->output, d_out, sizeof(__nv_bfloat16) * (size_t)T * hidden, cudaMemcpyDeviceToHost, h->pipe_out);
    if (e == cudaSuccess) e = cudaEventRecord(h->pipe_out_done[set], h->pipe_out);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "pipeline copy-out: %s", cudaGetErrorString(e));
    *ticket = seq;
    h->pipe_seq = seq + 1;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_copy_rows_h2d(void* dst_device, size_t dst_pitch, const void* src_host, size_t src_pitch,
                               size_t row_bytes, size_t rows, void* stream)
{
    if (!dst_device || !src_host || row_bytes > dst_pitch || row_bytes > src_pitch) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (rows == 0 || row_bytes == 0) return MOE_FP8_B200_OK;
    const cudaError_t e = cudaMemcpy2DAsync(dst_device, dst_pitch, src_host, src_pitch, row_bytes, rows,
                                            cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MOE_FP8_B200_OK : MOE_FP8_B200_ERR_CUDA;
}

int moe_fp8_b200_copy_device(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                             size_t rows, void* stream)
{
    if (!dst || !src || row_bytes > dst_pitch || row_bytes > src_pitch) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (rows == 0 || row_bytes == 0) return MOE_FP8_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const cudaError_t e = (rows == 1 || (dst_pitch == row_bytes && src_pitch == row_bytes))
                              ? cudaMemcpyAsync(dst, src, row_bytes * rows, cudaMemcpyDeviceToDevice, s)
                              : cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDeviceToDevice, s);
    return e == cudaSuccess ? MOE_FP8_B200_OK : MOE_FP8_B200_ERR_CUDA;
}

namespace {
int peer_view(moe_fp8_b200_handle h, void* const* peer_bases, int world, int rank, ExchangeView& v)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (!peer_bases || (world != 1 && world != 2 && world != 4 && world != 8) || rank < 0 || rank >= world)
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "peer hand-shake: world %d / rank %d invalid", world, rank);
    std::memset(&v, 0, sizeof v);
    for (int i = 0; i < world; ++i) {
        if (!peer_bases[i] || ((uintptr_t)peer_bases[i] & 3u))
            return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "peer hand-shake: buffer %d is NULL or misaligned", i);
        v.peer[i] = static_cast<uint8_t*>(peer_bases[i]);
    }
    v.world = world;
    v.rank = rank;
    v.wait_limit_us = (uint32_t)h->opt_wait_limit_us;
    return MOE_FP8_B200_OK;
}
}  // namespace

int moe_fp8_b200_signal_peers(moe_fp8_b200_handle h, void* const* peer_bases, int world, int rank, size_t flag_offset,
                              uint32_t value, void* stream)
{
    ExchangeView v;
    const int rc = peer_view(h, peer_bases, world, rank, v);
    if (rc != MOE_FP8_B200_OK) return rc;
    const cudaError_t e = launch_signal_peers(v, flag_offset, value, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MOE_FP8_B200_OK : fail(h, MOE_FP8_B200_ERR_CUDA, "signal launch: %s", cudaGetErrorString(e));
}

int moe_fp8_b200_wait_peers(moe_fp8_b200_handle h, void* const* peer_bases, int world, int rank, size_t flag_offset,
                            uint32_t value, void* stream)
{
    ExchangeView v;
    const int rc = peer_view(h, peer_bases, world, rank, v);
    if (rc != MOE_FP8_B200_OK) return rc;
    const cudaError_t e = launch_wait_peers(v, flag_offset, value, h->ws.ctrl, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? MOE_FP8_B200_OK : fail(h, MOE_FP8_B200_ERR_CUDA, "wait launch: %s", cudaGetErrorString(e));
}

int moe_fp8_b200_host_wait(moe_fp8_b200_handle h, int64_t ticket)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    if (ticket < 0 || ticket >= h->pipe_seq)
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "ticket %lld was never issued", (long long)ticket);
    // The set's event is re-recorded by every later call that uses the set, in the same stream as the
    // ticket's own copy-out: waiting for its latest record therefore also covers an older ticket.
    const cudaError_t e = cudaEventSynchronize(h->pipe_out_done[ticket & 1]);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "waiting for copy-out: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_check(moe_fp8_b200_handle h, void* stream)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "stream synchronize: %s", cudaGetErrorString(e));
    int st[2] = {0, 0};
    e = cudaMemcpy(st, &h->ws.ctrl->status, sizeof(st), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
    if (st[0] != kStatusOk) {
        // The word is sticky on the device (kernels only ever move it from 0 to the first failure); it
        // is cleared here, once reported.  A cut-short run may have left counters behind: the next run
        // clears the whole control block first.
        h->counters_dirty = true;
        cudaMemset(&h->ws.ctrl->status, 0, 2 * sizeof(int));
    }
    if (st[0] != kStatusOk)
        return fail(h, MOE_FP8_B200_ERR_DEVICE, "device status %d (detail %d): %s", st[0], st[1],
                    st[0] == kStatusGemm1Timeout   ? "GEMM1 gave up on a bounded wait"
                    : st[0] == kStatusGemm2Timeout ? "GEMM2 gave up on a bounded wait"
                    : st[0] == kStatusRowOverflow  ? "routed rows exceed the workspace capacity"
                    : st[0] == kStatusExchangeTimeout ? "a peer rank's rows did not arrive within the wait limit"
                    : st[0] == kStatusDecodeTimeout   ? "the decode kernel gave up on a grid barrier"
                                                   : "unknown");
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_inject_device_status(moe_fp8_b200_handle h, int status, unsigned stale_barrier_arrivals, void* stream)
{
    if (!h) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&h->ws.ctrl->status, &status, sizeof(int), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(&h->ws.ctrl->dec_count, &stale_barrier_arrivals, sizeof(unsigned), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "status injection: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_stage_times(moe_fp8_b200_handle h, float out_ms[6], int* out_runs)
{
    if (!h || !out_ms) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < 6; ++i) out_ms[i] = 0.0f;
    const int n = h->timed_runs < moe_fp8_b200_ctx::kTimedRuns ? h->timed_runs : moe_fp8_b200_ctx::kTimedRuns;
    if (out_runs) *out_runs = n;
    if (n == 0) return MOE_FP8_B200_OK;
    for (int r = 0; r < n; ++r) {
        cudaError_t e = cudaEventSynchronize(h->events[r][6]);
        for (int i = 0; i < 6 && e == cudaSuccess; ++i) {
            float ms = 0.0f;
            e = cudaEventElapsedTime(&ms, h->events[r][i], h->events[r][i + 1]);
            out_ms[i] += ms / n;
        }
        if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "stage timing: %s", cudaGetErrorString(e));
    }
    h->timed_runs = 0;
    return MOE_FP8_B200_OK;
}

int moe_fp8_b200_read_intermediate(moe_fp8_b200_handle h, int buffer, void* dst, size_t bytes, size_t offset,
                                   void* stream)
{
    if (!h || !dst) return MOE_FP8_B200_ERR_INVALID_ARGUMENT;
    const Workspace& w = h->ws;
    const size_t T = (size_t)h->max_tokens, M = (size_t)w.m_cap;
    const void* src = nullptr;
    size_t size = 0;
    switch (buffer) {
        case MOE_FP8_B200_BUF_EXPERT_COUNT: src = w.ctrl->expert_rows; size = sizeof(int) * h->num_local_experts; break;
        case MOE_FP8_B200_BUF_EXPERT_OFFSET: src = w.expert_offset; size = sizeof(int) * (h->num_local_experts + 1); break;
        case MOE_FP8_B200_BUF_TOPK_IDX: src = w.topk_idx; size = sizeof(int) * T * kTopK; break;
        case MOE_FP8_B200_BUF_TOPK_WEIGHT: src = w.topk_weight; size = sizeof(float) * T * kTopK; break;
        case MOE_FP8_B200_BUF_PAIR_COUNT: src = w.pair_count; size = sizeof(int) * T; break;
        case MOE_FP8_B200_BUF_PAIR_CODE: src = w.pair_code; size = sizeof(uint32_t) * T * kTopK; break;
        case MOE_FP8_B200_BUF_PAIR_WEIGHT: src = w.pair_weight; size = sizeof(float) * T * kTopK; break;
        case MOE_FP8_B200_BUF_NUM_TILES: src = w.num_tiles; size = sizeof(int); break;
        case MOE_FP8_B200_BUF_ROW_TOKEN: src = w.row_token; size = sizeof(int) * M; break;
        case MOE_FP8_B200_BUF_A1: src = w.a1; size = M * w.geo.hidden; break;
        case MOE_FP8_B200_BUF_SFA1: src = w.sfa1; size = sizeof(float) * (w.geo.hidden / kBlock) * M; break;
        case MOE_FP8_B200_BUF_A2: src = w.a2; size = M * w.geo.inter; break;
        case MOE_FP8_B200_BUF_SFA2: src = w.sfa2; size = sizeof(float) * (w.geo.inter / kBlock) * M; break;
        case MOE_FP8_B200_BUF_Y: src = w.y; size = sizeof(__nv_bfloat16) * M * w.geo.hidden; break;
        case MOE_FP8_B200_BUF_STATUS: src = &w.ctrl->status; size = sizeof(int) * 2; break;
        case MOE_FP8_B200_BUF_DECODE_TIMELINE: src = w.ctrl->dec_time; size = sizeof(w.ctrl->dec_time); break;
        case MOE_FP8_B200_BUF_EXCHANGE_TIMELINE: src = w.ctrl->xch_time; size = sizeof(w.ctrl->xch_time); break;
        case MOE_FP8_B200_BUF_PAIR_ROW: src = w.pair_row; size = sizeof(int) * T * kTopK; break;
        default: return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "unknown buffer id %d", buffer);
    }
    if (offset > size || bytes > size - offset)
        return fail(h, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "buffer %d holds %zu bytes; asked for %zu at offset %zu",
                    buffer, size, bytes, offset);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(dst, static_cast<const uint8_t*>(src) + offset, bytes, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(h, MOE_FP8_B200_ERR_CUDA, "intermediate read: %s", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}

}  // extern "C"
