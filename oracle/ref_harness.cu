// TEST INFRASTRUCTURE ONLY (never part of the product path).
//
// Compiles the UNMODIFIED reference translation unit kernel/moe_fp8.cu by textual
// inclusion (the file stays where it lies in the reference checkout; build_ref.sh passes
// its directory with -I) and appends C entry points that launch the reference's own
// routing / dispatch / offset kernels on caller-provided buffers.  The reference keeps
// those intermediates in a static workspace that no caller can reach; this is the only
// way to compare them bit for bit.  The reference's `run` and its `__tvm_ffi_run` export
// are part of the same object, unchanged.
#include "moe_fp8.cu"

#define HARNESS_API extern "C" __attribute__((visibility("default")))

// Routing only: route_topk_kernel<false,false> (kernel/moe_fp8.cu:329-456) for any T.
HARNESS_API int ref_harness_route(const float* logits, const void* bias, int T, int32_t* topk_idx,
                                  float* topk_weight, int32_t* token_local_count, void* stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const size_t shmem = (2 * kNumExperts + kNumGroups + kNumGroups + kTopK + kTopK) * sizeof(float);
    route_topk_kernel<false, false><<<T, kNumExperts, shmem, stream>>>(
        logits, static_cast<const __nv_bfloat16*>(bias), topk_idx, topk_weight, token_local_count, nullptr, nullptr,
        nullptr, nullptr, nullptr, T, 0, 1.0f);
    return (int)cudaGetLastError();
}

// Routing + dispatch + offsets with the kernel choice run() makes for this T
// (kernel/moe_fp8.cu:2729-2811).  Buffers: topk_idx/topk_weight [T,8], token_local_count [T],
// expert_token_count [32], expert_token_list/weight [32,T], token_pair_code/weight [T,8],
// expert_offsets_m [33], expert_token_padded [32].  Returns which variant ran:
// 0 = fused exact (T <= 1), 1 = fused pruning, 2 = unfused exact; negative = CUDA error.
HARNESS_API int ref_harness_dispatch(const float* logits, const void* bias_v, int T, int local_expert_offset,
                                     float rsf, int32_t* topk_idx, float* topk_weight, int32_t* token_local_count,
                                     int32_t* expert_token_count, int32_t* expert_token_list,
                                     float* expert_token_weight, int32_t* token_pair_code, float* token_pair_weight,
                                     int32_t* expert_offsets_m, int32_t* expert_token_padded,
                                     int32_t* scratch_sfa_offsets /* [2*33 + 1] */, void* stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(bias_v);
    const size_t shmem = (2 * kNumExperts + kNumGroups + kNumGroups + kTopK + kTopK) * sizeof(float);
    int variant;
    if (T <= MOE_FUSED_ROUTE_DISPATCH_MAX_T) {
        variant = 0;
        route_topk_kernel<true, false><<<T, kNumExperts, shmem, stream>>>(
            logits, bias, topk_idx, topk_weight, token_local_count, expert_token_count, expert_token_list,
            expert_token_weight, token_pair_code, token_pair_weight, T, local_expert_offset, rsf);
    } else if (T >= MOE_KEEP_ONE_LOCAL_MIN_T || T == MOE_KEEP_ONE_LOCAL_EXTRA_T || T == MOE_KEEP_ONE_LOCAL_EXTRA_T2) {
        variant = 1;
        route_topk_kernel<true, true><<<T, kNumExperts, shmem, stream>>>(
            logits, bias, topk_idx, topk_weight, token_local_count, expert_token_count, expert_token_list,
            expert_token_weight, token_pair_code, token_pair_weight, T, local_expert_offset, rsf);
    } else {
        variant = 2;
        route_topk_kernel<false, false><<<T, kNumExperts, shmem, stream>>>(
            logits, bias, topk_idx, topk_weight, token_local_count, expert_token_count, expert_token_list,
            expert_token_weight, token_pair_code, token_pair_weight, T, local_expert_offset, rsf);
        build_dispatch_kernel<<<kNumLocal, 256, 0, stream>>>(
            topk_idx, topk_weight, expert_token_count, expert_token_list, expert_token_weight, token_local_count,
            token_pair_code, token_pair_weight, T, local_expert_offset, rsf);
    }
    const int sfa_pad_m = (T <= 2048) ? 64 : 128;
    scan_offsets_kernel<<<1, 32, 0, stream>>>(expert_token_count, nullptr, nullptr, kBM_g1, kBM_g2, 0, 0, sfa_pad_m,
                                              nullptr, expert_offsets_m, expert_token_padded, scratch_sfa_offsets,
                                              scratch_sfa_offsets + 33, scratch_sfa_offsets + 66);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? variant : -(int)e;
}
