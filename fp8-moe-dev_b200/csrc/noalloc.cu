// Routing + dispatch for callers that are not allowed to allocate device memory.
//
// Some hosts embed this library where a cudaMalloc is off the table: inside a region that
// is being captured into a CUDA graph, in a real-time serving loop whose memory pool is
// frozen after start-up, or behind a runtime that hands out every byte itself and forbids
// library-side allocations.  For them the routing stage is offered once more with its
// scratch memory (per-expert row counters and the per-token pair tables) living in a
// fixed device array that is part of the library image, so the call neither allocates
// nor frees anything: no cudaMalloc / cudaFree, no handle, no torch, no allocating
// library routine.
//
// The array costs kScratchBytes on every GPU that loads the library, until the process
// exits.  All calls on a device share it and it keeps the previous call's contents, so
// the counters are cleared at the start of every call; two calls that overlap on the
// same GPU (different streams or threads) race on it and must be serialised by the caller.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/moe_fp8_b200.h"
#include "layer.cuh"

namespace moe {
cudaError_t launch_route_dispatch(const float*, const void*, const Workspace&, int, int, int, float,
                                  const DispatchPolicy&, int, cudaStream_t);
}
using namespace moe;

namespace {

constexpr int kMaxTokens = MOE_FP8_B200_NOALLOC_MAX_TOKENS;
constexpr size_t kCtrlBytes = (sizeof(Control) + 255) / 256 * 256;
constexpr size_t kPairCountBytes = sizeof(int) * (size_t)kMaxTokens;
constexpr size_t kPairCodeBytes = sizeof(uint32_t) * (size_t)kMaxTokens * kTopK;
constexpr size_t kPairWeightBytes = sizeof(float) * (size_t)kMaxTokens * kTopK;
constexpr size_t kScratchBytes = kCtrlBytes + kPairCountBytes + kPairCodeBytes + kPairWeightBytes;

// The scratch itself.  In host code this name is only a stand-in for the symbol, not a
// device address; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_route_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {};

int report(char* err, size_t err_len, int code, const char* msg, const char* detail = "")
{
    if (err && err_len) std::snprintf(err, err_len, "%s%s", msg, detail);
    return code;
}

// Device address of the scratch array on the current device (looked up once per device).
cudaError_t scratch_for_current_device(unsigned char** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] != nullptr) {
        // A cudaDeviceReset since the look-up would have unloaded the module the address came from:
        // keep the remembered address only while the runtime still knows it as memory of this device.
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, g_scratch_ptr[dev]) != cudaSuccess || at.type != cudaMemoryTypeDevice ||
            at.device != dev) {
            cudaGetLastError();
            g_scratch_ptr[dev] = nullptr;
        }
    }
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_route_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

// True when `p` is device memory of device `dev` (or memory every device can reach: managed).
bool on_device(const void* p, int dev)
{
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
    if (at.type == cudaMemoryTypeManaged) return true;
    return at.type == cudaMemoryTypeDevice && at.device == dev;
}

}  // namespace

extern "C" int moe_fp8_b200_route_noalloc(const float* routing_logits, const void* routing_bias, int32_t num_tokens,
                                          int64_t local_expert_offset, int32_t num_local_experts,
                                          double routed_scaling_factor, int32_t reference_pruning,
                                          int32_t* topk_idx_out, float* topk_weight_out, int32_t* expert_count_out,
                                          void* stream_v, char* err, size_t err_len)
{
    if (num_tokens < 0) return report(err, err_len, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "num_tokens is negative");
    if (num_tokens > kMaxTokens) {
        char d[96];
        std::snprintf(d, sizeof d, " (%d > %d)", num_tokens, kMaxTokens);
        return report(err, err_len, MOE_FP8_B200_ERR_CAPACITY,
                      "num_tokens exceeds MOE_FP8_B200_NOALLOC_MAX_TOKENS, the size of the built-in scratch", d);
    }
    if (num_local_experts != 32 && num_local_experts != 64 && num_local_experts != 128 && num_local_experts != 256)
        return report(err, err_len, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "num_local_experts must be 32, 64, 128 or 256");
    // whole 32-expert shards of the reference inside the 256 experts, as in moe_fp8_b200_run
    if (local_expert_offset < 0 || local_expert_offset % kShardExperts != 0 ||
        local_expert_offset + num_local_experts > kNumExperts)
        return report(err, err_len, MOE_FP8_B200_ERR_INVALID_ARGUMENT,
                      "local_expert_offset must be a multiple of 32 with offset + num_local_experts <= 256");
    if (num_tokens == 0) return MOE_FP8_B200_OK;
    if (!routing_logits || !routing_bias || !topk_idx_out || !topk_weight_out || !expert_count_out)
        return report(err, err_len, MOE_FP8_B200_ERR_INVALID_ARGUMENT, "a pointer argument is NULL");

    // The scratch and the launch belong to the CURRENT device: tensors of another GPU are refused
    // rather than read through whatever peer mapping may exist.
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess)
        return report(err, err_len, MOE_FP8_B200_ERR_CUDA, "cudaGetDevice failed");
    if (!on_device(routing_logits, cur) || !on_device(routing_bias, cur) || !on_device(topk_idx_out, cur) ||
        !on_device(topk_weight_out, cur) || !on_device(expert_count_out, cur))
        return report(err, err_len, MOE_FP8_B200_ERR_INVALID_ARGUMENT,
                      "a tensor does not live on the current CUDA device (make the tensors' GPU current before the call)");
    unsigned char* scratch = nullptr;
    cudaError_t e = scratch_for_current_device(&scratch);
    if (e != cudaSuccess)
        return report(err, err_len, MOE_FP8_B200_ERR_CUDA, "cudaGetSymbolAddress(scratch): ", cudaGetErrorString(e));

    Workspace ws;
    std::memset(&ws, 0, sizeof ws);
    ws.geo = Geometry{kHidden, kInter};
    ws.ctrl = reinterpret_cast<Control*>(scratch);
    ws.pair_count = reinterpret_cast<int*>(scratch + kCtrlBytes);
    ws.pair_code = reinterpret_cast<uint32_t*>(scratch + kCtrlBytes + kPairCountBytes);
    ws.pair_weight = reinterpret_cast<float*>(scratch + kCtrlBytes + kPairCountBytes + kPairCodeBytes);
    ws.topk_idx = topk_idx_out;
    ws.topk_weight = topk_weight_out;

    int32_t flags[5];
    float fracs[3];
    DispatchPolicy pol;
    std::memset(&pol, 0, sizeof pol);
    pol.keep_limit = 3;
    if (reference_pruning) {
        moe_fp8_b200_reference_policy(num_tokens, flags, fracs);
        pol.prune = flags[0]; pol.skip_zero_weight = flags[1]; pol.keep_limit = flags[2];
        pol.drop_third = flags[3]; pol.renorm = flags[4];
        pol.drop_third_frac = fracs[0]; pol.drop_second_frac_2 = fracs[1]; pol.drop_second_frac_ge3 = fracs[2];
    }

    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // The array still holds the previous call's counters: they must start at zero.
    e = cudaMemsetAsync(ws.ctrl, 0, sizeof(Control), stream);
    if (e == cudaSuccess)
        e = launch_route_dispatch(routing_logits, routing_bias, ws, num_tokens, (int)local_expert_offset,
                                  num_local_experts, (float)routed_scaling_factor, pol, /*do_scan=*/0, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(expert_count_out, ws.ctrl->expert_count, sizeof(int) * (size_t)num_local_experts,
                            cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return report(err, err_len, MOE_FP8_B200_ERR_CUDA, "launch failed: ", cudaGetErrorString(e));
    return MOE_FP8_B200_OK;
}
