// `__tvm_ffi_run`: the reference's exported symbol with its 11-argument typed signature
// (kernel/moe_fp8.cu:2663-2669, exported at kernel/moe_fp8.cu:3674), implemented on top of
// the plain C ABI of include/moe_fp8_b200.h.  A loader that drives the reference with
// tvm_ffi.load_module(path).run(...) drives this library the same way.
//
// Differences a caller can observe, all deliberate:
//   * shapes, dtypes and devices are checked and a ValueError / RuntimeError is raised
//     through TVM-FFI (the reference checks nothing, kernel/moe_fp8.cu:2671-2672);
//   * work is enqueued on the TVM-FFI environment stream of the tensors' device (the
//     reference always uses the legacy default stream, kernel/moe_fp8.cu:2691);
//   * nothing is cached by pointer identity, so changed tensor contents are always seen
//     (the reference replays cached routing and graphs, kernel/moe_fp8.cu:2696-2702).
// The workspace is one grow-only handle per host thread, device and expert count, as in
// kernel/moe_fp8.cu:2677-2689.
#include <tvm/ffi/container/tensor.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <tvm/ffi/function.h>

#include <map>
#include <utility>

#include "moe_fp8_b200.h"

namespace ffi = tvm::ffi;

namespace {

struct HandleSlot {
    moe_fp8_b200_handle h = nullptr;
    int capacity = 0;
};

void expect(const ffi::TensorView& t, const char* name, int code, int bits, std::initializer_list<int64_t> shape)
{
    const DLDataType dt = t.dtype();
    // e4m3 payloads may also arrive as raw bytes (uint8 views of the same memory).
    const bool raw_fp8 = code == kDLFloat8_e4m3fn && dt.code == kDLUInt && dt.bits == 8;
    if (!raw_fp8 && (dt.code != code || dt.bits != bits || dt.lanes != 1))
        TVM_FFI_THROW(ValueError) << name << ": unexpected dtype";
    if (t.ndim() != (int32_t)shape.size()) TVM_FFI_THROW(ValueError) << name << ": unexpected rank";
    int i = 0;
    for (int64_t s : shape) {
        if (t.size(i) != s) TVM_FFI_THROW(ValueError) << name << ": dimension " << i << " is " << t.size(i) << ", expected " << s;
        ++i;
    }
    if (t.device().device_type != kDLCUDA) TVM_FFI_THROW(ValueError) << name << ": must be a CUDA tensor";
}

void* ptr(const ffi::TensorView& t) { return static_cast<char*>(t.data_ptr()) + t.byte_offset(); }

void run(ffi::TensorView routing_logits, ffi::TensorView routing_bias, ffi::TensorView hidden_states,
         ffi::TensorView hidden_states_scale, ffi::TensorView gemm1_weights, ffi::TensorView gemm1_weights_scale,
         ffi::TensorView gemm2_weights, ffi::TensorView gemm2_weights_scale, int64_t local_expert_offset,
         double routed_scaling_factor, ffi::TensorView output)
{
    const int64_t T = routing_logits.size(0);
    if (T <= 0) return;
    const int64_t E = gemm1_weights.size(0);
    expect(routing_logits, "routing_logits", kDLFloat, 32, {T, 256});
    expect(routing_bias, "routing_bias", kDLBfloat, 16, {256});
    expect(hidden_states, "hidden_states", kDLFloat8_e4m3fn, 8, {T, 7168});
    expect(hidden_states_scale, "hidden_states_scale", kDLFloat, 32, {56, T});
    expect(gemm1_weights, "gemm1_weights", kDLFloat8_e4m3fn, 8, {E, 4096, 7168});
    expect(gemm1_weights_scale, "gemm1_weights_scale", kDLFloat, 32, {E, 32, 56});
    expect(gemm2_weights, "gemm2_weights", kDLFloat8_e4m3fn, 8, {E, 7168, 2048});
    expect(gemm2_weights_scale, "gemm2_weights_scale", kDLFloat, 32, {E, 56, 16});
    expect(output, "output", kDLBfloat, 16, {T, 7168});

    const int device = routing_logits.device().device_id;
    static thread_local std::map<std::pair<int, int>, HandleSlot> slots;
    HandleSlot& slot = slots[{device, (int)E}];
    if (slot.h == nullptr || slot.capacity < T) {
        if (slot.h) moe_fp8_b200_destroy(slot.h);
        slot.h = nullptr;
        const int cap = T < 16 ? 16 : (int)T;
        if (moe_fp8_b200_create(&slot.h, device, cap, (int)E) != MOE_FP8_B200_OK)
            TVM_FFI_THROW(RuntimeError) << "moe_fp8_b200_create: " << moe_fp8_b200_last_error(nullptr);
        slot.capacity = cap;
    }
    moe_fp8_b200_args a;
    a.routing_logits = static_cast<const float*>(ptr(routing_logits));
    a.routing_bias = ptr(routing_bias);
    a.hidden_states = ptr(hidden_states);
    a.hidden_states_scale = static_cast<const float*>(ptr(hidden_states_scale));
    a.gemm1_weights = ptr(gemm1_weights);
    a.gemm1_weights_scale = static_cast<const float*>(ptr(gemm1_weights_scale));
    a.gemm2_weights = ptr(gemm2_weights);
    a.gemm2_weights_scale = static_cast<const float*>(ptr(gemm2_weights_scale));
    a.local_expert_offset = local_expert_offset;
    a.routed_scaling_factor = routed_scaling_factor;
    a.output = ptr(output);
    a.num_tokens = (int32_t)T;
    void* stream = TVMFFIEnvGetStream(kDLCUDA, device);
    if (moe_fp8_b200_run(slot.h, &a, stream) != MOE_FP8_B200_OK)
        TVM_FFI_THROW(RuntimeError) << "moe_fp8_b200_run: " << moe_fp8_b200_last_error(slot.h);
}

}  // namespace

TVM_FFI_DLL_EXPORT_TYPED_FUNC(run, run);
