// Interface of the single-kernel decode path (decode.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "layer.cuh"

namespace moe {

constexpr int kDecodeMaxTokens = 8;   // every expert then has at most 8 rows: one n = 8 MMA tile

struct DecodeArgs {
    const float* logits;            // [T, 256]
    const __nv_bfloat16* bias;      // [256]
    const uint8_t* hidden;          // [T, 7168] e4m3
    const float* hscale;            // [56, T]
    const uint8_t* w1;              // [E, 4096, 7168] e4m3
    const float* s1;                // [E, 32, 56]
    const uint8_t* w2;              // [E, 7168, 2048] e4m3
    const float* s2;                // [E, 56, 16]
    __nv_bfloat16* out;             // [T, 7168]
    int T, local_expert_offset, num_local_experts;
    float rsf;
    int silu_exact;
    DispatchPolicy pol;
};

// Prepares the decode kernel on the current device (shared-memory opt-in) and returns how many
// of its CTAs fit on one SM (0: it cannot run here).  Call once per device before launching.
int decode_max_ctas_per_sm();
// tmap_w1 / tmap_w2: tensor maps of the weights as rows of 32-bit words with 1 KB x 8 / 1 KB x 16 boxes.
cudaError_t launch_decode_layer(const DecodeArgs& args, const void* tmap_w1, const void* tmap_w2, const Workspace& ws,
                                int num_ctas, cudaStream_t stream);

}  // namespace moe
