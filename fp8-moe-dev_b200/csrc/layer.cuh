// Shared definitions of the FP8 block-scaled MoE layer (DeepSeek-V3 geometry):
// problem constants, the dispatch policy record, and the device-side workspace view
// that every stage kernel receives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace moe {

constexpr int kHidden = 7168;        // H
constexpr int kInter = 2048;         // I
constexpr int kGemm1Out = 4096;      // 2 I  (columns [0,I) linear branch, [I,2I) gated branch)
constexpr int kNumExperts = 256;     // global experts
constexpr int kShardExperts = 32;    // experts of one reference shard == one routing group
constexpr int kBlock = 128;          // quantisation block
constexpr int kHiddenBlocks = kHidden / kBlock;  // 56
constexpr int kInterBlocks = kInter / kBlock;    // 16
constexpr int kTopK = 8;
constexpr int kNumGroups = 8;
constexpr int kTopKGroup = 4;
constexpr int kTileM = 128;          // rows of one expert tile (expert row ranges are padded to it)
constexpr int kMaxLocalExperts = 256;
// Split-K (batches of at most four tokens): a tile's K range is divided over several CTAs when
// there are fewer tiles than SMs; their fp32 partial rows meet in a scratch of kSplitKSlots slots
// (one per work unit).
constexpr int kSplitKSlots = 320;

// What the dispatch step does with a token's experts that fall into one 32-expert
// shard.  The fields restate, as data, the branch structure of the reference's
// routing kernel (kernel/moe_fp8.cu:457-607) after its compile-time knobs
// (kernel/moe_fp8.cu:93-194) and its T-keyed kernel choice (kernel/moe_fp8.cu:2732-2790)
// have been resolved on the host for the call's T.
struct DispatchPolicy {
    int prune;              // 0: every selected local expert is kept (exact dispatch)
    int skip_zero_weight;   // exact dispatch only: drop pairs whose weight is exactly 0
    int keep_limit;         // prune: at most this many experts per token and shard (3)
    int drop_third;         // prune: third expert dropped when w3 <= drop_third_frac * sum
    float drop_third_frac;
    float drop_second_frac_2;    // prune: second dropped when w2 <= frac * sum (0 = never),
    float drop_second_frac_ge3;  //        separate fractions for 2 and for >=3 local experts
    int renorm;             // prune: kept weights rescaled by sum(local) / sum(kept)
    // Which global experts are local.  stride <= 1: the contiguous block [local_expert_offset,
    // local_expert_offset + E) as in the reference.  stride S > 1 (multi-GPU wrapper only): every
    // S-th expert, global id g is local iff g % S == phase, with local index g / S; stride -1: the
    // table Workspace::expert_map (global id -> local index, -1 = not local).  In both of these the
    // policy above is still evaluated per 32-expert shard of GLOBAL ids, so the ranks' pairs together
    // are exactly those of the reference's shard calls.
    int expert_stride;
    int expert_phase;
    // Routing constants (the reference compiles 8 / 8 / 4 in, kernel/moe_fp8.cu:301-304; FlashInfer's
    // definition of the layer carries them as axes).  0 in all three = the reference's values.
    int top_k;        // experts selected per token, <= 8
    int n_group;      // routing groups: 1, 2, 4 or 8 (256 / n_group experts each)
    int topk_group;   // groups kept per token, <= n_group
};

// Run-time geometry of a handle.  The reference's layer is hidden 7168 / intermediate 2048; other
// multiples of the 128 block (hidden a multiple of 256, both at most 8192) run through the generic
// instantiations of the kernels, the reference's own geometry through the compile-time ones.
struct Geometry {
    int hidden, inter;
    __host__ __device__ bool is_reference() const { return hidden == kHidden && inter == kInter; }
};

// Integer control block.  Zeroed when the handle is created; after that the last CTA of the
// routing kernel turns the counters into offsets and tiles and puts them back to zero for
// the next call, so a call needs no memset node.
struct Control {
    int expert_count[kMaxLocalExperts];  // routed rows per local expert (atomic counters)
    int status;                          // 0 ok; otherwise the first error a kernel recorded
    int status_detail;
    int blocks_done;                     // routing CTAs finished (ticket for the last-CTA scan)
    int pad;
    int expert_rows[kMaxLocalExperts];   // copy of the counters of the last call (diagnostics)
    int splitk_ticket[kSplitKSlots];     // per-tile arrival counters of the split-K reduction (self-clearing)
    int push_done;                       // combine-and-push CTAs finished (ticket, self-clearing)
    unsigned dec_count;                  // arrival counters of the decode kernel's two grid barriers
    unsigned dec_phase;                  // (cleared by CTA 0 of each launch, see decode.cu)
    int pad2;
    unsigned long long dec_time[16];     // phase timestamps (ns) of CTA 0 in the last decode-kernel run
    // Timestamps (ns, %globaltimer) of the last fused combine + reduce-scatter on this rank:
    // [0] first CTA of the push starts, [1] last CTA of the push done (flags published), [2] first CTA of the
    // owner step starts waiting, [3] last CTA has seen all peers' flags, [4] last CTA of the owner step done.
    // [0] and [2] are minima (reset to all-ones by the routing kernel's scan), the others maxima (reset to 0).
    unsigned long long xch_time[8];
};

enum KernelStatus : int {
    kStatusOk = 0,
    kStatusGemm1Timeout = 101,
    kStatusGemm2Timeout = 102,
    kStatusRowOverflow = 103,
    kStatusExchangeTimeout = 104,
    kStatusDecodeTimeout = 105,
};

// Cross-GPU exchange of the fused combine + reduce-scatter (expert-parallel ranks of one NVSwitch
// box).  Every rank owns one receive buffer of identical layout in peer-mapped memory:
//   [world sources] u32 (first 256 bytes)                    epoch of the last complete push
//   [2 parities][world sources][slot_rows][7168] bf16   partial rows, written by the source
//   [2 parities][world sources][present_stride]  u8     1 if the source sent that row
// slot_rows = ceil(capacity / world) comes from the buffer's token capacity, not from the call's T: a
// call with fewer tokens uses the first ceil(T / world) rows of every slot, and the regions of the two
// parities stay disjoint whatever sequence of T the ranks run.
// Rank r owns tokens [r * tokens_per_rank, (r + 1) * tokens_per_rank).  Data are double-buffered
// by epoch parity; a source may push epoch e + 2 only after it has reduced epoch e + 1, which
// implies that every owner has finished reading epoch e (its push of e + 1 follows its own
// reduce of e in stream order), so no further back-signal is needed.
constexpr int kMaxRanks = 8;
struct ExchangeView {
    uint8_t* peer[kMaxRanks];   // receive buffer of every rank, mapped into this process
    int rank, world;
    int tokens_per_rank;        // ceil(T / world): who owns which token of THIS call
    int slot_rows;              // rows of one source's slot = ceil(capacity / world): fixed per buffer, so that
                                // the two parity regions never move when T changes from call to call
    int present_stride;         // slot_rows rounded up to 16
    uint32_t epoch;
    uint32_t wait_limit_us;     // bound of the owner's wait for its peers' flags
    size_t data_offset;         // rows start here (the flags occupy the bytes before)
    size_t rows_bytes_per_parity, present_bytes_per_parity;
};

// Device pointers into the workspace (all owned by the handle).
struct Workspace {
    Control* ctrl;
    int* expert_offset;     // [E+1] first packed row of each expert (multiples of 128)
    int4* tile_info;        // [max_tiles] per 128-row tile: {local expert, first tile of that expert,
                            //             tiles of that expert, routed rows of that expert}
    int* num_tiles;         // [1]
    int* expert_map;        // [256] global expert -> local index or -1 (table placement only)
    int* topk_idx;          // [T,8] global expert ids in selection order
    float* topk_weight;     // [T,8] normalised weights (before routed_scaling_factor)
    int* pair_count;        // [T]   kept (token, local expert) pairs
    uint32_t* pair_code;    // [T,8] (local expert << 24) | slot inside the expert
    float* pair_weight;     // [T,8] weight * (renorm) * routed_scaling_factor
    int* pair_row;          // [T,8] packed row of each kept pair, -1 past the token's pair count (written by the
                            //       permute kernel; lets the fused exchange find a token's rows in one load)
    int* row_token;         // [M_cap] token of each packed row (diagnostics / tests)
    uint8_t* a1;            // [M_cap, H]   e4m3 rows gathered per expert
    float* sfa1;            // [56, M_cap]  their 1x128 scales, k-block major
    uint8_t* a2;            // [M_cap, I]   e4m3 SwiGLU output
    float* sfa2;            // [16, M_cap]
    __nv_bfloat16* y;       // [M_cap, H]   GEMM2 rows before the weighted combine
    float* splitk_partial;  // [kSplitKSlots, 4, 256] fp32 partial rows of split-K work units
    int m_cap;              // packed-row capacity (multiple of 128)
    int max_tiles;
    Geometry geo;
    int w_tiled;            // the GEMMs' weight map covers the tile-ordered copy (one 32 KB piece per tile and K block)
};

}  // namespace moe
