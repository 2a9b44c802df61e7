/*
 * moe_fp8_b200 -- C ABI of the B200 (sm_100a) FP8 block-scaled MoE layer.
 *
 * One call computes one DeepSeek-V3 MoE layer shard: no-aux routing over 256 global
 * experts, dispatch to the `num_local_experts` experts this GPU holds, FP8 grouped GEMM1
 * (7168 -> 2 x 2048) with fused SwiGLU + 1x128 e4m3 requantisation, FP8 grouped GEMM2
 * (2048 -> 7168) and the weighted combine into a bf16 output.
 *
 * The argument set, dtypes, layouts and semantics of `moe_fp8_b200_run` are those of the
 * reference operator `run(...)` in kernel/moe_fp8.cu:2663-2669 (exported as
 * `__tvm_ffi_run` at kernel/moe_fp8.cu:3674); only the carrier changes from TVM-FFI
 * tensor views to plain device pointers.  All functions return 0 on success and a
 * negative `moe_fp8_b200_status` otherwise; `moe_fp8_b200_last_error` gives the text.
 *
 * Pointers are DEVICE pointers of the handle's device unless a function says otherwise.
 * A handle is not thread-safe; use one per host thread and GPU (the reference keeps one
 * thread-local workspace, kernel/moe_fp8.cu:2677-2689).
 */
#ifndef MOE_FP8_B200_H_
#define MOE_FP8_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MOE_FP8_B200_API __attribute__((visibility("default")))
#else
#define MOE_FP8_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct moe_fp8_b200_ctx* moe_fp8_b200_handle;

typedef enum {
    MOE_FP8_B200_OK = 0,
    MOE_FP8_B200_ERR_INVALID_ARGUMENT = -1,
    MOE_FP8_B200_ERR_CUDA = -2,
    MOE_FP8_B200_ERR_CAPACITY = -3, /* num_tokens above the handle's max_tokens */
    MOE_FP8_B200_ERR_DEVICE = -4,   /* a kernel reported a bounded wait that ran out */
    MOE_FP8_B200_ERR_UNSUPPORTED = -5
} moe_fp8_b200_status;

/* Replaces the positional arguments of run(), kernel/moe_fp8.cu:2663-2669. */
typedef struct {
    const float* routing_logits;        /* fp32 [T, 256] */
    const void* routing_bias;           /* bf16 [256] */
    const void* hidden_states;          /* e4m3 [T, 7168] */
    const float* hidden_states_scale;   /* fp32 [56, T]  (k-block major, tokens contiguous) */
    const void* gemm1_weights;          /* e4m3 [E_local, 4096, 7168] */
    const float* gemm1_weights_scale;   /* fp32 [E_local, 32, 56] */
    const void* gemm2_weights;          /* e4m3 [E_local, 7168, 2048] */
    const float* gemm2_weights_scale;   /* fp32 [E_local, 56, 16] */
    int64_t local_expert_offset;        /* first global expert held here (32 * rank): a multiple of 32 with
                                         * offset + E_local <= 256, anything else is refused */
    double routed_scaling_factor;
    void* output;                       /* bf16 [T, 7168], fully overwritten */
    int32_t num_tokens;                 /* T; 0 is a no-op (kernel/moe_fp8.cu:2671-2672) */
} moe_fp8_b200_args;

/* Options (moe_fp8_b200_set_option). */
enum {
    /* 1 (default): dispatch follows the reference's T-keyed policy table, i.e. exact
     * dispatch for T < 32 (T != 15) and the keep-3 / drop-third / renormalise pruning
     * of kernel/moe_fp8.cu:476-607 otherwise, applied per 32-expert shard.
     * 0: exact dispatch at every T (the FlashInfer definition's semantics). */
    MOE_FP8_B200_OPT_REFERENCE_PRUNING = 1,
    /* 0 (default): the reference's rsqrt sigmoid approximant in SwiGLU
     * (kernel/moe_fp8.cu:313-315, 1803-1804).  1: x / (1 + exp(-x)). */
    MOE_FP8_B200_OPT_EXACT_SILU = 2,
    /* 1: record CUDA events around every stage of each run (not capturable into a graph
     * while on); read them with moe_fp8_b200_stage_times.  Setting it restarts the count. */
    MOE_FP8_B200_OPT_STAGE_TIMING = 3,
    /* Diagnostics: N > 0 enqueues only the first N stages of a run (1 routing+dispatch+scan,
     * 2 +permute, 3 +GEMM1, 4 +GEMM2, 5 = all); the output is then not (fully) written.
     * 0 (default) runs the whole layer. */
    MOE_FP8_B200_OPT_STOP_AFTER_STAGE = 4,
    /* 1 (default): batches of at most MOE_FP8_B200_DECODE_MAX_TOKENS tokens run as one
     * cooperative kernel (routing, both GEMMs on warp-level MMAs straight from global memory,
     * combine; two bounded grid barriers) instead of the five-kernel chain.  Same results up
     * to fp32 summation order inside GEMM1.  That kernel fills only the routing and pair
     * tables of the workspace (EXPERT_COUNT, TOPK_*, PAIR_*); 0 selects the chain, which also
     * leaves the packed rows, tiles and offsets behind for moe_fp8_b200_read_intermediate.
     * Unfinalised, stage-limited and multi-GPU-exchange runs always use the chain. */
    MOE_FP8_B200_OPT_DECODE_KERNEL = 5,
    /* Expert placement for the multi-GPU wrapper (no counterpart in the reference, whose shards are
     * contiguous blocks of 32 experts).  S = 1 (default): the handle's experts are the global ids
     * [local_expert_offset, local_expert_offset + E).  S in {2, 4, 8} with E * S == 256: the handle's
     * experts are every S-th global expert, g with g % S == local_expert_offset (which must then be
     * < S), stacked in increasing g; the dispatch policy is still evaluated per 32-expert shard of
     * global ids, so the S handles together produce exactly the pairs of the reference's shard calls
     * while every handle carries an equal share of every routing group. */
    MOE_FP8_B200_OPT_EXPERT_STRIDE = 6,
    /* Bound, in microseconds, of the wait of moe_fp8_b200_run_reduce_scatter's owner step for its peers'
     * rows (default 1 000 000).  When it runs out the kernel completes with zero rows, the device status
     * word records it and moe_fp8_b200_check returns MOE_FP8_B200_ERR_DEVICE; the GPU never hangs on a
     * peer that does not arrive.  The waits inside the GEMM and decode kernels keep their fixed 1 s. */
    MOE_FP8_B200_OPT_WAIT_LIMIT_US = 7,
    /* 1: the chain's GEMMs read the weights from tile-ordered copies kept by the handle (the operand of one
     * (expert, n tile, K block) is one contiguous 32 KB piece instead of 256 pieces of 128 bytes a weight row
     * apart), which is what a batch that is bound by streaming the weights wants.  Switching it on allocates
     * num_local_experts x 44 MB (reference geometry) on the handle's device, outside the workspace; the copies are
     * filled by one kernel in front of the first run that sees a weight pointer and remembered by address, like
     * the scale layout (moe_fp8_b200_invalidate_weights drops them).  Results are bit-identical either way.
     * Replaces the reference's per-pointer W1 pre-layout cache (kernel/moe_fp8.cu:981-994, 3007-3014).
     * Default 0.  The decode kernel (batches of at most 8 tokens) always reads the caller's weights. */
    MOE_FP8_B200_OPT_WEIGHT_PRELAYOUT = 8,
    /* Batches of 5 to 64 tokens (reference geometry): the GEMMs load 64-row activation boxes (an expert cannot
     * have more rows) and use the room for a fourth operand stage, i.e. more weight bytes in flight per SM
     * (default 1).  0 = the three-stage kernel of the larger batches.  Bit-identical results. */
    MOE_FP8_B200_OPT_SMALL_BATCH_RING = 9
};
#define MOE_FP8_B200_DECODE_MAX_TOKENS 8

/* Intermediate buffers readable after a run (moe_fp8_b200_read_intermediate). */
enum {
    MOE_FP8_B200_BUF_EXPERT_COUNT = 0,  /* int32 [E_local]  routed rows per local expert */
    MOE_FP8_B200_BUF_EXPERT_OFFSET = 1, /* int32 [E_local+1] first packed row per expert */
    MOE_FP8_B200_BUF_TOPK_IDX = 2,      /* int32 [T, 8] */
    MOE_FP8_B200_BUF_TOPK_WEIGHT = 3,   /* fp32  [T, 8] */
    MOE_FP8_B200_BUF_PAIR_COUNT = 4,    /* int32 [T] */
    MOE_FP8_B200_BUF_PAIR_CODE = 5,     /* uint32 [T, 8]  (local expert << 24) | slot */
    MOE_FP8_B200_BUF_PAIR_WEIGHT = 6,   /* fp32  [T, 8] */
    MOE_FP8_B200_BUF_NUM_TILES = 7,     /* int32 [1] */
    MOE_FP8_B200_BUF_ROW_TOKEN = 8,     /* int32 [M_cap] */
    MOE_FP8_B200_BUF_A1 = 9,            /* e4m3 [M_cap, 7168] */
    MOE_FP8_B200_BUF_SFA1 = 10,         /* fp32 [56, M_cap] */
    MOE_FP8_B200_BUF_A2 = 11,           /* e4m3 [M_cap, 2048] */
    MOE_FP8_B200_BUF_SFA2 = 12,         /* fp32 [16, M_cap] */
    MOE_FP8_B200_BUF_Y = 13,            /* bf16 [M_cap, 7168] */
    MOE_FP8_B200_BUF_STATUS = 14,       /* int32 [2] device status word + detail */
    MOE_FP8_B200_BUF_DECODE_TIMELINE = 15, /* uint64 [16] ns clock of CTA 0 in the last decode-kernel run: [0..6] start, tables
                                           * built, phase 1 done, barrier 1 passed, phase 2 done, barrier 2 passed, end;
                                           * [8..11] inside the table build: token routed, pairs listed, tables merged, published */
    MOE_FP8_B200_BUF_EXCHANGE_TIMELINE = 16, /* uint64 [8] ns clock of the last moe_fp8_b200_run_reduce_scatter on this rank:
                                            * [0] push starts, [1] push done and flags published, [2] owner step starts
                                            * waiting for its peers, [3] all peers' flags seen, [4] owner step done */
    MOE_FP8_B200_BUF_PAIR_ROW = 17       /* int32 [T, 8] packed row of each kept pair (expert offset + slot), -1 past the
                                          * token's pair count; written by the permute stage of the chain */
};

/* Library version, (major << 16) | minor.  No counterpart in the reference. */
MOE_FP8_B200_API int moe_fp8_b200_version(void);

/* Bytes of device workspace a handle of this capacity allocates.  Replaces the
 * reference's grow-only alloc_workspace sizing, kernel/moe_fp8.cu:2473-2585. */
MOE_FP8_B200_API size_t moe_fp8_b200_workspace_bytes(int max_tokens, int num_local_experts);

/* Packed-row capacity M_cap for that sizing (multiple of 128). */
MOE_FP8_B200_API int moe_fp8_b200_row_capacity(int max_tokens, int num_local_experts);

/* Allocates the workspace on `device` (every cudaMalloc of the library happens here,
 * except the staging buffers of run_host and run_host_async, which the first call of each allocates
 * once, sized for max_tokens).  num_local_experts in {32, 64, 128, 256}.  Replaces the thread-local
 * Workspace of kernel/moe_fp8.cu:2349-2461, 2677-2689. */
MOE_FP8_B200_API int moe_fp8_b200_create(moe_fp8_b200_handle* out, int device, int max_tokens, int num_local_experts);

/* Other shapes of the same layer.  The reference compiles hidden 7168 / intermediate 2048 and the routing
 * constants 8 / 8 / 4 in (kernel/moe_fp8.cu:292-304); FlashInfer's definition of the operator carries them
 * as axes.  A handle made here runs the five-kernel chain with those values at run time:
 *   hidden        multiple of 256, 256 .. 8192     tensors [T, hidden], scales [hidden/128, T]
 *   intermediate  multiple of 128, 128 .. 8192     W1 [E, 2*intermediate, hidden], W2 [E, hidden, intermediate]
 *   top_k         1 .. 8                            experts per token; table rows keep 8 entries, the unused ones
 *                                                   hold expert -1 and weight 0
 *   n_group       1, 2, 4 or 8                      routing groups of 256 / n_group experts
 *   topk_group    1 .. n_group, with topk_group * (256 / n_group) >= top_k
 * The number of global experts stays 256.  shape == NULL, or the reference's values, gives exactly the
 * handle of moe_fp8_b200_create.  With another hidden or intermediate size the single-kernel decode path,
 * the split-K GEMMs, moe_fp8_b200_run_reduce_scatter and moe_fp8_b200_route_noalloc are not available
 * (MOE_FP8_B200_ERR_UNSUPPORTED where they are asked for explicitly, the chain otherwise). */
typedef struct moe_fp8_b200_shape {
    int32_t hidden, intermediate;
    int32_t top_k, n_group, topk_group;
} moe_fp8_b200_shape;
MOE_FP8_B200_API int moe_fp8_b200_create_shaped(moe_fp8_b200_handle* out, int device, int max_tokens, int num_local_experts,
                                                const moe_fp8_b200_shape* shape);
/* Workspace bytes of such a handle (0 for a shape that create_shaped refuses). */
MOE_FP8_B200_API size_t moe_fp8_b200_workspace_bytes_shaped(int max_tokens, int num_local_experts,
                                                            const moe_fp8_b200_shape* shape);
/* The shape a handle was made with. */
MOE_FP8_B200_API int moe_fp8_b200_get_shape(moe_fp8_b200_handle h, moe_fp8_b200_shape* out);

MOE_FP8_B200_API int moe_fp8_b200_destroy(moe_fp8_b200_handle h);

/* Text of the last error on this handle (or of the last failed create when h is NULL).
 * The reference only prints to stderr (kernel/moe_fp8.cu:2683, 3130, 3162). */
MOE_FP8_B200_API const char* moe_fp8_b200_last_error(moe_fp8_b200_handle h);

MOE_FP8_B200_API int moe_fp8_b200_set_option(moe_fp8_b200_handle h, int option, int value);

/* The layer.  Enqueues every stage on `stream` (a cudaStream_t; NULL = legacy default
 * stream, which is what the reference always uses, kernel/moe_fp8.cu:2691) and returns
 * without synchronising, like the reference (kernel/moe_fp8.cu:45-47).  No host read of
 * device data happens, so the call may be captured into a CUDA graph; routing is
 * recomputed on every call (the reference caches it by pointer identity,
 * kernel/moe_fp8.cu:2696-2702).  Replaces run(), kernel/moe_fp8.cu:2663-3672. */
MOE_FP8_B200_API int moe_fp8_b200_run(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream);

/* Same layer with HOST pointers for the per-call tensors (routing_logits,
 * hidden_states, hidden_states_scale, output); routing_bias and the weights stay device
 * pointers.  Copies in, runs, copies out and synchronises `stream`.  This is the
 * end-to-end form a host-resident caller of the reference operator sees. */
MOE_FP8_B200_API int moe_fp8_b200_run_host(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream);

/* Pipelined form of moe_fp8_b200_run_host for a caller that feeds batch after batch from host
 * memory: the call enqueues copy-in, the layer and copy-out on three streams and returns a
 * ticket without waiting; two staging sets alternate, so the copy-in of call i+1 and the
 * copy-out of call i-1 run while call i computes (PCIe is full duplex and needs no SM).  The
 * host tensors of a call (inputs and output) must stay untouched until
 * moe_fp8_b200_host_wait(handle, ticket) has returned for it, and at most two calls may be
 * outstanding (wait for ticket i-1 before issuing call i+1).  Host memory should be pinned;
 * pageable memory works but serialises.  `stream` carries the compute, as in run().  No
 * counterpart in the reference, which takes device tensors only. */
MOE_FP8_B200_API int moe_fp8_b200_run_host_async(moe_fp8_b200_handle h, const moe_fp8_b200_args* args, void* stream,
                                                 int64_t* ticket);
MOE_FP8_B200_API int moe_fp8_b200_host_wait(moe_fp8_b200_handle h, int64_t ticket);

/* Strided host-to-device copy of `rows` pieces of `row_bytes` bytes (one cudaMemcpy2DAsync on `stream`):
 * what a rank of the multi-GPU wrapper uses to fetch ITS token columns [lo, lo + n) of the host-resident
 * hidden_states_scale [56, T] -- a strided view that a plain copy would first have to pack on the host.
 * The source should be pinned.  No counterpart in the reference (device tensors only). */
MOE_FP8_B200_API int moe_fp8_b200_copy_rows_h2d(void* dst_device, size_t dst_pitch, const void* src_host,
                                                size_t src_pitch, size_t row_bytes, size_t rows, void* stream);

/* Plumbing of the multi-GPU wrapper's host-resident form, in which the ranks fill each other's input staging
 * with copy engines instead of an SM-based all-gather (no counterpart in the reference):
 *   copy_device    `rows` pieces of `row_bytes` bytes device-to-device on `stream` (one cudaMemcpyAsync or
 *                  cudaMemcpy2DAsync: copy engines, no SM; dst may be a peer's mapped memory);
 *   signal_peers   after the copies: this rank's 32-bit word (index `rank`) of the flag array at `flag_offset`
 *                  inside EVERY rank's buffer takes `value` (release at system scope).  A tiny kernel: where
 *                  no SM may be free (behind persistent kernels) the wrapper stores the word with a 4-byte
 *                  copy from pinned host memory instead (moe_fp8_b200_copy_rows_h2d), which needs none;
 *   wait_peers     before the consumer: spins, bounded by MOE_FP8_B200_OPT_WAIT_LIMIT_US, until all `world`
 *                  words of the LOCAL flag array have reached `value` (wrap-safe); on expiry the device
 *                  status word records it and moe_fp8_b200_check returns MOE_FP8_B200_ERR_DEVICE.
 * peer_bases[i] is rank i's buffer as mapped into this process (peer_bases[rank] the local one). */
MOE_FP8_B200_API int moe_fp8_b200_copy_device(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                              size_t row_bytes, size_t rows, void* stream);
MOE_FP8_B200_API int moe_fp8_b200_signal_peers(moe_fp8_b200_handle h, void* const* peer_bases, int world, int rank,
                                               size_t flag_offset, uint32_t value, void* stream);
MOE_FP8_B200_API int moe_fp8_b200_wait_peers(moe_fp8_b200_handle h, void* const* peer_bases, int world, int rank,
                                             size_t flag_offset, uint32_t value, void* stream);

/* ---- expert-parallel run with the reduce-scatter fused into the combine step -----------
 * No counterpart in the reference (it has no multi-GPU code; its local_expert_offset
 * argument, kernel/moe_fp8.cu:2671, only says which 32 experts a rank holds).  `world` ranks
 * of one NVLink box each run the layer for their own experts on the full, replicated token
 * batch.  Instead of writing a partial [T, 7168] output for a collective, the combine kernel
 * stores each token's weighted row sum straight into the receive buffer of the rank that owns
 * the token (rank r owns tokens [r * ceil(T / world), (r + 1) * ceil(T / world))), with plain
 * peer stores, and the owner adds the rows it received in rank order in fp32.  Rows of tokens
 * without an expert on the sending rank are not sent.
 *
 * peer_buffers[i] is rank i's receive buffer as mapped into THIS process (peer access or an
 * IPC / symmetric-memory mapping; peer_buffers[rank] is the local one); every buffer holds at
 * least moe_fp8_b200_exchange_bytes(capacity, world) bytes, is 256-byte aligned and was zeroed
 * once before the first call.  The layout inside a buffer depends on its token capacity and on
 * `world` only, never on a call's T, so consecutive calls may use different T (all ranks the same
 * T in the same call) without a barrier between them; `capacity_tokens` must be the same on every
 * rank (0 = the handle's max_tokens, which then must be the same on every rank).  `epoch` starts
 * at 1 and grows by exactly 1 on every call, on every rank alike.  The waits on peers are bounded
 * (MOE_FP8_B200_OPT_WAIT_LIMIT_US, default 1 s): a rank that never arrives leaves
 * MOE_FP8_B200_ERR_DEVICE in moe_fp8_b200_check, not a hung GPU. */
typedef struct moe_fp8_b200_exchange {
    void* peer_buffers[8];
    size_t buffer_bytes;   /* size of each buffer */
    int32_t rank;
    int32_t world;         /* 1, 2, 4 or 8 */
    uint32_t epoch;
    int32_t capacity_tokens; /* token capacity the buffers were sized for; 0 = the handle's max_tokens */
} moe_fp8_b200_exchange;

/* Bytes of one receive buffer for calls of up to `capacity_tokens` tokens. */
MOE_FP8_B200_API size_t moe_fp8_b200_exchange_bytes(int capacity_tokens, int world);

/* Where the regions of a receive buffer lie (bytes from its start): out_offsets = {rows of parity 0,
 * rows of parity 1, presence bytes of parity 0, of parity 1}, out_sizes = {bytes of one row region, of
 * one presence region}.  A function of (capacity_tokens, world) alone -- the property the exchange's
 * "no back-signal" argument rests on when T varies between calls.  Host only. */
MOE_FP8_B200_API int moe_fp8_b200_exchange_regions(int capacity_tokens, int world, size_t out_offsets[4],
                                                   size_t out_sizes[2]);

/* args->output receives this rank's owned rows only: [ceil(T / world), 7168] bf16 (rows past
 * T, on the last ranks, are not written).  Everything else as moe_fp8_b200_run. */
MOE_FP8_B200_API int moe_fp8_b200_run_reduce_scatter(moe_fp8_b200_handle h, const moe_fp8_b200_args* args,
                                                     const moe_fp8_b200_exchange* exchange, void* stream);

/* What the handle derives from the weight tensors is made once and remembered BY ADDRESS: the TMA
 * descriptors of gemm1_weights / gemm2_weights and a copy of the two weight-scale tensors in the order
 * the GEMMs' accumulator promotion walks them (one pair of block scales per output tile and K block).
 * A run whose weight or scale pointers differ from the remembered ones redoes that step in front of
 * its kernels, stream-ordered.  If the CONTENTS of the scale tensors change under the same addresses
 * (weights reloaded in place), call this before the next run.  The reference keeps the same kind of
 * pointer-keyed cache for its transposed weight scales (kernel/moe_fp8.cu:3007-3014, 3501-3508) and has
 * no way to invalidate it; its activations-side caches have no counterpart here. */
MOE_FP8_B200_API int moe_fp8_b200_invalidate_weights(moe_fp8_b200_handle h);

/* Table form of the expert placement (see MOE_FP8_B200_OPT_EXPERT_STRIDE): local_slot[g] is the
 * index inside this handle's weight tensors of global expert g, or -1 if another handle holds it;
 * every slot 0 .. num_local_experts-1 must appear exactly once.  Lets the multi-GPU wrapper place
 * experts by measured load.  local_expert_offset is ignored while a table is set; passing NULL
 * drops the table and returns to the placement MOE_FP8_B200_OPT_EXPERT_STRIDE names (contiguous
 * unless that option was set).  Host pointer; synchronises the device once. */
MOE_FP8_B200_API int moe_fp8_b200_set_expert_map(moe_fp8_b200_handle h, const int32_t* local_slot);

/* ---- the operators either side of the layer ---------------------------------------------
 * Quantise-on-entry: bf16 activations x [num_tokens, 7168] (device) -> e4m3 q [num_tokens, 7168]
 * and scales fp32 [56, num_tokens], i.e. exactly the hidden_states / hidden_states_scale pair
 * that run() takes (kernel/moe_fp8.cu:2665-2666; the reference expects its caller to have done
 * this).  1x128 blocks, scale = amax / 448 (1 for an all-zero block), payload
 * e4m3_rn_satfinite(x / scale) -- the scheme of kernel/moe_fp8.cu:1823-1830 with a true division.
 * Asynchronous on `stream`.  x and q must be 16-byte aligned. */
MOE_FP8_B200_API int moe_fp8_b200_quantize_hidden(moe_fp8_b200_handle h, const void* x_bf16, int num_tokens,
                                                  void* q_out, float* scale_out, void* stream);

/* The layer without its last step (what FlashInfer's fused-MoE operator calls
 * do_finalize = false): routing, dispatch, both GEMMs, but no weighted combine.  The views
 * point into the handle's workspace and stay valid until the next run on this handle.
 * Row r of the (token t, pair p) contribution is
 *     expert_offset[pair_code[t*8+p] >> 24] + (pair_code[t*8+p] & 0xffffff),
 * and run()'s output is  out[t,:] = bf16(sum_{p < pair_count[t]} float(y[row_p,:]) * pair_weight[t*8+p])
 * accumulated with fp32 FMAs in pair order (kernel/moe_fp8.cu:2276-2321).  args->output may be
 * NULL.  moe_fp8_b200_finalize applies exactly that last step to the state the latest
 * unfinalized run left in the workspace. */
typedef struct moe_fp8_b200_unfinalized {
    const void* y;                 /* bf16 [row_capacity, 7168] GEMM2 rows, grouped by expert */
    const int32_t* expert_offset;  /* [num_local_experts + 1] first row of each expert (multiples of 128) */
    const int32_t* pair_count;     /* [T] kept (token, local expert) pairs */
    const uint32_t* pair_code;     /* [T, 8] (local expert << 24) | slot inside the expert */
    const float* pair_weight;      /* [T, 8] routing weight * renormalisation * routed_scaling_factor */
    int32_t row_capacity;
} moe_fp8_b200_unfinalized;

MOE_FP8_B200_API int moe_fp8_b200_run_unfinalized(moe_fp8_b200_handle h, const moe_fp8_b200_args* args,
                                                  moe_fp8_b200_unfinalized* views, void* stream);
MOE_FP8_B200_API int moe_fp8_b200_finalize(moe_fp8_b200_handle h, int num_tokens, void* output, void* stream);

/* Synchronises `stream` and returns MOE_FP8_B200_ERR_DEVICE if any kernel of any run since the last
 * check recorded a failure in the device status word.  The word is sticky: kernels only ever move it
 * from 0 to the first failure, a later run does not erase it, and this call clears it once it has
 * reported it (the next run then also clears any counters the failed run left behind).  While a
 * failure is pending the decode kernel (batches of at most 8 tokens) does nothing. */
MOE_FP8_B200_API int moe_fp8_b200_check(moe_fp8_b200_handle h, void* stream);

/* Failure injection FROM THE HOST, for tests of the error path (nothing on the GPU faults, traps or
 * hangs): writes `status` into the device status word as if a kernel had recorded it, and
 * `stale_barrier_arrivals` into the arrival counter of the decode kernel's first grid barrier as a
 * launch that gave up half-way would leave it.  Synchronises `stream`.  No counterpart in the
 * reference, whose errors go to stderr only. */
MOE_FP8_B200_API int moe_fp8_b200_inject_device_status(moe_fp8_b200_handle h, int status,
                                                       unsigned stale_barrier_arrivals, void* stream);

/* Mean device time in ms of the six stages (routing+dispatch, offset scan, permute, GEMM1,
 * GEMM2, combine) over the runs recorded since stage timing was switched on (at most the
 * last 64), measured with CUDA events on the runs' stream; waits for those runs to
 * finish and restarts the count.  Stands in for the per-stage numbers the reference never
 * reports (it has no profiling hooks). */
MOE_FP8_B200_API int moe_fp8_b200_stage_times(moe_fp8_b200_handle h, float out_ms[6], int* out_runs);

/* Copies one intermediate buffer of the last run to host memory (synchronises `stream`).
 * Test and diagnostics hook; stands in for the reference's compile-time debug dumps
 * (kernel/moe_fp8.cu:3166-3300). */
MOE_FP8_B200_API int moe_fp8_b200_read_intermediate(moe_fp8_b200_handle h, int buffer, void* dst_host, size_t bytes,
                                   size_t offset_bytes, void* stream);

/* Resolves the reference's T-keyed dispatch policy on the host (no GPU needed):
 * out[0]=prune, [1]=skip_zero_weight, [2]=keep_limit, [3]=drop_third, and
 * fracs[0]=drop_third_frac, [1]=drop_second_frac (2 local), [2]=drop_second_frac (>=3),
 * out[4]=renorm.  Restates kernel/moe_fp8.cu:508-591, 2732-2790. */
MOE_FP8_B200_API int moe_fp8_b200_reference_policy(int num_tokens, int32_t out_flags[5], float out_fracs[3]);

/* Largest batch the allocation-free routing entry point accepts; its built-in scratch is
 * sized for it (about 270 KB of device memory per GPU, held until the process exits). */
#define MOE_FP8_B200_NOALLOC_MAX_TOKENS 4096

/* Routing + dispatch without any allocation.  This entry point has no counterpart in the
 * reference.  It exists for callers that cannot call cudaMalloc where they need the routing
 * result: code running under a frozen memory pool, inside a latency-critical serving loop,
 * or in a host runtime that forbids allocations by libraries.  It needs no handle: the
 * scratch the stage works in (per-expert row counters, per-token pair tables) is a fixed
 * device array inside the library, so the call performs no cudaMalloc / cudaFree and calls
 * no allocating routine.
 *
 * Inputs: routing_logits fp32 [T,256], routing_bias bf16 [256] (device pointers).
 * Outputs (device pointers, caller-owned): topk_idx_out int32 [T,8], topk_weight_out fp32
 * [T,8] -- the same values moe_fp8_b200_run leaves in MOE_FP8_B200_BUF_TOPK_IDX / _WEIGHT --
 * and expert_count_out int32 [num_local_experts], the routed rows per local expert under
 * the chosen dispatch policy (reference_pruning as in MOE_FP8_B200_OPT_REFERENCE_PRUNING).
 * Work is enqueued on `stream` and the call returns without synchronising.
 *
 * Limits and rules:
 *  - num_tokens above MOE_FP8_B200_NOALLOC_MAX_TOKENS is refused with
 *    MOE_FP8_B200_ERR_CAPACITY (err, if given, receives the text).
 *  - The call works on the CURRENT CUDA device: its scratch and its launch are that device's, and
 *    tensors that live on another GPU are refused with MOE_FP8_B200_ERR_INVALID_ARGUMENT.
 *  - local_expert_offset is a multiple of 32 with offset + num_local_experts <= 256, as in
 *    moe_fp8_b200_run.
 *  - The first call on each GPU looks up the scratch array's device address; make that
 *    first call with the GPU current and before any stream capture begins.
 *  - Every call on a GPU uses the same scratch and the scratch keeps the last call's
 *    contents (the counters are cleared at the start of each call).  Calls that overlap
 *    on one GPU race on it: serialise them (one stream, or events between streams).
 * err / err_len: optional buffer for an error message (may be NULL / 0). */
MOE_FP8_B200_API int moe_fp8_b200_route_noalloc(const float* routing_logits, const void* routing_bias,
                                                int32_t num_tokens, int64_t local_expert_offset,
                                                int32_t num_local_experts, double routed_scaling_factor,
                                                int32_t reference_pruning, int32_t* topk_idx_out,
                                                float* topk_weight_out, int32_t* expert_count_out, void* stream,
                                                char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* MOE_FP8_B200_H_ */
