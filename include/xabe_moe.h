/*
 * xabe_moe.h -- C ABI of the sm_100a MoE FFN kernel set (libxabe_moe_sm100.so).
 *
 * The reference project has no FFI layer on this path: xabe-engine calls Rust
 * methods of `xabe_cuda::kernels::moe::MoeKernels` and of
 * `xabe_engine::block::moe::MoeBlock`.  Each entry point below mirrors one of
 * those methods one to one (cited by file:line, paths relative to the
 * reference project root), so that a thin `extern "C"` shim in xabe-cuda can
 * replace their bodies.
 *
 * Conventions
 *  - Every pointer named `dev_*`, every `const float*`/`float*` argument of a
 *    launch call and every buffer in `xabe_moe_buffer_view` is DEVICE memory
 *    on the handle's device.  The caller owns weights, inputs and outputs;
 *    the handle owns only scratch allocated once by xabe_moe_create.
 *  - `stream` is a `cudaStream_t` passed as `void*`.  Launch calls only
 *    enqueue: no synchronisation, no allocation, no host read-back, and every
 *    grid is a function of the geometry alone.  The live token count lives in
 *    a device scalar (crates/xabe-cuda/src/kernels/moe.rs:34-41).
 *  - Quantized tensors stay in GGUF FILE layout: 210-byte Q6_K superblocks and
 *    34-byte Q8_0 blocks, not re-strided (the reference pads Q6_K to 224 B in
 *    `to_device_layout`, moe.rs:410-444; this library reads the raw bytes).
 *    `dev_bytes` must be 16-byte aligned.
 *  - Every call returns an `xabe_status`; on failure a thread-local message
 *    is available from xabe_moe_last_error().  Shapes and formats are
 *    validated before anything is launched (moe.rs:6729-6746).  Nothing
 *    throws across the boundary.
 *  - One handle per host thread (the reference takes `&mut self`).
 *  - There is no CPU fallback: without a CUDA device every entry point that
 *    needs one returns XABE_ERR_DRIVER.
 */
#ifndef XABE_MOE_H
#define XABE_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* MoeError / MoeBlockError variants (moe.rs:4602-4637, crates/xabe-engine/src/block/moe.rs:493-547) */
typedef enum xabe_status {
    XABE_OK = 0,
    XABE_ERR_UNSUPPORTED_GEOMETRY = 1,   /* MoeError::UnsupportedGeometry */
    XABE_ERR_RAGGED_WEIGHTS = 2,         /* MoeError::RaggedWeights */
    XABE_ERR_WRONG_ELEMENT_COUNT = 3,    /* MoeError::WrongElementCount */
    XABE_ERR_TOO_MANY_TOKENS = 4,        /* MoeError::TooManyTokens / MoeBlockError::TooManyTokens */
    XABE_ERR_SHARED_ONLY_BUFFERS = 5,    /* MoeError::SharedOnlyBuffers */
    XABE_ERR_DRIVER = 6,                 /* MoeError::Driver */
    XABE_ERR_BUFFER_LENGTH = 7,          /* MoeBlockError::BufferLength */
    XABE_ERR_UNSUPPORTED_EXPERT_TYPE = 8,/* MoeBlockError::UnsupportedExpertType */
    XABE_ERR_UNSUPPORTED_DENSE_TYPE = 9, /* MoeBlockError::UnsupportedDenseType */
    XABE_ERR_INVALID_ARGUMENT = 10,      /* null pointer, misaligned tensor */
    XABE_ERR_DEVICE_STATUS = 11          /* a kernel recorded a bounded-wait timeout */
} xabe_status;

/* ExpertQuant::code (moe.rs:319-327) */
#define XABE_QUANT_Q6_K 0
#define XABE_QUANT_Q8_0 1

/* BufferScope (moe.rs:4682-4694) */
#define XABE_SCOPE_ROUTED 0
#define XABE_SCOPE_SHARED_ONLY 1

/* MoeGeometry (moe.rs:4523-4540) */
typedef struct xabe_moe_geometry {
    uint32_t num_experts;
    uint32_t experts_per_token;
    uint32_t hidden;
    uint32_t intermediate;
    uint32_t block_size;
    uint32_t max_tokens;
} xabe_moe_geometry;

/* QuantTensor (moe.rs:448-464) */
typedef struct xabe_quant_tensor {
    const void* dev_bytes;
    size_t n_bytes;
    int32_t quant;
} xabe_quant_tensor;

/* MoeLayerWeights (crates/xabe-engine/src/block/moe.rs:634-658) */
typedef struct xabe_moe_layer_weights {
    const float* post_norm;          /* [hidden] */
    const float* router;             /* [num_experts][hidden], expert row contiguous */
    const float* router_bias;        /* [num_experts] added to the logits, or NULL.  Not in the reference
                                        (Qwen3.6 has none); carries the benchmark's Zipf routing skew. */
    xabe_quant_tensor gate_exps;     /* [num_experts][intermediate][hidden] */
    xabe_quant_tensor up_exps;       /* [num_experts][intermediate][hidden] */
    xabe_quant_tensor down_exps;     /* [num_experts][hidden][intermediate] */
    const float* shared_gate_inp;    /* [hidden] */
    xabe_quant_tensor shared_gate;   /* [intermediate][hidden] */
    xabe_quant_tensor shared_up;     /* [intermediate][hidden] */
    xabe_quant_tensor shared_down;   /* [hidden][intermediate] */
} xabe_moe_layer_weights;

/* MoeBuffers accessors (moe.rs:4713-4864) and the MoeBlock intermediates
 * (crates/xabe-engine/src/block/moe.rs:1022-1060). */
typedef struct xabe_moe_buffer_view {
    const int32_t* valid_tokens;        /* device scalar */
    const int32_t* topk_ids;            /* [max_tokens][k] */
    const float* topk_weights;          /* [max_tokens][k] */
    const int32_t* sorted_token_ids;    /* [sorted_capacity] */
    const int32_t* expert_ids;          /* [expert_block_capacity] */
    const int32_t* num_tokens_post_pad; /* device scalar */
    const float* partial;               /* [max_tokens*k][hidden], weighted contributions */
    const float* normed;                /* [max_tokens][hidden]  attn_post_norm */
    const float* logits;                /* [max_tokens][num_experts] */
    const float* routed;                /* [max_tokens][hidden]  ffn_moe_out */
    const float* shexp;                 /* [max_tokens][hidden]  shared expert, ungated */
    const float* gate;                  /* [max_tokens]          sigmoid gate */
    uint64_t sorted_capacity;           /* MoeGeometry::sorted_capacity, moe.rs:4575-4584 */
    uint64_t expert_block_capacity;     /* moe.rs:4587-4589 */
} xabe_moe_buffer_view;

typedef struct xabe_moe xabe_moe;

/* Thread-local text of the last failure on this thread ("" if none). */
const char* xabe_moe_last_error(void);

/* ABI revision of this header. */
int xabe_moe_abi_version(void);

/* How many kernels this library has launched in this process so far, counted at the launch sites
 * (a launch recorded into a CUDA graph during capture counts once, at capture).  No counterpart in
 * the reference; a benchmark uses the difference around a step to state its launches per step. */
uint64_t xabe_kernel_launch_count(void);

/* MoeGeometry::{sorted_capacity, expert_block_capacity} (moe.rs:4575-4589). Pure host. */
uint64_t xabe_moe_sorted_capacity(const xabe_moe_geometry* g);
uint64_t xabe_moe_expert_block_capacity(const xabe_moe_geometry* g);

/* MoeKernels::new + MoeKernels::buffers + MoeBlock::new (moe.rs:5038-5111,
 * 5362-5403; block/moe.rs:948-977).  Validates the geometry exactly as the
 * reference does, then allocates every scratch buffer once.  `scope` is
 * XABE_SCOPE_ROUTED or XABE_SCOPE_SHARED_ONLY (dense FFN: no routing tables).
 * `eps` is the RMSNorm epsilon (block/moe.rs:179). */
int xabe_moe_create(const xabe_moe_geometry* geometry, int device, int scope, float eps,
                    xabe_moe** out);
void xabe_moe_destroy(xabe_moe* m);

/* MoeKernels::set_valid_tokens (moe.rs:5473-5491): publishes the live token
 * count into the device scalar; a no-op when unchanged.  Call it before a
 * stream capture, as MoeBlock::publish_tokens does (block/moe.rs:1074-1089). */
int xabe_moe_set_valid_tokens(xabe_moe* m, void* stream, int tokens);

/* LayerOpsKernels::rms_norm as the block calls it (layer_ops.rs:777,
 * block/moe.rs:1121-1129): normed = x * (1/sqrt(mean(x^2)+eps)) * weight for
 * the live rows.  Result lands in the handle's `normed` buffer (and a
 * half-precision copy the expert kernels read). */
int xabe_moe_rms_norm(xabe_moe* m, void* stream, const float* x, const float* weight);

/* moe_block_router_logits (block/moe.rs:301-382): logits[t][e] =
 * dot(router[e], normed[t]), summed in the order that kernel pins, so logits
 * are bit-identical at every batch width.  Reads the handle's `normed`.
 * `bias` ([num_experts], may be NULL) is added to each logit afterwards. */
int xabe_moe_router_logits(xabe_moe* m, void* stream, const float* router, const float* bias);

/* MoeKernels::route_and_dispatch (moe.rs:5498-5558): softmax over all experts,
 * top-k (probability desc, index asc), renormalise over the selected k, then
 * the block-aligned dispatch tables of moe_align_block_size.  `logits` is
 * [max_tokens][num_experts]; pass NULL to use the handle's own logits. */
int xabe_moe_route_and_dispatch(xabe_moe* m, void* stream, const float* logits);

/* MoeKernels::build_dispatch (moe.rs:5623-5714): the dispatch tables from a
 * routing decision that already exists.  `topk_ids` [max_tokens][k] int32 and
 * `topk_weights` [max_tokens][k] f32 are copied into the handle (either may be
 * NULL = keep what the handle holds).  Expert parallelism uses it on the rank
 * that owns the experts: the rows it received are "tokens" with k = 1. */
int xabe_moe_build_dispatch(xabe_moe* m, void* stream, const int32_t* topk_ids, const float* topk_weights);

/* The last launch of MoeBlock::forward on its own (moe_block_gate_and_combine,
 * block/moe.rs:424-483, 1297-1326): routed = ascending-k sum of the handle's
 * `partial`, gate = sigmoid(dot(shared_gate_inp, normed)), ffn_out = routed +
 * shexp * gate, l_out = ffn_out + residual.  Expert parallelism calls it after
 * the combine exchange has filled `partial`. */
int xabe_moe_gate_and_combine(xabe_moe* m, void* stream, const float* shared_gate_inp, const float* residual,
                              size_t residual_len, float* ffn_out, size_t ffn_out_len, float* l_out,
                              size_t l_out_len);

/* MoeKernels::grouped_forward_partial (moe.rs:5727-6188): routed experts over
 * the current dispatch tables; leaves weight * expert_mlp in `partial`.
 * `hidden_states` NULL = the handle's `normed`. */
int xabe_moe_grouped_forward_partial(xabe_moe* m, void* stream, xabe_quant_tensor gate,
                                     xabe_quant_tensor up, xabe_quant_tensor down,
                                     const float* hidden_states);

/* grouped_forward_partial over caller-provided f16 rows ([n_rows][hidden],
 * 16-byte aligned), read in place: row r is "token" r of the current dispatch
 * tables.  No counterpart in the reference (whose multi-GPU model is one
 * replica per device): expert parallelism uses it on the rank that owns the
 * experts, directly on the buffer the dispatch exchange filled. */
int xabe_moe_grouped_forward_partial_f16(xabe_moe* m, void* stream, xabe_quant_tensor gate,
                                         xabe_quant_tensor up, xabe_quant_tensor down,
                                         const void* rows_f16, size_t n_rows);

/* Expert parallelism, sender side; no counterpart in the reference.
 * ep_pack: for i < n_pairs, send_rows_f16[i] = the handle's normalised f16
 * activation row of the token of flat (token, k) pair order[i];
 * send_local_expert[i] = topk_ids[order[i]] % experts_per_rank;
 * inverse[order[i]] = i.  `order` holds every live pair once, grouped by
 * owner rank.
 * ep_combine: gate_and_combine with the routed term taken from `back_rows`
 * ([n_rows][hidden] f32, unweighted expert outputs in the order of `order`):
 * routed[t] = sum over ascending k of topk_weights[t][k] *
 * back_rows[inverse[t*k_per_token + k]], each product rounded before it is
 * added, which is bit-identical to the one-GPU block. */
/* ep_plan_pack: ep_pack with the send order taken from the dispatch tables the
 * handle already holds (pairs sorted by expert are grouped by owner rank):
 * fills the same three outputs for all live pairs and writes the number of
 * pairs bound for each rank to send_counts[num_experts / experts_per_rank]
 * (device memory).  No counterpart in the reference. */
int xabe_moe_ep_plan_pack(xabe_moe* m, void* stream, int experts_per_rank, void* send_rows_f16,
                          int32_t* send_local_expert, int32_t* inverse, int32_t* send_counts);
int xabe_moe_ep_pack(xabe_moe* m, void* stream, const int64_t* order, size_t n_pairs, int experts_per_rank,
                     void* send_rows_f16, int32_t* send_local_expert, int32_t* inverse);
int xabe_moe_ep_combine(xabe_moe* m, void* stream, const float* back_rows, size_t n_rows,
                        const int32_t* inverse, const float* shared_gate_inp, const float* residual,
                        size_t residual_len, float* ffn_out, size_t ffn_out_len, float* l_out,
                        size_t l_out_len);

/* MoeKernels::grouped_forward (moe.rs:6345-6375): the above plus the
 * ascending-k sum of moe_reduce (moe.rs:4049-4065) into `out`
 * [max_tokens][hidden]. */
int xabe_moe_grouped_forward(xabe_moe* m, void* stream, xabe_quant_tensor gate,
                             xabe_quant_tensor up, xabe_quant_tensor down,
                             const float* hidden_states, float* out);

/* MoeKernels::shared_expert (moe.rs:6488-6727): expert_mlp of one expert for
 * every live token, ungated.  `out` NULL = the handle's `shexp`. Also the
 * dense FFN of the 27B sibling (block/dense_ffn.rs:9-16). */
int xabe_moe_shared_expert(xabe_moe* m, void* stream, xabe_quant_tensor gate,
                           xabe_quant_tensor up, xabe_quant_tensor down,
                           const float* hidden_states, float* out);

/* MoeBlock::forward (block/moe.rs:1091-1329): the whole block.  `residual`,
 * `ffn_out`, `l_out` are [max_tokens][hidden] f32 device buffers whose element
 * counts are checked like check_len (block/moe.rs:1107-1110).  Rows at and
 * beyond `tokens` are never written. */
int xabe_moe_block_forward(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w,
                           const float* residual, size_t residual_len, int tokens,
                           float* ffn_out, size_t ffn_out_len, float* l_out, size_t l_out_len);

/* The MoE half of Forward::body (crates/xabe-engine/src/forward.rs:3497-3618)
 * for a stack whose layers are MoE blocks only (the mixers between them are
 * not part of this library): layer i runs xabe_moe_block_forward with layer
 * i's weights on the hidden state layer i - 1 left, `hidden_a` holding the
 * input and the two buffers alternating as residual and l_out, as
 * `mixer_out` and `hidden_state` do there.  Launches only: nothing reads host
 * memory, allocates or synchronises, and the live token count is the device
 * scalar, so the call can be captured once as a CUDA graph and replayed at any
 * `tokens` published with xabe_moe_set_valid_tokens.  Every layer's tensors
 * are checked before the first launch (check_stack, moe.rs:6729-6746).
 * `*final_hidden` (may be NULL) receives the buffer that holds the last
 * layer's l_out (`hidden_a` for an even layer count); `ffn_out` holds the last
 * layer's. */
int xabe_moe_stack_forward(xabe_moe* m, void* stream, const xabe_moe_layer_weights* layers, int n_layers,
                           float* hidden_a, float* hidden_b, size_t hidden_len, int tokens,
                           float* ffn_out, size_t ffn_out_len, float** final_hidden);

/* The same call for a caller that holds HOST buffers: copies `tokens` rows of
 * `host_residual` to the device, runs the block and copies `ffn_out`/`l_out`
 * rows back, all on `stream`; returns after enqueueing (synchronise the
 * stream before reading).  Host buffers should be pinned.  Either output may
 * be NULL.  (The reference reaches this through `Forward`, which uploads the
 * step's inputs itself: crates/xabe-engine/src/forward.rs:3534-3585.) */
int xabe_moe_block_forward_host(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w,
                                const float* host_residual, int tokens, float* host_ffn_out,
                                float* host_l_out);

/* DenseFfnBlock::forward (block/dense_ffn.rs:1047): l_out = mlp(rmsnorm(x)) + x.
 * The handle must have been created with geometry.hidden/intermediate of the
 * dense model; XABE_SCOPE_SHARED_ONLY is enough. */
int xabe_dense_ffn_block_forward(xabe_moe* m, void* stream, const float* post_norm,
                                 xabe_quant_tensor gate, xabe_quant_tensor up,
                                 xabe_quant_tensor down, const float* residual,
                                 size_t residual_len, int tokens, float* ffn_out,
                                 size_t ffn_out_len, float* l_out, size_t l_out_len);

/* MoeBlock::buffers and the intermediate accessors (block/moe.rs:1022-1060). */
int xabe_moe_buffers(xabe_moe* m, xabe_moe_buffer_view* out);

/* MoeKernels::set_exact_decode_regime (moe.rs:5450): pin the routed experts to
 * the decode-shaped kernels whatever the token width, so a row's floats land
 * exactly where plain decode's would. */
int xabe_moe_set_exact_decode_regime(xabe_moe* m, int on);

/* MoeKernels::disable_tensor_cores (moe.rs:5416-5418): from now on this handle never runs the
 * tcgen05 grouped GEMMs; every width takes the decode-shaped kernels (exact integer codes, fp32
 * scales), which is the path the tight differential gate is stated on.  Not reversible, as in the
 * reference.  Contractions the decode kernels cannot hold (the dense 27B block) fall back to the
 * one-tile-per-CTA kernels.  tensor_cores_enabled mirrors moe.rs:5456-5458. */
int xabe_moe_disable_tensor_cores(xabe_moe* m);
int xabe_moe_tensor_cores_enabled(const xabe_moe* m);

/* The opposite switch, for differential tests of the tcgen05 kernels at widths that would not
 * select them (the reference's tests reach its MMA path the same way, by handle switch rather than
 * by environment: tests/moe_differential.rs:118-145).  Must be chosen before route_and_dispatch,
 * which builds the work list of the kernels that will run.  Ignored while the exact-decode regime
 * or disable_tensor_cores is in force. */
int xabe_moe_force_prefill_path(xabe_moe* m, int on);

/* Per-handle tuning switches; none changes a result, only which launch shape produces it.  They
 * replace process-wide environment reads: a host with several handles sets each one's own.
 * PREFILL_WIDE allocates (set-up time only); the others are plain field writes. */
#define XABE_TUNE_PDL 0                /* 1: programmatic dependent launch between the block's kernels */
#define XABE_TUNE_STREAM_STAGES 1      /* ring depth cap of the streaming kernels (0 = as many as fit) */
#define XABE_TUNE_STREAM_RUNS 2        /* k_expert_stream work split override (0 = the kernel's choice) */
#define XABE_TUNE_ROWS_MIN_TOKENS 3    /* narrowest handle that runs gate/up through k_gateup_rows (0 = never, -1 = default) */
#define XABE_TUNE_ROUTER_REGW 4        /* router kernel with expert rows in registers: 0 off, 1 sixteen rows per CTA
                                          (one CTA per SM), 2 eight rows (two CTAs per SM), -1 by width (from 256 tokens: 2) */
#define XABE_TUNE_FORCE_TILE_KERNELS 5 /* 1: the one-tile-per-CTA expert kernels everywhere */
#define XABE_TUNE_PREFILL_WIDE 6       /* 1 or 4: k_prefill_gemm_wide with up to four 128-column accumulators per unpacked
                                          weight pair; 2, 3: up to two or three; 0: k_prefill_gemm (one) */
#define XABE_TUNE_FUSED_DECODE 7       /* bit 0: handles under 16 tokens fold gate-and-combine into the down launch;
                                          bit 1: handles up to 256 tokens run norm, router, routing and dispatch as one
                                          launch.  3 = a three-launch layer at up to 15 tokens; both measured no
                                          faster than the separate launches under CUDA-graph replay, so they are off;
                                          bit 2: handles of one or two tokens let the router normalise its input rows
                                          itself (no RMSNorm launch).  Default 4. */
#define XABE_TUNE_DENSE_ROWS 8         /* 0: the dense block of up to 64 tokens through the tcgen05 kernels instead of
                                          k_dense_rows (default 1) */
int xabe_moe_set_tuning(xabe_moe* m, int key, int value);

/* Iteration limit (x 200 ns) of this handle's waits on other ranks' flags in the peer-memory
 * exchange; 0 restores the default of several seconds.  A wait that runs out records device
 * status 3 and the owner-side step that follows it moves nothing (see ep_p2p_receive). */
int xabe_moe_set_peer_wait_limit(xabe_moe* m, uint32_t iterations);

/* Reads (and clears) the device status word the kernels' bounded waits write:
 * 0 when every wait completed.  Synchronises `stream`. */
int xabe_moe_device_status(xabe_moe* m, void* stream, int* status_out);

/* StageProfile (crates/xabe-engine/src/forward.rs:783-855): CUDA-event spans
 * around the stages of xabe_moe_block_forward, pre-allocated, off by default.
 * Stages: 0 rms_norm, 1 router logits, 2 route + dispatch, 3 gate/up + SwiGLU
 * (routed and shared), 4 down, 5 gate-and-combine.  xabe_moe_stage_times
 * synchronises `stream`, returns the summed milliseconds per stage over the
 * calls recorded since the last read (at most 256) and resets the record. */
#define XABE_STAGE_COUNT 6
int xabe_moe_stage_profile(xabe_moe* m, int on);
int xabe_moe_stage_times(xabe_moe* m, void* stream, float* ms_sum, int* calls);

/* Standalone dequantisation (crates/xabe-cuda/src/kernels/dequant.rs, gated
 * bit-identical by crates/xabe-engine/tests/dequant_differential.rs:1-18):
 * `out` receives n_bytes / block_bytes * block_elements floats. */
int xabe_dequantize(void* stream, xabe_quant_tensor t, float* out);

/* Shared-expert MLP (expert_mlp of one expert for `tokens` rows, ungated) for
 * callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Who needs it: a worker whose device memory was all handed out at
 * start-up and is guarded by its own arena, or code that runs where the CUDA
 * allocator must not be entered (a latency-critical callback, a region under
 * another allocator's lock) -- such callers cannot call xabe_moe_create, which
 * allocates.  This call allocates nothing, on the host or on the device: its
 * scratch (f16 activations, f16 SwiGLU intermediate, two control words) is a
 * 327,936-byte static device array that every GPU loading the library holds
 * until the process exits.
 *   limits: tokens <= 64, hidden <= 2048, intermediate <= 512 (both multiples
 *           of 256); anything larger is rejected with a status and a message.
 *   `hidden_states` [tokens][hidden] f32 and `out` [tokens][hidden] f32 are
 *   device buffers of the caller; weights as for xabe_moe_shared_expert.
 *   The first call on a device looks up the array's device address; make that
 *   first call before any stream capture.  All calls share the one array, which
 *   keeps the previous call's contents (the call rewrites every word it later
 *   reads): two calls whose kernels overlap on the GPU -- different streams, or
 *   different host threads -- race on it, so keep them on one stream.  The array
 *   belongs to the CURRENT device: make the stream's device current before the
 *   call.  Host threads may make their first calls concurrently (the address
 *   look-up is an atomic, same-value store). */
int xabe_shared_expert_noalloc(void* stream, xabe_quant_tensor gate, xabe_quant_tensor up,
                               xabe_quant_tensor down, int hidden, int intermediate,
                               const float* hidden_states, int tokens, float* out);

/* Companion of xabe_shared_expert_noalloc, equally without a counterpart in the
 * reference and equally allocation-free: the kernels' bounded waits on their
 * bulk copies record a status word inside the static array, and a caller with
 * no handle has no other way to learn that one ran out (`out` is then partly
 * unwritten).  Copies that word into `*status_out` (host memory) and
 * synchronises `stream`: 0 = every wait of the last call completed; otherwise
 * XABE_ERR_DEVICE_STATUS is returned as well. */
int xabe_shared_expert_noalloc_status(void* stream, int* status_out);

/* Expert-parallel exchange over peer memory (NVLink) instead of a library
 * all-to-all; no counterpart in the reference.  Every rank owns six buffers
 * that the other ranks have mapped (CUDA IPC); entry r of each array is rank
 * r's buffer as THIS process sees it (entry `rank` = the rank's own).
 * G = world, C = cap = the most pairs one rank can send (its max_tokens x k):
 *   rows      [G][C][hidden] f16   region s is written by rank s
 *   eid       [G][C] int32         expert id local to the owner
 *   meta      [G][2] int32         {rows rank s sent, their start in s's send order}
 *   flag_in   [G] int32            rank s stores `step` once rows and meta are written
 *   back      [C][hidden] f32      owners write results in this rank's send order
 *   flag_back [G] int32            owner d stores `step` once its results are written
 * `step` must grow by one per layer call (flags are never reset; start the
 * buffers at zero).  Call order per layer: on the tokens' handle, after
 * route_and_dispatch: ep_p2p_send; on the owner-side handle (k = 1, max_tokens
 * = G*C): ep_p2p_receive -> build_dispatch(ids) -> grouped_forward_partial_f16
 * (rows = this rank's `rows` buffer) -> ep_p2p_return; on the tokens' handle:
 * ep_p2p_wait_results -> ep_combine(back).  Waits on other ranks are bounded
 * (xabe_moe_set_peer_wait_limit): a timeout sets device status 3; ep_p2p_receive
 * then reports every slot empty (ids -1, null destinations), so the experts do
 * not run and nothing is stored into a peer; the step's output is meaningless. */
/* Buffers for the peer-memory exchange: device memory of the CURRENT device
 * that another process of this node can map.  ipc_alloc: cudaMalloc, zeroed,
 * plus its 64-byte CUDA IPC handle (send it to the other ranks by any means);
 * ipc_open: maps a peer's buffer into this process with peer access from the
 * current device; ipc_close / ipc_free undo them.  Set-up time only. */
int xabe_ipc_alloc(size_t bytes, void** dev_ptr, unsigned char* handle64);
int xabe_ipc_open(const unsigned char* handle64, void** dev_ptr);
int xabe_ipc_close(void* dev_ptr);
int xabe_ipc_free(void* dev_ptr);

typedef struct xabe_ep_peers {
    void* rows[8];
    void* eid[8];
    void* meta[8];
    void* flag_in[8];
    void* back[8];
    void* flag_back[8];
} xabe_ep_peers;
int xabe_moe_ep_p2p_send(xabe_moe* m, void* stream, int experts_per_rank, int world, int rank, int cap,
                         const xabe_ep_peers* peers, int step, int32_t* inverse);
int xabe_moe_ep_p2p_receive(xabe_moe* m, void* stream, int world, int rank, int cap, const xabe_ep_peers* peers,
                            int step, int32_t* ids_out, void* result_dst);
int xabe_moe_ep_p2p_return(xabe_moe* m, void* stream, int world, int rank, int cap, const xabe_ep_peers* peers,
                           int step, const void* result_dst);
/* Fused form of the result push: while `table` (the `result_dst` array that
 * ep_p2p_receive filled: one destination row pointer per receive slot) is set,
 * the down projection stores weight * value of row r through table[r] -- peer
 * stores over NVLink straight from the GEMM epilogue -- instead of into the
 * handle's `partial`, and ep_p2p_return with the same table only raises the
 * flags.  NULL restores the normal destination.  No counterpart in the
 * reference. */
int xabe_moe_set_result_destinations(xabe_moe* m, const void* table);
int xabe_moe_ep_p2p_wait_results(xabe_moe* m, void* stream, int world, int rank, const xabe_ep_peers* peers,
                                 int step);

/* MoeBlock::forward with a dtype tag on the residual stream: XABE_DTYPE_F32 is
 * xabe_moe_block_forward; XABE_DTYPE_BF16 takes [max_tokens][hidden] bf16 rows
 * (a prefill chunk as the layers before it produce it), widens the live rows
 * exactly (a 16-bit shift) and proceeds as above; ffn_out and l_out stay f32,
 * and the residual added into l_out is the widened value.  The reference's
 * block takes f32 only (block/moe.rs:1091-1099). */
#define XABE_DTYPE_F32 0
#define XABE_DTYPE_BF16 1
int xabe_moe_block_forward_typed(xabe_moe* m, void* stream, const xabe_moe_layer_weights* w,
                                 const void* residual, int residual_dtype, size_t residual_len, int tokens,
                                 float* ffn_out, size_t ffn_out_len, float* l_out, size_t l_out_len);

/* Benchmark calibration, no counterpart in the reference's kernel set (its
 * benchmark prints the same row, docs/BENCHMARKS.md:448-452): one pass of
 * 128-bit coalesced loads over [dev_bytes, dev_bytes + n_bytes) with no
 * arithmetic.  `sink` is 4 bytes of device memory (practically never written). */
int xabe_stream_read(void* stream, const void* dev_bytes, size_t n_bytes, void* sink);

/* ---------------------------------------------------------------------------
 * LM head (crates/xabe-cuda/src/kernels/lm_head.rs): logits = W x over the
 * whole vocabulary, W in file layout.  Next to the MoE path because it is the
 * same streaming machinery on the largest single tensor of the model.
 * --------------------------------------------------------------------------- */

/* LmHeadGeometry (lm_head.rs:1304-1314) */
typedef struct xabe_lm_head_geometry {
    uint32_t hidden;
    uint32_t vocab;
    uint32_t max_tokens;
} xabe_lm_head_geometry;

typedef struct xabe_lm_head xabe_lm_head;

/* LmHeadKernels::new (lm_head.rs:1528-1680): validates the geometry (hidden a
 * multiple of 256, at most 4096) and allocates the handle's scratch (two f16
 * copies of the activations).  The only call of this group that allocates. */
int xabe_lm_head_create(const xabe_lm_head_geometry* geometry, int device, xabe_lm_head** out);
void xabe_lm_head_destroy(xabe_lm_head* m);

/* LmHeadKernels::forward (lm_head.rs:1695-1937).  `weight` is the head tensor
 * [vocab][hidden] in file layout, XABE_QUANT_Q8_0 (HeadFormat::Q8_0, the
 * Qwen3.6 head) or XABE_QUANT_Q6_K (HeadFormat::Q6K); the dense 16-bit and the
 * community formats return XABE_ERR_UNSUPPORTED_DENSE_TYPE.  `hidden_states`
 * is [max_tokens][hidden] f32 and `logits` [max_tokens][vocab] f32, both
 * length-checked; rows at and past `tokens` are neither read nor written.  A
 * batch costs ceil(tokens / 8) passes over the weights (weight_passes,
 * lm_head.rs:1380-1383).  Launches only. */
int xabe_lm_head_forward(xabe_lm_head* m, void* stream, xabe_quant_tensor weight, const float* hidden_states,
                         size_t hidden_states_len, int tokens, float* logits, size_t logits_len);

/* LmHeadKernels::argmax (lm_head.rs:1950-2015): out[t] = index of the largest
 * logit of row t, ties to the lower index (gemv.rs:102-111).  `out` holds
 * max_tokens int32 on the device. */
int xabe_lm_head_argmax(xabe_lm_head* m, void* stream, const float* logits, size_t logits_len, int tokens,
                        int32_t* out);

/* As xabe_moe_device_status, for this handle's kernels. */
int xabe_lm_head_device_status(xabe_lm_head* m, void* stream, int* status_out);

#ifdef __cplusplus
}
#endif
#endif /* XABE_MOE_H */
