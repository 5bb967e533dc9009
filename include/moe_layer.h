/* The MoE expert layer's C ABI: router, pack, quantised expert FFN, shared expert and combine on one B200.
 *
 * The reference's own ABI (include/engine_api.h:308-421) is whole-engine: open, admit, submit, poll. Its MoE block
 * has no entry point of its own; it runs inside Model::step (core/models/qwen4exp/model.cpp:1348-1418) and
 * Model::prompt_runs (core/models/qwen4exp/prompt.cpp:606-656), with the CPU's share behind CpuExperts::compute_many
 * (core/cpu/experts.h:32-53). This header is the layer-level boundary those call sites would bind, written to the
 * same rules as engine_api.h:1-10: plain structs and buffers only, every call returns a status, no exception and no
 * callback crosses, the library owns all device memory and streams. Weights come in the GGUF block formats of
 * shared/quant.h:36-169 in the file's layout; results are the ones the reference's kernels leave in ids, w, inv and
 * tiles (shared/moe_tile.h:9-18) and the block's output rows. */
#ifndef MOE_LAYER_H
#define MOE_LAYER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(MOE_API_EXPORT)
#define MOE_API __attribute__((visibility("default")))
#else
#define MOE_API
#endif

#define MOE_API_VERSION 2

/* engine_status's values (include/engine_api.h:28-34). */
typedef enum {
  MOE_OK = 0,
  MOE_ERROR = 1, /* see moe_last_error */
  MOE_BAD_ARGUMENT = 2,
  MOE_BUSY = 3,
  MOE_TIMEOUT = 4
} moe_status;

/* Weight types, ggml's numbers (shared/quant.h:10-33). */
#define MOE_TYPE_Q8_0 8
#define MOE_TYPE_Q4_K 12
#define MOE_TYPE_Q6_K 14
#define MOE_TYPE_IQ3_XXS 18
#define MOE_TYPE_IQ4_NL 20
#define MOE_TYPE_IQ3_S 21
#define MOE_TYPE_IQ2_S 22
#define MOE_TYPE_IQ4_XS 23
#define MOE_TYPE_Q2_0 42 /* the reference's fork of ggml (shared/quant.h:33) */

typedef struct moe_layer moe_layer;

/* The shape CpuExperts takes as ExpertShape (core/cpu/experts.h:23-30), with the router's sizes and where the layer
 * lives. Zero means the default given. */
typedef struct {
  uint32_t n_embd;            /* hidden size, a multiple of 256 */
  uint32_t n_ff;              /* an expert's inner size, a multiple of 256 */
  uint32_t n_experts;         /* routed experts, a multiple of 32, at most 512 */
  uint32_t n_used;            /* experts per row, at most 16 */
  uint32_t gate_type;         /* the routed experts' gate and up */
  uint32_t down_type;         /* the routed experts' down */
  uint32_t shexp_gate_type;   /* the shared expert's gate and up; 0: no shared expert */
  uint32_t shexp_down_type;
  uint32_t expert_first;      /* expert parallel: this GPU holds experts [expert_first, expert_first + expert_count) */
  uint32_t expert_count;      /* 0: all of them */
  uint32_t max_tokens;        /* rows a call may bring; default 4352, the reference's prompt chunk */
  int32_t device;             /* CUDA device ordinal */
  float swiglu_limit;         /* ExpertShape::swiglu_limit; 0: off */
  uint32_t flags;             /* MOE_FLAG_* */
  uint32_t tensor_min_rows;   /* an expert with at least this many rows in a call goes to the tensor-core kernels, one
                                 with fewer to the integer-dot kernels; default 16 */
  uint32_t max_expert_rows;   /* expert parallel: rows moe_layer_experts_device may receive; default max_tokens * n_used */
  uint32_t host_chunk_rows;   /* moe_layer_forward (host buffers): calls of at least twice this many rows are cut into
                                 chunks of about this many, and a chunk's copies to and from the GPU run beside its
                                 neighbours' computation; a row's output does not depend on the cut, but
                                 moe_layer_read_route then describes the last chunk only. 0: never cut */
} moe_layer_config;

#define MOE_FLAG_PROFILE 1u     /* time every stage of a call with events (moe_layer_stage_ms) */
#define MOE_FLAG_NO_TENSOR 2u   /* every expert product by the integer-dot kernels, whatever its rows */
#define MOE_FLAG_GATHER_IN_KERNEL 4u /* long steps (163,840 expert rows and more): the gate/up tile kernel gathers its rows by
                                      * index itself instead of reading a copy made in expert order; that copy and its traffic
                                      * go, the tile kernel runs at the pace of its own copies (slower in all: off by default) */

/* Host pointers, read during moe_layer_create and not kept. Experts are the file's tensors
 * blk.N.ffn_{gate,up,down}_exps.weight cut to this GPU's experts: expert e's slice at e * its bytes, rows of whole
 * blocks (docs/spec/MODEL_LAYER.md 4.1). */
typedef struct {
  const float *router;          /* ffn_gate_inp, [n_experts][n_embd] f32 */
  const float *shexp_gate_inp;  /* ffn_gate_inp_shexp, [n_embd] f32; null with no shared expert */
  const float *router_bias;     /* [n_experts] f32 added to the logits, or null */
  const void *gate_exps;        /* [expert_count][n_ff][n_embd values] */
  const void *up_exps;
  const void *down_exps;        /* [expert_count][n_embd][n_ff values] */
  const void *gate_shexp;       /* [n_ff][n_embd values] */
  const void *up_shexp;
  const void *down_shexp;       /* [n_embd][n_ff values] */
} moe_layer_weights;

/* MoeTile (shared/moe_tile.h:11-16). slot is the expert's index among this GPU's experts. */
typedef struct {
  uint32_t expert;
  uint32_t slot;
  uint32_t start;
  uint32_t count; /* 1 .. 64 */
} moe_tile;

/* Counters since create, read by snapshot as engine_stats is (include/engine_api.h:225-306). */
typedef struct {
  uint64_t calls;             /* forwards run */
  uint64_t rows;              /* rows in them */
  uint64_t assignments;       /* rows x n_used */
  uint64_t kernels;           /* kernels this library launched */
  uint64_t h2d_bytes;         /* copied for host-buffer calls */
  uint64_t d2h_bytes;
  uint64_t last_tiles;        /* of the last call */
  uint64_t last_experts_hit;  /* distinct experts the last call's rows routed to */
  uint64_t last_tensor_rows;  /* of its assignments, those the tensor-core kernels computed */
} moe_layer_stats;

#define MOE_STAGES 8
/* Stage names, in order: "quantize", "router", "pack", "gate_up", "down", "shared", "combine", "copies". */

/* Uploads the weights in the layout the kernels read and allocates every buffer a call needs. */
MOE_API moe_status moe_layer_create(const moe_layer_config *config, const moe_layer_weights *weights, moe_layer **out);
MOE_API void moe_layer_destroy(moe_layer *l);

/* The block on T rows: out[t] = sum over k of w[t][k] * expert ids[t][k] (x[t]) + sigmoid(gate . x[t]) * shared(x[t]).
 * x and out are HOST buffers of T * n_embd floats; the call copies them to and from the GPU and returns when out is
 * written. Page-locked buffers let the copies run at the bus's rate and, with host_chunk_rows set, beside the
 * computation. */
MOE_API moe_status moe_layer_forward(moe_layer *l, const float *x, uint32_t T, float *out);

/* The same on DEVICE buffers, queued on the layer's stream (or on stream, a cudaStream_t, when not null); returns
 * without waiting. Every device pointer of rows this header takes (x, out, y, rows) must be 16-byte aligned, as whole
 * allocations are: the kernels read rows through 16-byte loads, and a pointer that is not is refused with
 * MOE_BAD_ARGUMENT. */
MOE_API moe_status moe_layer_forward_device(moe_layer *l, const float *x_dev, uint32_t T, float *out_dev, void *stream);
/* out = residual + block(x): a stack of layers steps x <- x + block(norm(x)) with no kernel between the layers but the
 * norm (the reference's layers add their block's result into the residual stream likewise,
 * docs/spec/MODEL_LAYER.md 4.4). out_dev may be residual_dev. */
MOE_API moe_status moe_layer_forward_residual_device(moe_layer *l, const float *x_dev, uint32_t T, const float *residual_dev,
                                                     float *out_dev, void *stream);

/* Expert parallel: a layer created with fewer than n_experts experts runs stage by stage, and the caller moves rows
 * between GPUs in between (one process per GPU, an all-to-all for the rows out and one for the results back). The
 * reference has no expert parallelism (both its cards hold the same experts, docs/DESIGN.md:294-297); these calls are
 * this library's own. All pointers are DEVICE pointers; every call queues on stream (null: the layer's) and returns.
 *   route:   quantises x, routes its T rows over all n_experts and sorts the T * n_used assignments by expert.
 *   counts:  copies the rows each expert got (n_experts words) to the host, and waits, or to a device buffer, queued:
 *            what the all-to-all's split sizes are made of.
 *   gather:  rows_dev[r] = the quantised activation row (moe_layer_wire_row_bytes bytes) of assignment row r in expert
 *            order, ids_dev[r] = its expert. Experts are owned in contiguous ranges, so this is destination order.
 *   received_ids: from every GPU's counts (cnt_all_dev [world][n_experts], the all-gather of counts), ids_dev[r] = the
 *            expert of the r-th row this GPU receives when every GPU sends its rows in gather's order: sources one
 *            after another, each in expert order. So no ids travel and the host computes none.
 *   experts: R rows received (any order) with their expert ids, all among this GPU's experts; y_dev[r] = that expert's
 *            FFN on row r, [R][n_embd] in the order received, f32 or (y_f16 != 0) f16.
 *   shared:  the shared expert on the routed rows (may run on another stream than the experts).
 *   combine: y_dev holds the results for this GPU's own assignments in expert order, as gather sent them;
 *            out[t] = sum over k of w[t][k] * y[inv[t n_used + k]] + gate[t] * shared[t]. */
MOE_API moe_status moe_layer_route_device(moe_layer *l, const float *x_dev, uint32_t T, void *stream);
MOE_API moe_status moe_layer_read_counts(moe_layer *l, uint32_t *cnt_host, void *stream);
MOE_API moe_status moe_layer_counts_device(moe_layer *l, uint32_t *cnt_dev, void *stream);
MOE_API moe_status moe_layer_received_ids_device(moe_layer *l, const uint32_t *cnt_all_dev, uint32_t world, int32_t *ids_dev, void *stream);
MOE_API uint32_t moe_layer_wire_row_bytes(const moe_layer *l);
MOE_API moe_status moe_layer_gather_rows_device(moe_layer *l, void *rows_dev, int32_t *ids_dev, void *stream);
MOE_API moe_status moe_layer_experts_device(moe_layer *l, const void *rows_dev, const int32_t *ids_dev, uint32_t R, void *y_dev,
                                            uint32_t y_f16, void *stream);
MOE_API moe_status moe_layer_shared_device(moe_layer *l, void *stream);
MOE_API moe_status moe_layer_combine_device(moe_layer *l, const void *y_dev, uint32_t y_f16, float *out_dev, void *stream);

/* A layer straight from a GGUF file (version 3, one file): the reference reads its layers' tensors through GgufModel
 * (core/load/gguf.h:13-71) and addresses expert e of blk.N.ffn_{gate,up,down}_exps.weight at the tensor's offset plus
 * e times the expert's bytes (core/models/qwen4exp/model.cpp:1045-1057); so does this. The file is mapped, not read:
 * moe_layer_create_from_gguf takes the weights from the mapping and keeps nothing of it.
 *   moe_gguf_open / _close: the file's header and tensor table. Failures' text: moe_last_error(NULL).
 *   moe_gguf_layers: "<general.architecture>.block_count", or 0 if the file does not say.
 *   moe_gguf_tensors: the table, up to cap rows into table (which may be null); returns how many tensors there are.
 *     name points into the handle and lives as long as it; shape is in ggml's order (shape[0] the contiguous axis);
 *     offset is from the file's start; bytes is 0 for a type this library does not read.
 *   moe_layer_create_from_gguf: layer N's blk.N.ffn_gate_inp.weight [n_embd][n_experts] (F32, F16 or BF16),
 *     ffn_gate_exps, ffn_up_exps [n_embd][n_ff][n_experts], ffn_down_exps [n_ff][n_embd][n_experts] and, when the file
 *     has them, ffn_gate_inp_shexp [n_embd] with ffn_{gate,up,down}_shexp. The sizes and types come from the tensors;
 *     of *config the call takes n_used (0: "<architecture>.expert_used_count"), expert_first, expert_count, max_tokens,
 *     device, swiglu_limit, flags, tensor_min_rows, max_expert_rows and host_chunk_rows. */
typedef struct moe_gguf moe_gguf;
typedef struct {
  const char *name;
  uint32_t type;    /* ggml type id */
  uint32_t n_dims;
  uint64_t shape[4];
  uint64_t offset;
  uint64_t bytes;
} moe_gguf_tensor;
MOE_API moe_status moe_gguf_open(const char *path, moe_gguf **out);
MOE_API void moe_gguf_close(moe_gguf *f);
MOE_API uint32_t moe_gguf_layers(const moe_gguf *f);
MOE_API uint32_t moe_gguf_tensors(const moe_gguf *f, moe_gguf_tensor *table, uint32_t cap);
MOE_API moe_status moe_layer_create_from_gguf(const moe_gguf *f, uint32_t layer, const moe_layer_config *config, moe_layer **out);

/* The norm a stack puts in front of each layer's block: out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight (weight null:
 * ones), rows of n_embd floats (a multiple of 4), DEVICE pointers 16-byte aligned, queued on stream. It is what the
 * engine behind include/engine_abi.h runs between its layers, exported so that a caller's own stack needs no other
 * library for it. */
MOE_API moe_status moe_rmsnorm_rows_device(const float *x_dev, const float *weight_dev, uint32_t T, uint32_t n_embd, float eps, float *out_dev,
                                           void *stream);

/* The configuration the layer runs with: the sizes and types it was created with or read from a file, defaults filled in. */
MOE_API moe_status moe_layer_read_config(const moe_layer *l, moe_layer_config *out);

/* Expert parallel with fewer bytes on the wire: one row per (token, GPU) instead of one per assignment. A token's
 * n_used experts live on a few GPUs (for 10 of 512: all of 2, 3.8 of 4, 5.9 of 8 on average), so its quantised row
 * travels once to each GPU that holds any of them, with the list of those experts and their routing weights beside it,
 * and each GPU returns one row: the weighted sum of its experts' results for the token, in the token's rank order, as
 * f16. At home the GPUs' sums are added in GPU order, then the shared expert's gated result. The sum over a token's
 * experts is thus taken GPU by GPU, not in one pass over its ranks: outputs agree with one GPU's within the layer's
 * tolerance, not bit for bit (the per-assignment calls above keep that). GPUs hold equal contiguous expert ranges.
 *   dispatch_plan:  after route. For every token the GPUs its experts live on; totals_dev (DEVICE, 16 words) receives
 *                   the rows this GPU sends to GPUs 0 .. 7 and then the assignments that go with them: what the
 *                   all-to-all's split sizes are made of.
 *   dispatch_rows:  rows_dev (DEVICE) receives the travelling rows, moe_layer_dispatch_row_bytes each, destination by
 *                   destination, each destination's in token order.
 *   experts_partial: R rows received (any order), `assignments` experts listed in them in all (0: unknown; an upper
 *                   bound will do); y_dev [R][n_embd] f16 receives the weighted sums, in the order received.
 *   combine_partials: back_dev holds the sums for the rows this GPU sent, in the order it sent them;
 *                   out[t] = the GPUs' sums for t + gate[t] * shared[t]. */
MOE_API uint32_t moe_layer_dispatch_row_bytes(const moe_layer *l);
MOE_API moe_status moe_layer_dispatch_plan_device(moe_layer *l, uint32_t *totals_dev, void *stream);
MOE_API moe_status moe_layer_dispatch_rows_device(moe_layer *l, void *rows_dev, void *stream);
MOE_API moe_status moe_layer_experts_partial_device(moe_layer *l, const void *rows_dev, uint32_t R, uint32_t assignments, void *y_dev,
                                                    void *stream);
MOE_API moe_status moe_layer_combine_partials_device(moe_layer *l, const void *back_dev, float *out_dev, void *stream);

/* Waits for the layer's stream. MOE_TIMEOUT after timeout_ms (0: 60 s), never an unbounded wait. */
MOE_API moe_status moe_layer_sync(moe_layer *l, uint32_t timeout_ms);

/* The last call's routing, copied to host buffers (any may be null): ids and w, T * n_used each, in rank order; inv,
 * the row each assignment t * n_used + k took in expert order; tiles, up to tiles_cap of them; *ntiles, how many
 * there are. Waits for the stream. */
MOE_API moe_status moe_layer_read_route(moe_layer *l, int32_t *ids, float *w, uint32_t *inv, moe_tile *tiles,
                                        uint32_t tiles_cap, uint32_t *ntiles);

/* The last call's groups for the integer-dot kernels (the reference's MoeGroup, shared/moe_tile.h:20-33, as a range:
 * its assignments are rows start .. start + n of the expert order, which lists an expert's assignments in ascending
 * order, so a group holds what core/tests/step_rows_test.cpp:40-58 puts in it; the list is in expert order, not in
 * order of first assignment). Up to cap of them; *ngroups, how many there are. Waits for the stream. */
typedef struct {
  uint32_t slot;
  uint32_t start;
  uint32_t n; /* 1 .. 8 */
} moe_group;
MOE_API moe_status moe_layer_read_groups(moe_layer *l, moe_group *groups, uint32_t cap, uint32_t *ngroups);

/* The last call's quantised activations, as the expert kernels read them (the a8 rows of kernels/include/a8.h:9-16;
 * here in the CPU path's own q8_0 / q8_K forms, docs/spec/QUANT_FORMATS.md:463-465,528-535). which 0: the step's rows
 * x, [T][n_embd]; which 1: the routed experts' inner rows h in expert order, [T * n_used][n_ff]. codes: one int8 a
 * value; scales: one float per 32 values (q8_0, the f16 scale widened) or per 256 (q8_K); sums: q8_K's int16 sums of
 * each 16 codes, untouched for q8_0. *is_q8k says which form. Any pointer may be null. Waits for the stream. */
MOE_API moe_status moe_layer_read_quantized(moe_layer *l, uint32_t which, int8_t *codes, float *scales, int16_t *sums,
                                            uint32_t *is_q8k);

/* The last call's router logits as its top-k read them, [T][n_experts]. Steps of more than 64 rows
 * take the router's product (the reference's kernels/gemm.cl:51-115 at prompt.cpp:608) on the tensor cores: then
 * *approximate is 1, and every logit is within eps_rel * |x_t| + eps_abs of the fp32 logit summed in the fixed order
 * (|x_t| the row's Euclidean norm); the top-k recomputes in that order whatever the bound leaves undecided, so the
 * expert ids are those of the fixed order all the same; these logits are without the router's bias. Else *approximate
 * is 0, the bounds are 0 and the logits are the fixed order's own, bias included. Any pointer may be null. Waits for the
 * stream. */
MOE_API moe_status moe_layer_read_logits(moe_layer *l, float *logits, uint32_t *approximate, float *eps_rel, float *eps_abs);

MOE_API moe_status moe_layer_read_stats(moe_layer *l, moe_layer_stats *out);
/* With MOE_FLAG_PROFILE: the last call's time in each stage, milliseconds, MOE_STAGES floats. Waits for the stream. */
MOE_API moe_status moe_layer_stage_ms(moe_layer *l, float *ms);
/* Turns the per-stage timing of MOE_FLAG_PROFILE on or off after create. While it is on, the stages run one after
 * another on one stream and small steps are not replayed from recorded graphs, so a call is slower than without. */
MOE_API moe_status moe_layer_set_profiling(moe_layer *l, uint32_t on);
/* The layer's cudaStream_t. */
MOE_API void *moe_layer_stream(moe_layer *l);

/* The last error's message, valid until the next call on l (or, for create's failures, with l null). */
MOE_API const char *moe_last_error(const moe_layer *l);

/* No counterpart in the reference. The router alone (logits, softmax, top n_used, renormalised weights, and the shared
 * expert's gate), for callers that must not allocate while a step runs: an engine that shared out all device memory at
 * load, or a step loop that cannot take the allocator's device-wide wait. It calls no cudaMalloc, cudaFree or
 * allocating library routine; the scratch between its two kernels is a fixed array inside the library (about 136 KB on
 * every GPU that loads it, held until the process ends), so T is at most MOE_ROUTE_STATIC_MAX_ROWS, n_experts at
 * most 512 and n_embd at most 4096; more is refused with MOE_BAD_ARGUMENT.
 *   x_dev [T][n_embd] f32; router_dev [n_experts + 1][n_embd] f32, the router's rows and then the shared expert's gate
 *   vector (zeros if there is none); bias_dev [n_experts] or null; out: ids_dev, w_dev [T][n_used] in rank order,
 *   gate_dev [T] = sigmoid(gate . x). All DEVICE pointers of the current device, the caller's (x_dev and router_dev
 *   16-byte aligned); queued on stream (a cudaStream_t; null: the default stream) without waiting.
 * The first call on a device looks up the array's device address and sets one kernel attribute: make that call before
 * any stream capture begins. All calls share the one array: two calls whose kernels may overlap on a GPU (different
 * streams, no ordering between them) race on it; order them. Nothing in it needs clearing between calls.
 * moe_route_rows_static_error: the calling thread's last message from it. */
#define MOE_ROUTE_STATIC_MAX_ROWS 64
MOE_API moe_status moe_route_rows_static(const float *x_dev, uint32_t T, uint32_t n_embd, const float *router_dev,
                                         const float *bias_dev, uint32_t n_experts, uint32_t n_used, int32_t *ids_dev,
                                         float *w_dev, float *gate_dev, void *stream);
MOE_API const char *moe_route_rows_static_error(void);

/* The layout the GPU holds a slice of nblocks blocks in: one run per field of the block, quants first, as the
 * reference's to_runs and from_runs make it (core/load/runs.cpp:12-41; shared/quant.h:172-176). Host only: a
 * permutation of the slice's bytes, src and dst nblocks * block bytes each. */
MOE_API moe_status moe_to_runs(uint32_t type, const void *file_blocks, uint64_t nblocks, void *dst);
MOE_API moe_status moe_from_runs(uint32_t type, const void *runs, uint64_t nblocks, void *dst);

/* For the ABI test, as engine_abi_layout (include/engine_api.h:414-421): one row per field, "struct.field" with its
 * offset and size, then one row per struct. Returns the number of rows; table may be null. */
typedef struct {
  const char *name;
  uint32_t offset;
  uint32_t size;
} moe_abi_row;
MOE_API uint32_t moe_abi_layout(moe_abi_row *table, uint32_t cap);

#ifdef __cplusplus
}
#endif
#endif
