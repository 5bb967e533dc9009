/* CPU oracle of the MoE expert layer. TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU
 * baseline. Nothing in the product (the c0ven_b200 package, libc0ven_moe.so) links, loads or calls it.
 *
 * It restates, in plain C, the reference's CPU expert path and the routing its GPU kernels do:
 *   experts      core/cpu/experts.cpp:109-284 (compute, compute_many), SwiGLU :21-27
 *   IQ3_S dot    core/cpu/multirow.cpp:180-245
 *   formats      shared/quant.h:36-169, docs/spec/QUANT_FORMATS.md (Q4_K :373-399, Q6_K :419-445, Q8_0 :447-468,
 *                IQ3_S :178-213, q8_K :528-535)
 *   router       kernels/models/qwen4exp/layer.cl:765-804, route.h:39-98, kernels/include/topk.h:12-15,
 *                prompt.cl:652-678
 *   pack         kernels/models/qwen4exp/prompt.cl:682-738, made deterministic (stable by expert, then assignment)
 *   combine      layer.cl:869-883, prompt.cl:769-786
 *
 * PARITY UNPINNED for the exact bits of ggml's dot products: the reference's CPU path calls ggml (llama.cpp at
 * 3cf03257f219afbe7334045ff7c6a06ac68c627d), which is not in the reference tree, and the reference holds no golden
 * vectors for this path. What is pinned: block decoding against gguf-py's dequantize (tests/golden), the q8_0
 * quantiser against gguf-py's, the IQ3_S grid's sha256, and every dot against its own dequantisation in double. */
#ifndef MOE_ORACLE_H
#define MOE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, as shared/quant.h:10-33 numbers them. */
#define ORC_Q8_0 8
#define ORC_Q4_K 12
#define ORC_Q6_K 14
#define ORC_Q8_K 15
#define ORC_IQ4_NL 20
#define ORC_IQ3_XXS 18
#define ORC_IQ3_S 21
#define ORC_IQ2_S 22
#define ORC_IQ4_XS 23
#define ORC_Q2_0 42 /* the reference's fork of ggml: shared/quant.h:33 */

uint32_t orc_block_values(uint32_t type);
uint32_t orc_block_bytes(uint32_t type);
/* The activation format a weight type's dot takes: ORC_Q8_0 or ORC_Q8_K (docs/spec/MODEL_LAYER.md, section 6). */
uint32_t orc_vec_dot_type(uint32_t type);
uint64_t orc_row_bytes(uint32_t type, uint64_t n);

void orc_dequantize_row(uint32_t type, const void *blocks, float *y, int64_t n);
void orc_quantize_row(uint32_t act_type, const float *x, void *y, int64_t n);
float orc_vec_dot(uint32_t type, int64_t n, const void *w, const void *a);

/* The runs layout (core/load/runs.cpp:12-41; shared/quant.h:172-176): field f of block k at
 * run_offset(f, n) + k * field_size(f). */
void orc_to_runs(uint32_t type, const uint8_t *file_blocks, uint64_t nblocks, uint8_t *dst);
void orc_from_runs(uint32_t type, const uint8_t *runs, uint64_t nblocks, uint8_t *dst);

/* rl[t][0..NE) = W[e] . x[t], rl[t][NE] = wsg . x[t]; stride NE + 1. Each product is summed in 8 equal pieces of the
 * row, every piece a chain of fused multiply-adds from 0 in index order, the pieces then added in order: the order
 * the CUDA kernels use, so that near-ties between logits fall the same way on both sides. bias (NE values, or null) is
 * added to an expert's logit last: the synthetic configurations' skew, which the reference's files do not have. */
void orc_router_logits(const float *x, uint32_t T, uint32_t E, const float *W, const float *wsg, const float *bias,
                       uint32_t NE, float *rl);
/* Top-K of NE per row in rank order (largest first, ties to the lower expert, -0 as +0), weights renormalised;
 * gs[t] = sigmoid(rl[t][NE]). */
void orc_router_topk(const float *rl, uint32_t T, uint32_t NE, uint32_t K, int32_t *ids, float *w, float *gs);

typedef struct {
  uint32_t expert, slot, start, count;
} orc_tile; /* shared/moe_tile.h:11-16 */

/* Stable counting sort of the assignments a = t * K + k by expert: cnt, base (NE each), inv[a] = row of a in expert
 * order, tiles of at most 64 rows in expert order. first_expert is subtracted from an expert's id to give its slot.
 * Returns the number of tiles. */
uint32_t orc_pack(const int32_t *ids, uint32_t A, uint32_t NE, uint32_t first_expert, uint32_t *cnt, uint32_t *base,
                  uint32_t *inv, orc_tile *tiles);

typedef struct {
  uint32_t gate_type, down_type;
  uint32_t n_embd, n_ff;
  float swiglu_limit;
} orc_shape; /* core/cpu/experts.h:23-30 */

typedef struct {
  const uint8_t *gate, *up, *down; /* file layout */
  uint32_t tok;
  float w;
} orc_job; /* core/cpu/experts.h:41-47 */

/* core/cpu/experts.cpp:152-284. y[tok] = sum over the token's jobs, in the order given, of w * down(swiglu(gate x,
 * up x)). threads 0: every core the process may run on. */
void orc_compute_many(const orc_shape *s, const orc_job *jobs, uint32_t n, uint32_t ntok, const float *x,
                      uint64_t x_stride, float *y, uint64_t y_stride, int threads);

typedef struct {
  uint32_t n_embd, n_ff, n_experts, n_used;
  uint32_t gate_type, down_type, shexp_gate_type, shexp_down_type;
  float swiglu_limit;
  const float *router;         /* [n_experts][n_embd] */
  const float *shexp_gate_inp; /* [n_embd] */
  const float *router_bias;    /* [n_experts] or null */
  const uint8_t *gate_exps, *up_exps, *down_exps; /* n_experts slices each, file layout */
  const uint8_t *gate_shexp, *up_shexp, *down_shexp;
} orc_layer;

/* The whole layer on T rows. Any of ids, w (T * K), inv (T * K), tiles (T * K / 64 + NE), ntiles may be null. */
void orc_moe_forward(const orc_layer *L, const float *x, uint32_t T, float *out, int32_t *ids, float *w,
                     uint32_t *inv, orc_tile *tiles, uint32_t *ntiles, int threads);

int orc_threads(void);
void orc_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
