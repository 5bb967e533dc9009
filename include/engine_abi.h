/* The whole-engine C ABI of avra-m3/c0ven (its include/engine_api.h, version 23), as this library implements it: the
 * same twenty engine_* symbols, the same plain structs field for field (engine_abi_layout reports every offset and
 * size, as the reference's does for tests/host/test_abi.py:31-45), the same status codes and ownership rules
 * (engine_api.h:1-10: no callbacks, only plain structs and buffers cross, every call returns a status, the library owns
 * all memory and threads). A caller built against the reference's header binds to this library unchanged.
 *
 * What stands behind it here is the MoE path only: a model whose layers are x <- x + moe_l(rmsnorm_l(x)), the
 * attention of each layer replaced by the identity, with tokens embedded from token_embd and the next token taken
 * greedily from output (or the tied embedding). One engine thread turns each engine_step_plan into ONE packed ragged
 * batch: the plan's prompt pieces and its decode rows concatenated, [rows][n_embd], with a run table beside it
 * (shared/step.h:99-104's PromptPlan {n, pos0, slot, row0}); the reference submits a device program per piece and one
 * for the step (core/api/engine_api.cpp:651-931). Calls whose subject the path does not have keep their signatures and
 * answer as the reference's header allows: see each below.
 *
 * Each declaration cites the line of the reference's header it mirrors. */
#ifndef ENGINE_ABI_H
#define ENGINE_ABI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(ENGINE_API_EXPORT)
#define ENGINE_API __attribute__((visibility("default")))
#else
#define ENGINE_API
#endif

#define ENGINE_API_VERSION 23 /* engine_api.h:26 */

typedef enum { /* engine_api.h:28-34 */
  ENGINE_OK = 0,
  ENGINE_ERROR = 1,
  ENGINE_BAD_ARGUMENT = 2,
  ENGINE_BUSY = 3,
  ENGINE_TIMEOUT = 4
} engine_status;

typedef struct engine_ctx engine_ctx;

/* engine_api.h:38-63. Zero means the default. Read here: model_path (a GGUF file with blk.N MoE tensors, see
 * INTEGRATION.md), slots (default 1), max_ctx (default 32768), max_cards (GPUs; default 1), prompt_chunk (rows a plan
 * may bring at most; default 4352), flags' ENGINE_CONFIG_PROMPT_SET. The other fields describe parts this model does
 * not have (an expert cache, CPU workers, drafting, images, a KV pool, an n-gram table) and are accepted and ignored. */
typedef struct {
  const char *model_path;
  uint32_t slots;
  uint32_t max_ctx;
  uint32_t max_cards;
  int32_t experts_per_layer;
  uint32_t cpu_threads;
  uint32_t flags;
  uint64_t reserve_bytes;
  uint32_t prompt_chunk;
  uint32_t checkpoints;
  const char *routing_profile;
  const char *mtp_dir;
  uint32_t draft_max;
  float draft_min_p;
  const char *vision_path;
  uint32_t kv_pages;
  uint32_t kv_resident_cells;
  uint64_t ngram_huge_bytes;
} engine_config;

/* engine_api.h:65-79 */
#define ENGINE_CONFIG_EXPERTS_SET 1u
#define ENGINE_CONFIG_PROMPT_SET 2u
#define ENGINE_CONFIG_SWAPS 4u
#define ENGINE_CONFIG_SHARE_KV 8u
#define ENGINE_CONFIG_NGRAM_RAM 16u
#define ENGINE_CONFIG_HUGETLB 32u

/* engine_api.h:82-126. Filled here: api_version, cards, slots, max_ctx, experts_per_layer (every expert is resident),
 * vocab, device_bytes, load_seconds, prompt_chunk, max_step_rows (the rows one packed batch may hold: prompt_chunk, far
 * above the reference's 16), kv_pages and pages_per_slot (the numbers a caller's page table needs to stay consistent;
 * no KV is kept). The rest are 0. */
typedef struct {
  uint32_t api_version;
  uint32_t cards;
  uint32_t slots;
  uint32_t max_ctx;
  uint32_t experts_per_layer;
  uint32_t vocab;
  uint64_t device_bytes[2];
  uint64_t arena_bytes;
  double load_seconds;
  uint32_t prompt_chunk;
  uint32_t checkpoints;
  uint32_t max_step_rows;
  uint32_t drafting;
  uint32_t image_tokens_max;
  uint32_t kv_pages;
  uint32_t pages_per_slot;
  double host_read_bytes_per_s;
  uint32_t loader_threads;
  uint32_t ngram_in_ram;
  double loader_bytes_per_s;
  double ngram_read_us;
  double copy_bytes_per_s[2];
  uint64_t expert_budget[2];
  uint32_t fetch_rows;
  uint32_t decode_weight;
  uint64_t ngram_cache_rows;
  uint64_t ngram_huge_bytes;
} engine_info;

/* engine_api.h:131-148. Copied by admit. Used here: max_tokens, n_stop and stop; tokens are chosen greedily whatever
 * the temperature (sampling is the control plane's concern, not this path's); min_p and the penalties are range-checked
 * as the reference does and otherwise unused. */
#define ENGINE_MAX_STOP 8
typedef struct {
  float temperature;
  uint32_t top_k;
  float top_p;
  uint32_t max_tokens;
  uint64_t seed;
  uint32_t n_stop;
  int32_t stop[ENGINE_MAX_STOP];
  float min_p;
  uint32_t penalty_last_n;
  float penalty_repeat;
  float penalty_freq;
  float penalty_present;
} engine_settings;

/* engine_api.h:157-165. The MoE path keeps no KV, so a page change moves no memory; the changes of a plan are checked
 * for the rules a caller's page table relies on (a known slot, a page below kv_pages or ENGINE_NO_PAGE, cells 0-3) and a
 * plan that breaks them is refused with ENGINE_BAD_ARGUMENT, as the reference refuses it. */
#define ENGINE_NO_PAGE 0xffffffffu
typedef struct {
  uint32_t slot;
  uint32_t logical;
  uint32_t page;
  uint32_t source;
  uint32_t cells;
} engine_page_change;

/* engine_api.h:178-199. One plan becomes one packed ragged batch: its prompt pieces in order (each the slot's next
 * `tokens` prompt tokens, 0: as many as remain, up to prompt_chunk in all), then one row per decode slot (the slot's
 * next prompt token while it still reads its prompt, else its last token). window_rows has no meaning here: every piece
 * rides in the same batch, whatever its length. */
#define ENGINE_MAX_STEP_SLOTS 8
#define ENGINE_MAX_PROMPT_PIECES 4
typedef struct {
  uint32_t slot;
  uint32_t tokens;
} engine_prompt_piece;

typedef struct {
  uint32_t nslots;
  uint32_t slots[ENGINE_MAX_STEP_SLOTS];
  uint32_t npieces;
  engine_prompt_piece pieces[ENGINE_MAX_PROMPT_PIECES];
  uint32_t npages;
  const engine_page_change *pages;
  uint32_t kv_free;
  uint32_t window_rows;
} engine_step_plan;

typedef enum { /* engine_api.h:201-208 */
  ENGINE_EVENT_TOKEN = 1,
  ENGINE_EVENT_PROMPT = 2,
  ENGINE_EVENT_DONE = 3,
  ENGINE_EVENT_STEP = 4,
  ENGINE_EVENT_ERROR = 5,
  ENGINE_EVENT_STALLED = 6
} engine_event_kind;

#define ENGINE_DONE_STOP 1 /* engine_api.h:210-212 */
#define ENGINE_DONE_LENGTH 2
#define ENGINE_DONE_CONTEXT 3

typedef struct { /* engine_api.h:214-219 */
  uint32_t kind;
  uint32_t slot;
  int32_t token;
  uint32_t value;
} engine_event;

typedef enum { /* engine_api.h:222-227 */
  ENGINE_TIMING_PROMPT = 1,
  ENGINE_TIMING_DECODE = 2,
  ENGINE_TIMING_ROUND = 3,
  ENGINE_TIMING_DRAFT = 4
} engine_timing_kind;

/* engine_api.h:229-236. One record per prompt piece and one for the decode rows of a plan, as the reference's callers
 * expect (engine/api/native.py derives its step-done from them); the records of one plan share the batch's start and
 * end, since its rows ran together. misses is 0: every expert is on the GPU. */
typedef struct {
  uint32_t kind;
  uint32_t plan;
  uint32_t rows;
  uint32_t misses;
  uint64_t start_ns;
  uint64_t end_ns;
} engine_timing;

/* engine_api.h:240-306: 62 counters, read by snapshot. Kept here: up_ns, plans, busy_ns, prompt_chunks, prompt_rows,
 * prompt_ns (the pieces of the packed batches), steps, step_rows, step_ns (their decode rows), experts_cached (all of
 * them). The rest stay 0. */
typedef struct {
  uint64_t up_ns, plans, busy_ns;
  uint64_t prompt_chunks, prompt_rows, prompt_ns;
  uint64_t window_pieces, window_rows, window_ns;
  uint64_t steps, step_rows, step_ns, step_misses, step_layers_missed, undrafted_steps;
  uint64_t rounds, round_rows, round_ns, round_misses, round_layers_missed;
  uint64_t layer_runs, layer_drafts, layer_accepted, layer_ns;
  uint64_t lookup_runs, lookup_drafts, lookup_accepted, lookup_ns;
  uint64_t swap_rounds, swaps, swap_ns;
  uint64_t stalls, checkpoints_taken, restores;
  uint64_t ngram_rows, ngram_hits, ngram_reads;
  uint64_t experts_cached, experts_floor, idle_rounds, reading_steps, reading_rounds;
  uint64_t draft_passes, draft_ns;
  uint64_t layer_drafts_1, layer_drafts_2, layer_drafts_3, layer_drafts_4, layer_drafts_5, layer_drafts_6, layer_drafts_7;
  uint64_t layer_accepted_1, layer_accepted_2, layer_accepted_3, layer_accepted_4, layer_accepted_5, layer_accepted_6, layer_accepted_7;
  uint64_t layer_stop_max, layer_stop_share, layer_stop_p, layer_stop_choice;
} engine_stats;

typedef struct { /* engine_api.h:309-317 */
  uint64_t steps, rounds, drafts, accepted, lookup_rounds, lookup_drafts, lookup_accepted;
} engine_slot_stats;

/* engine_api.h:320: loads the model's MoE tensors onto the GPU(s) and starts the engine thread. Blocks until ready. */
ENGINE_API engine_status engine_open(const engine_config *config, engine_info *info, engine_ctx **out);

/* engine_api.h:326-327: copies a request into a free slot. ENGINE_BUSY for a slot in use; ENGINE_BAD_ARGUMENT for a slot
 * out of range, no prompt, a token outside the vocabulary, min_p outside [0, 1], or a penalty with penalty_repeat <= 0. */
ENGINE_API engine_status engine_admit(engine_ctx *e, uint32_t slot, const engine_settings *settings, const int32_t *prompt,
                                      uint32_t n_prompt);

typedef struct { /* engine_api.h:333-338 */
  uint32_t first;
  uint32_t grid_h, grid_w;
  uint32_t frames;
  const uint8_t *pixels;
} engine_image;

/* engine_api.h:344: this model has no image encoder (image_tokens_max is 0): ENGINE_BAD_ARGUMENT for n > 0. */
ENGINE_API engine_status engine_admit_images(engine_ctx *e, uint32_t slot, const engine_image *images, uint32_t n);

ENGINE_API engine_status engine_release(engine_ctx *e, uint32_t slot);                 /* engine_api.h:347 */
ENGINE_API engine_status engine_submit(engine_ctx *e, const engine_step_plan *plan);   /* engine_api.h:351; BUSY when 64 plans wait */
ENGINE_API engine_status engine_poll(engine_ctx *e, engine_event *buf, uint32_t cap, uint32_t *n); /* engine_api.h:354 */
ENGINE_API engine_status engine_wait(engine_ctx *e, uint32_t timeout_ms);              /* engine_api.h:357 */

/* engine_api.h:362-373: the MoE path has no state that outlives a row (no KV, no recurrent state), so a checkpoint
 * holds only the slot's position and token history; config.checkpoints of them. ENGINE_BAD_ARGUMENT for an id past
 * them or a slot not admitted. Each waits for the plans queued before it. */
ENGINE_API engine_status engine_checkpoint(engine_ctx *e, uint32_t slot, uint32_t id);
ENGINE_API engine_status engine_restore(engine_ctx *e, uint32_t slot, uint32_t id);
ENGINE_API engine_status engine_drop(engine_ctx *e, uint32_t id);

ENGINE_API engine_status engine_read_timing(engine_ctx *e, engine_timing *buf, uint32_t cap, uint32_t *n); /* engine_api.h:376; a ring of 4,096 */
ENGINE_API engine_status engine_read_stats(engine_ctx *e, engine_stats *out);          /* engine_api.h:379 */
ENGINE_API engine_status engine_read_slot_stats(engine_ctx *e, uint32_t slot, engine_slot_stats *out); /* engine_api.h:382 */

/* engine_api.h:389-394: sleep frees the layers' device memory (ENGINE_BUSY while a slot is admitted); wake loads the
 * file again. While asleep admit, submit, checkpoint and restore fail with ENGINE_ERROR. */
ENGINE_API engine_status engine_sleep(engine_ctx *e);
ENGINE_API engine_status engine_wake(engine_ctx *e, engine_info *info);

ENGINE_API const char *engine_last_error(const engine_ctx *e); /* engine_api.h:397; e null: open's and cards' failures */
ENGINE_API void engine_close(engine_ctx *e);                   /* engine_api.h:401 */
/* engine_api.h:407: 1 once a wait on the GPU has run out in this process (a step that did not finish in 60 s), else 0. */
ENGINE_API int engine_queue_stuck(void);

/* engine_api.h:410-421: a GPU as the CUDA runtime reports it. device_id: PCI device id; ip_version: compute capability
 * major << 8 | minor; xe_cores: multiprocessors; the PCIe fields -1 (not reported by the runtime). */
typedef struct {
  char name[64];
  char pci[16];
  uint64_t memory;
  uint32_t device_id;
  uint32_t ip_version;
  uint32_t xe_cores;
  int32_t pcie_gen;
  int32_t pcie_width;
  uint32_t reserved;
  int64_t pcie_bytes_per_s;
} engine_card;

ENGINE_API engine_status engine_cards(engine_card *cards, uint32_t cap, uint32_t *n); /* engine_api.h:425 */

typedef struct { /* engine_api.h:429-433 */
  const char *name;
  uint32_t offset;
  uint32_t size;
} engine_abi_row;
ENGINE_API uint32_t engine_abi_layout(engine_abi_row *table, uint32_t cap); /* engine_api.h:434 */

/* This build's own, outside the reference's twenty: the hidden rows the last plan's batch ended with, [rows][n_embd]
 * f32 in batch order, and its run table, for tests that hold the stack to the oracle (the reference's events carry
 * tokens only). rows_cap in rows; *rows and *runs receive the counts. Waits for the plans queued before it. */
typedef struct {
  uint32_t n;    /* rows of the run */
  uint32_t pos0; /* position of its first row in the slot's sequence */
  uint32_t slot;
  uint32_t row0; /* its first row in the batch */
} engine_batch_run;
ENGINE_API engine_status engine_read_batch(engine_ctx *e, float *hidden, uint32_t rows_cap, uint32_t *rows, engine_batch_run *runs,
                                           uint32_t runs_cap, uint32_t *nruns);

#ifdef __cplusplus
}
#endif
#endif
