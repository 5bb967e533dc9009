// The model behind the engine ABI: a stack of MoE layers, x <- x + moe_l(rmsnorm_l(x)), attention replaced by the
// identity, on one GPU. It stands where the reference has engine::Model (core/api/model.h:160-299) with its step() and
// prompt_runs(); here both are one call, batch(): a plan's rows, whatever they are, run as one packed ragged batch.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

struct moe_layer;
struct moe_gguf;

namespace moe {

// A run of the batch: n consecutive rows of one slot (shared/step.h:99-104, PromptPlan).
struct BatchRun {
  uint32_t n, pos0, slot, row0;
};

class EngineModel {
 public:
  // Reads the file's blk.N MoE tensors onto `device`. max_rows: the most rows a batch may hold. Throws on failure.
  EngineModel(const std::string &gguf_path, int device, uint32_t max_rows);
  ~EngineModel();
  EngineModel(const EngineModel &) = delete;
  EngineModel &operator=(const EngineModel &) = delete;

  uint32_t layers() const { return (uint32_t)layers_.size(); }
  uint32_t n_embd() const { return n_embd_; }
  uint32_t n_experts() const { return n_experts_; }
  uint32_t vocab() const { return vocab_; }
  uint32_t max_rows() const { return max_rows_; }
  uint64_t device_bytes() const { return device_bytes_; }

  // Runs the batch: tokens[rows] embedded, every layer applied, and for each row listed in want (ascending row
  // indices) the next token chosen greedily (ties to the lower id) into next[i]. Waits for the GPU, at most timeout_ms;
  // throws moe::Timeout when that runs out.
  void batch(const int32_t *tokens, uint32_t rows, const uint32_t *want, uint32_t nwant, int32_t *next, uint32_t timeout_ms);
  // The hidden rows the last batch ended with, [rows][n_embd].
  void read_hidden(float *dst, uint32_t rows) const;
  uint64_t kernels() const;  // launched by the layers since the model was made

 private:
  struct Buffers;
  int device_ = 0;
  uint32_t n_embd_ = 0, n_experts_ = 0, vocab_ = 0, max_rows_ = 0;
  float norm_eps_ = 1e-6f;
  uint64_t device_bytes_ = 0;
  moe_gguf *file_ = nullptr;
  std::vector<moe_layer *> layers_;
  std::unique_ptr<Buffers> buf_;
};

}  // namespace moe
