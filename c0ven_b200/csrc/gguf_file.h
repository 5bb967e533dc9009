// A GGUF version 3 file, read-only: its metadata and its table of tensors, whose bytes are mapped from the file. It
// stands where the reference has core/load/gguf.h:13-71 (GgufModel) and serves one purpose here: finding a layer's MoE
// tensors (blk.N.ffn_gate_inp, ffn_gate_inp_shexp, ffn_{gate,up,down}_exps, ffn_{gate,up,down}_shexp, ffn_norm) in
// the layout the file holds them in, which is the layout moe_layer_create takes. One file, not a set of shards.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace moe {

// ggml's numbers for the unquantised types a router or a norm may be stored in (shared/quant.h:10-33).
enum : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_BF16 = 30 };

struct GgufTensorInfo {
  std::string name;
  uint32_t type = 0;            // ggml type id
  std::vector<uint64_t> shape;  // ggml order: shape[0] is the contiguous axis
  uint64_t offset = 0;          // from the start of the file
  uint64_t bytes = 0;
  const uint8_t *data = nullptr;  // mapped

  uint64_t elements() const {
    uint64_t n = 1;
    for (uint64_t d : shape) n *= d;
    return n;
  }
};

class GgufFile {
 public:
  explicit GgufFile(const std::string &path);  // throws std::runtime_error with the reason
  ~GgufFile();
  GgufFile(const GgufFile &) = delete;
  GgufFile &operator=(const GgufFile &) = delete;

  const std::string &path() const { return path_; }
  const std::vector<GgufTensorInfo> &tensors() const { return tensors_; }
  const GgufTensorInfo *find(const std::string &name) const;
  const GgufTensorInfo &tensor(const std::string &name) const;  // throws when absent

  // Metadata: numbers of any integer type as int64, floats as double, strings; arrays are skipped over.
  bool has_int(const std::string &key) const { return ints_.count(key) != 0; }
  int64_t get_int(const std::string &key, int64_t otherwise) const;
  double get_float(const std::string &key, double otherwise) const;
  std::string get_string(const std::string &key, const std::string &otherwise = "") const;
  // "<general.architecture>.<suffix>", the form the per-model keys have (block_count, expert_used_count, ...).
  int64_t arch_int(const std::string &suffix, int64_t otherwise) const;

 private:
  std::string path_;
  int fd_ = -1;
  const uint8_t *base_ = nullptr;
  uint64_t size_ = 0;
  std::vector<GgufTensorInfo> tensors_;
  std::map<std::string, size_t> index_;
  std::map<std::string, int64_t> ints_;
  std::map<std::string, double> floats_;
  std::map<std::string, std::string> strings_;
};

// Bytes of a tensor of this type and element count; 0 for a type this library does not read.
uint64_t gguf_type_bytes(uint32_t type, uint64_t elements);

// n values of an F32, F16 or BF16 tensor as floats. Throws for another type.
std::vector<float> gguf_to_f32(const GgufTensorInfo &t);

}  // namespace moe
