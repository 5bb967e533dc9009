// The C ABI over gguf_file.h: open a file, list its tensors, make a layer from a block's MoE tensors.
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "formats.h"
#include "gguf_file.h"
#include "internal.h"
#include "moe_layer.h"

using namespace moe;

struct moe_gguf {
  std::unique_ptr<GgufFile> file;
};

namespace {

std::string blk(uint32_t layer, const char *rest) { return "blk." + std::to_string(layer) + "." + rest; }

// An expert tensor [rows' values][rows][experts] of a block type this library decodes.
void need_experts(const GgufTensorInfo &t, uint64_t values, uint64_t rows, uint64_t experts) {
  if (!type_known(t.type)) throw std::runtime_error(t.name + " is of ggml type " + std::to_string(t.type) + ", which this library does not decode");
  if (t.shape.size() != 3 || t.shape[0] != values || t.shape[1] != rows || t.shape[2] != experts)
    throw std::runtime_error(t.name + " does not have the shape its layer's other tensors give it");
}

}  // namespace

extern "C" {

MOE_API moe_status moe_gguf_open(const char *path, moe_gguf **out) {
  if (!path || !out) {
    set_create_error("path and out are required");
    return MOE_BAD_ARGUMENT;
  }
  *out = nullptr;
  try {
    auto h = std::make_unique<moe_gguf>();
    h->file = std::make_unique<GgufFile>(path);
    *out = h.release();
    return MOE_OK;
  } catch (const std::exception &e) {
    set_create_error(e.what());
    return MOE_ERROR;
  }
}

MOE_API void moe_gguf_close(moe_gguf *f) { delete f; }

MOE_API uint32_t moe_gguf_layers(const moe_gguf *f) { return f ? (uint32_t)f->file->arch_int("block_count", 0) : 0; }

MOE_API uint32_t moe_gguf_tensors(const moe_gguf *f, moe_gguf_tensor *table, uint32_t cap) {
  if (!f) return 0;
  const auto &ts = f->file->tensors();
  for (uint32_t i = 0; table && i < cap && i < ts.size(); i++) {
    moe_gguf_tensor &r = table[i];
    std::memset(&r, 0, sizeof(r));
    r.name = ts[i].name.c_str();
    r.type = ts[i].type;
    r.n_dims = (uint32_t)ts[i].shape.size();
    for (uint32_t d = 0; d < r.n_dims && d < 4; d++) r.shape[d] = ts[i].shape[d];
    r.offset = ts[i].offset, r.bytes = ts[i].bytes;
  }
  return (uint32_t)ts.size();
}

MOE_API moe_status moe_layer_create_from_gguf(const moe_gguf *f, uint32_t layer, const moe_layer_config *config, moe_layer **out) {
  if (!f || !config || !out) {
    set_create_error("file, config and out are required");
    return MOE_BAD_ARGUMENT;
  }
  *out = nullptr;
  try {
    const GgufFile &g = *f->file;
    const GgufTensorInfo &router = g.tensor(blk(layer, "ffn_gate_inp.weight"));
    if (router.shape.size() != 2) throw std::runtime_error(router.name + " is not a matrix");
    const uint64_t E = router.shape[0], NE = router.shape[1];
    const GgufTensorInfo &gate = g.tensor(blk(layer, "ffn_gate_exps.weight")), &up = g.tensor(blk(layer, "ffn_up_exps.weight")),
                         &down = g.tensor(blk(layer, "ffn_down_exps.weight"));
    if (gate.shape.size() != 3) throw std::runtime_error(gate.name + " is not [values][rows][experts]");
    const uint64_t F = gate.shape[1];
    need_experts(gate, E, F, NE), need_experts(up, E, F, NE), need_experts(down, F, E, NE);
    if (up.type != gate.type) throw std::runtime_error("gate and up of layer " + std::to_string(layer) + " differ in type");
    moe_layer_config c = *config;
    c.n_embd = (uint32_t)E, c.n_ff = (uint32_t)F, c.n_experts = (uint32_t)NE;
    c.gate_type = gate.type, c.down_type = down.type;
    if (!c.n_used) c.n_used = (uint32_t)g.arch_int("expert_used_count", 0);
    if (!c.n_used) throw std::runtime_error("n_used is 0 and the file has no expert_used_count");
    const uint32_t first = c.expert_first, count = c.expert_count ? c.expert_count : (uint32_t)NE - first;
    if ((uint64_t)first + count > NE) throw std::runtime_error("expert_first + expert_count passes the file's experts");
    const std::vector<float> router_f32 = gguf_to_f32(router);
    std::vector<float> shgate_f32;
    moe_layer_weights w{};
    w.router = router_f32.data();
    const uint64_t gslice = F * row_bytes(gate.type, E), dslice = E * row_bytes(down.type, F);
    w.gate_exps = gate.data + first * gslice, w.up_exps = up.data + first * gslice, w.down_exps = down.data + first * dslice;
    const GgufTensorInfo *sgi = g.find(blk(layer, "ffn_gate_inp_shexp.weight"));
    c.shexp_gate_type = c.shexp_down_type = 0;
    if (sgi) {
      const GgufTensorInfo &sg = g.tensor(blk(layer, "ffn_gate_shexp.weight")), &su = g.tensor(blk(layer, "ffn_up_shexp.weight")),
                           &sd = g.tensor(blk(layer, "ffn_down_shexp.weight"));
      if (sgi->elements() != E || !sgi->data) throw std::runtime_error(sgi->name + " is not a vector of n_embd values");
      if (!type_known(sg.type) || !type_known(sd.type) || su.type != sg.type || sg.elements() != E * F || su.elements() != E * F ||
          sd.elements() != E * F)
        throw std::runtime_error("the shared expert of layer " + std::to_string(layer) + " is not three block-quantised matrices of the experts' shape");
      shgate_f32 = gguf_to_f32(*sgi);
      w.shexp_gate_inp = shgate_f32.data();
      w.gate_shexp = sg.data, w.up_shexp = su.data, w.down_shexp = sd.data;
      c.shexp_gate_type = sg.type, c.shexp_down_type = sd.type;
    }
    return moe_layer_create(&c, &w, out);
  } catch (const std::exception &e) {
    set_create_error(e.what());
    return MOE_ERROR;
  }
}

}  // extern "C"
