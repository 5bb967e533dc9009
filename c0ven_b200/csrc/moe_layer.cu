// The C ABI of include/moe_layer.h over the kernels of this directory: one layer's weights in the runs layout, the
// buffers a call needs, and the order of a call's stages. It does, for one GPU that holds every expert, what the
// reference's Model::step and Model::prompt_runs record for a layer's MoE block
// (core/models/qwen4exp/model.cpp:1348-1418, prompt.cpp:606-656) with its CPU path's arithmetic
// (core/cpu/experts.cpp:152-284).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "cuda_rt.h"
#include "expert_rows.cuh"
#include "expert_tiles.cuh"
#include "formats.h"
#include "internal.h"
#include "iq3s_grid.h"
#include "moe_layer.h"
#include "route_kernels.cuh"
#include "router_mma.cuh"
#include "tensor_map.h"

namespace moe {

template <int QT, int NMAT>
cudaError_t launch_expert_rows(const ExpertRowsArgs &a, int M, uint32_t max_groups, const uint32_t *grid_global, const LaunchCtx &ctx, cudaStream_t st);

static cudaError_t launch_rows(uint32_t qt, int nmat, const ExpertRowsArgs &a, int M, uint32_t max_groups, const uint32_t *grid,
                               const LaunchCtx &ctx, cudaStream_t st) {
#define ROWS_CASE(T)                                                                                            \
  case T:                                                                                                       \
    return nmat == 2 ? launch_expert_rows<T, 2>(a, M, max_groups, grid, ctx, st) : launch_expert_rows<T, 1>(a, M, max_groups, grid, ctx, st);
  switch (qt) {
    ROWS_CASE(QT_Q8_0)
    ROWS_CASE(QT_Q4_K)
    ROWS_CASE(QT_Q6_K)
    ROWS_CASE(QT_IQ3_S)
    ROWS_CASE(QT_IQ4_NL)
    ROWS_CASE(QT_IQ4_XS)
    ROWS_CASE(QT_IQ3_XXS)
    ROWS_CASE(QT_IQ2_S)
    ROWS_CASE(QT_Q2_0)
    default: return cudaErrorInvalidValue;
  }
#undef ROWS_CASE
}

static cudaError_t launch_tiles(uint32_t qt, int nmat, const ExpertTilesArgs &a, const CUtensorMap &map, uint32_t max_tiles, const uint32_t *grid,
                                const LaunchCtx &ctx, cudaStream_t st) {
#define TILES_CASE(T)                                                                                  \
  case T:                                                                                              \
    return nmat == 2 ? launch_expert_tiles<T, 2>(a, map, max_tiles, grid, ctx, st) : launch_expert_tiles<T, 1>(a, map, max_tiles, grid, ctx, st);
  switch (qt) {
    TILES_CASE(QT_Q8_0)
    TILES_CASE(QT_Q4_K)
    TILES_CASE(QT_Q6_K)
    TILES_CASE(QT_IQ3_S)
    TILES_CASE(QT_IQ4_NL)
    TILES_CASE(QT_IQ4_XS)
    TILES_CASE(QT_IQ3_XXS)
    TILES_CASE(QT_IQ2_S)
    TILES_CASE(QT_Q2_0)
    default: return cudaErrorInvalidValue;
  }
#undef TILES_CASE
}

// Quantised activation rows on the device, in the format a weight type's dot takes.
struct ActBuffers {
  DeviceBuffer<int8_t> q;
  DeviceBuffer<float> d;
  DeviceBuffer<int16_t> bs;
  DeviceBuffer<__half> h;  // the codes dequantised, f16: the tensor-core kernels' operand
  CUtensorMap h_map{};     // over h, for the tile kernels' copies
  CUtensorMap h_row_map{}; // over h with a box of one row: for copies that gather rows by index
  bool q8k = false;
  uint32_t K = 0;
  void alloc(uint64_t rows, uint32_t Kv, bool k, bool with_f16) {
    q8k = k, K = Kv;
    q.alloc(rows * K);
    d.alloc(rows * (k ? K / 256 : K / 32));
    if (k) bs.alloc(rows * (K / 16));
    if (with_f16) {
      const uint64_t hr = std::max<uint64_t>(rows, kMapBoxRows);  // a map's tensor is at least one box high
      h.alloc(hr * K);
      h_map = make_rows_map(h.get(), hr, K);
      h_row_map = make_rows_map(h.get(), hr, K, 1);
    }
  }
  ActView view(uint64_t row0 = 0) const {
    const uint32_t dn = q8k ? K / 256 : K / 32;
    return ActView{q.get() + row0 * K, d.get() + row0 * dn, q8k ? bs.get() + row0 * (K / 16) : nullptr, K, dn * 4, K / 8};
  }
};

// Where a call's expert kernels read their activation rows: int8 rows for the integer-dot kernels, f16 rows for the
// tensor-core kernels, and the map from an expert-order row to its activation row (null: the same row).
struct ActSource {
  ActView view;
  const __half *h;
  const uint32_t *act_row;
};

// One pack: `rows` assignments sorted by expert over `nexp` experts.
struct PackBuffers {
  DeviceBuffer<uint32_t> chunk_hist, chunk_off, group_off, cnt, base, counters, inv, row_src;
  DeviceBuffer<MoeTile> tiles;
  DeviceBuffer<MoeGroup> groups;
  DeviceBuffer<BigTile> big;
  uint32_t nexp = 0;
  void alloc(uint64_t max_rows, uint32_t n, uint32_t chunk_len) {
    nexp = n;
    const uint64_t nchunks = (max_rows + chunk_len - 1) / chunk_len + 1;
    chunk_hist.alloc(nchunks * n), chunk_off.alloc(nchunks * n), group_off.alloc((nchunks / kScanGroup + 1) * n);
    cnt.alloc(n), base.alloc(n), counters.alloc(8), inv.alloc(max_rows), row_src.alloc(max_rows);
    tiles.alloc(max_rows / kTileRows + n), big.alloc(max_rows / kTileN + n);
    // As long as any grid over it: the integer-dot kernel reads its entry before it knows the list's length.
    groups.alloc(max_rows + n);
  }
  PackOut out() const { return PackOut{cnt.get(), base.get(), chunk_off.get(), tiles.get(), groups.get(), big.get(), counters.get()}; }
};

enum Stage { ST_QUANT, ST_ROUTER, ST_PACK, ST_GATE_UP, ST_DOWN, ST_SHARED, ST_COMBINE, ST_COPIES };

constexpr uint32_t kRouterExactRows = 64;  // steps of up to this many rows take the exact fp32 router product
constexpr uint32_t kLocalChunk = 512;  // entries per chunk when packing rows that came from other GPUs

}  // namespace moe

using namespace moe;

struct moe_layer {
  moe_layer_config cfg{};
  uint32_t E = 0, F = 0, NE = 0, K = 0, N = 0, local = 0, Tmax = 0;
  uint64_t Rmax = 0;  // expert rows a call may bring: max_tokens * n_used, or max_expert_rows
  bool has_shared = false, profile = false, can_tensor = false;
  uint32_t sms = 148;  // the device's SM count
  LaunchCtx ctx;
  std::unique_ptr<Stream> stream, aux;  // aux: the shared expert runs beside the routed ones
  std::unique_ptr<Event> fork_ev, join_ev;
  // Host-buffer calls cut into chunks: the copies in and out on streams of their own, an event per chunk and direction.
  std::unique_ptr<Stream> copy_in, copy_out;
  std::vector<std::unique_ptr<Event>> in_done, comp_done;
  // Steps of few rows are bound by launches, not work: the whole call is recorded once per (rows, buffers, stream)
  // as a CUDA graph and replayed (the reference records its per-width step lists once too: core/ze/ze.h:155-189).
  struct StepGraph {
    uint32_t T;
    const float *x, *res;
    float *out;
    cudaStream_t st;
    cudaGraphExec_t exec;
    uint64_t kernels;
    uint32_t seen;
  };
  std::vector<StepGraph> graphs;
  bool graphs_ok = true;
  // Weights.
  DeviceBuffer<float> router, bias;
  DeviceBuffer<uint8_t> wg, wu, wd, sg, su, sd;
  DeviceBuffer<uint32_t> grid;
  uint64_t gate_slice = 0, down_slice = 0;
  // Maps over the quants runs, for the matrices whose type's quants reach the tile kernels by copy (tensor_map.h).
  CUtensorMap wg_q{}, wu_q{}, wd_q{}, sg_q{}, su_q{}, sd_q{};
  // A call's buffers.
  DeviceBuffer<float> x, out, rl, gate_parts, w, gs, h, y, s;
  // The router's product on the tensor cores (steps of more than 64 rows): the router's rows and the step's rows as
  // pairs of f16 numbers, the approximate logits, and what bounds their error.
  bool router_tensor = false, router_attr_set = false;
  DeviceBuffer<__half> rw_hi, rw_lo, rx_hi, rx_lo;
  DeviceBuffer<float> rw_unscale, approx, norm2_parts;
  CUtensorMap rw_hi_map{}, rw_lo_map{}, rx_hi_map{}, rx_lo_map{};
  float router_eps_rel = 0.0f, router_eps_abs = 0.0f;
  DeviceBuffer<int32_t> ids, ids_local;
  DeviceBuffer<uint32_t> error;
  DeviceBuffer<__half> xg;      // the routed experts' activation rows in expert order, f16: what their tile kernel copies from
  CUtensorMap xg_map{};

  PackBuffers pack, pack_local;  // the step's own rows over every expert; the rows received, over this GPU's experts
  // Expert parallel with one row per (token, GPU): where each token's row goes, and the received rows' lists.
  DeviceBuffer<uint32_t> dest_pos, dest_chunk_cnt, dest_chunk_asg, dest_totals;
  DeviceBuffer<float> w_local;
  uint32_t dest_world = 0;
  ActBuffers xq_routed, xq_shared, hq_routed, hq_shared;
  bool shared_x_same = true, rows_attr_set = false, shared_on_tensor = false;
  bool pdl_ok = true;  // off when C0VEN_NO_PDL is set in the environment at create
  uint32_t last_T = 0, last_tensor_min = 0;
  const float *residual = nullptr;  // of the call being queued: rows the combine adds last (moe_layer_forward_residual_device)
  PackBuffers *last_pack = nullptr;
  // Profiling: one event before each stage and one after the last.
  std::vector<std::unique_ptr<Event>> ev;
  bool ev_valid = false;
  moe_layer_stats stats{};
  std::string err;
  std::mutex mu;
};

static thread_local std::string g_create_error;

namespace moe {
void set_create_error(const std::string &message) { g_create_error = message; }
}  // namespace moe

namespace {

void launched(moe_layer *l, cudaError_t e, const char *what) {
  cuda_check(e, what, __FILE__, __LINE__);
  l->stats.kernels++;
}

// From the chunks' counts (pk.chunk_hist) to the pack: the scan over chunks and experts, then every chunk's rows handed
// out. Steps of more than two groups of chunks take the scan in two levels.
struct PackJob {
  const int32_t *ids;
  uint32_t entries, chunk_len, nchunks, first_expert, tensor_min, tensor_budget, group_max, src_div;
};
void launch_pack(moe_layer *l, PackBuffers &pk, const PackJob &j, cudaStream_t st) {
  const uint32_t ngroups = (j.nchunks + kScanGroup - 1) / kScanGroup;
  uint32_t *groups = ngroups > 2 ? pk.group_off.get() : nullptr;
  if (groups) {
    k_pack_scan_groups<<<ngroups, 512, 0, st>>>(pk.chunk_hist.get(), j.nchunks, pk.nexp, pk.chunk_off.get(), groups);
    launched(l, cudaGetLastError(), "pack scan of the groups");
  }
  k_pack_scan<<<1, 512, 0, st>>>(pk.chunk_hist.get(), j.nchunks, pk.nexp, j.first_expert, j.tensor_min, j.tensor_budget, j.group_max, pk.out(), groups,
                                 ngroups);
  launched(l, cudaGetLastError(), "pack scan");
  if (j.chunk_len > 512 || pk.nexp > 512) throw std::logic_error("pack fill: a chunk of at most 512 entries, at most 512 experts");
  k_pack_fill<<<j.nchunks, 512, 16 * pk.nexp * sizeof(uint32_t), st>>>(j.ids, j.entries, j.chunk_len, pk.nexp, pk.base.get(), pk.chunk_off.get(), j.src_div,
                                                                 pk.inv.get(), pk.row_src.get(), j.first_expert, groups);
  launched(l, cudaGetLastError(), "pack fill");
}

void mark(moe_layer *l, int stage, cudaStream_t st) {
  if (l->profile) l->ev[stage]->record(st);
}

void upload_matrix(DeviceBuffer<uint8_t> &dst, uint32_t type, const void *src, uint64_t nblk, uint64_t nslices, cudaStream_t st) {
  const uint64_t bytes = nblk * nslices * block_bytes(type);
  std::vector<uint8_t> runs(bytes);
  to_runs_slices(type, (const uint8_t *)src, nblk, nslices, runs.data(), std::max(1u, std::thread::hardware_concurrency()));
  dst.alloc(bytes + 16);  // room for a 16-byte load that starts inside the last run
  CUDA_OK(cudaMemcpyAsync(dst.get(), runs.data(), bytes, cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaStreamSynchronize(st));
}

void check_config(const moe_layer_config &c, const moe_layer_weights &w) {
  auto bad = [](const std::string &m) { throw BadArgument(m); };
  if (c.n_embd == 0 || c.n_embd % 256 || c.n_embd > kRowsMaxK) bad("n_embd must be a multiple of 256, at most 16384");
  if (c.n_ff == 0 || c.n_ff % 256 || c.n_ff > kRowsMaxK) bad("n_ff must be a multiple of 256, at most 16384");
  if (c.n_experts == 0 || c.n_experts % 32 || c.n_experts > 512) bad("n_experts must be a multiple of 32, at most 512");
  if (c.n_used == 0 || c.n_used > 16 || c.n_used > c.n_experts) bad("n_used must be 1 .. 16 and at most n_experts");
  if (!type_known(c.gate_type) || !type_known(c.down_type)) bad("the experts' types must be Q8_0, Q4_K, Q6_K, IQ3_S, IQ4_NL, IQ4_XS, IQ3_XXS, IQ2_S or Q2_0");
  if (c.shexp_gate_type && (!type_known(c.shexp_gate_type) || !type_known(c.shexp_down_type)))
    bad("the shared expert's types must be Q8_0, Q4_K, Q6_K or IQ3_S");
  if (c.expert_first + (c.expert_count ? c.expert_count : c.n_experts - c.expert_first) > c.n_experts)
    bad("expert_first + expert_count passes n_experts");
  if (!w.router || !w.gate_exps || !w.up_exps || !w.down_exps) bad("router and the experts' three tensors are required");
  if (c.shexp_gate_type && (!w.shexp_gate_inp || !w.gate_shexp || !w.up_shexp || !w.down_shexp))
    bad("a shared expert needs its gate vector and three matrices");
}

void setup_router_tensor(moe_layer *l, const float *router, const float *bias, cudaStream_t st);

void create(moe_layer *l, const moe_layer_config &c, const moe_layer_weights &w) {
  check_config(c, w);
  int ndev = 0;
  CUDA_OK(cudaGetDeviceCount(&ndev));
  if (c.device < 0 || c.device >= ndev) throw BadArgument("no CUDA device " + std::to_string(c.device));
  CUDA_OK(cudaSetDevice(c.device));
  l->cfg = c;
  l->E = c.n_embd, l->F = c.n_ff, l->NE = c.n_experts, l->K = c.n_used, l->N = c.n_experts + 1;
  l->local = c.expert_count ? c.expert_count : c.n_experts - c.expert_first;
  l->Tmax = c.max_tokens ? c.max_tokens : 4352;
  l->has_shared = c.shexp_gate_type != 0;
  l->profile = c.flags & MOE_FLAG_PROFILE;
  {
    int n = 0;
    CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, c.device));
    l->sms = n > 0 ? (uint32_t)n : 148;
    l->ctx = LaunchCtx{c.device, l->sms};
  }
  l->can_tensor = !(c.flags & MOE_FLAG_NO_TENSOR) && c.n_embd % kTileK == 0 && c.n_ff % kTileM == 0;
  l->stream = std::make_unique<Stream>();
  l->aux = std::make_unique<Stream>();
  l->fork_ev = std::make_unique<Event>(), l->join_ev = std::make_unique<Event>();
  l->pdl_ok = std::getenv("C0VEN_NO_PDL") == nullptr;
  cudaStream_t st = l->stream->get();
  const uint32_t E = l->E, F = l->F, NE = l->NE, K = l->K, T = l->Tmax;
  const uint64_t A = (uint64_t)T * K;
  const bool ep = l->local != NE;
  l->Rmax = c.max_expert_rows ? c.max_expert_rows : A;
  if (l->Rmax < A && !ep) l->Rmax = A;
  const uint64_t R = l->Rmax;
  {
    // The integer-dot kernels take one group per index of their grid's second extent, 65,535 at most: a layer whose
    // largest call could list more groups than that is refused here, not in the middle of a step.
    const uint32_t tm = !l->can_tensor ? 0 : c.tensor_min_rows ? c.tensor_min_rows : 16;
    const uint64_t routed = tm ? std::min<uint64_t>(R, (uint64_t)l->local * ((tm > 1 ? tm - 2 : 0) / kGroupMax + 1)) : std::min<uint64_t>(R, R / kGroupMax + l->local);
    const uint64_t dense = l->has_shared && (!l->can_tensor || tm > T) ? ((uint64_t)T + 7) / 8 : 0;
    if (routed > 65535 || dense > 65535)
      throw BadArgument("max_tokens (or max_expert_rows) is too large for the integer-dot kernels' grid: lower it, or leave the tensor-core kernels on");
  }

  // The router's rows, then the shared expert's gate vector as row NE (zeros without one).
  std::vector<float> rw((size_t)l->N * E, 0.0f);
  std::memcpy(rw.data(), w.router, (size_t)NE * E * sizeof(float));
  if (l->has_shared) std::memcpy(rw.data() + (size_t)NE * E, w.shexp_gate_inp, E * sizeof(float));
  l->router.alloc(rw.size());
  CUDA_OK(cudaMemcpyAsync(l->router.get(), rw.data(), rw.size() * sizeof(float), cudaMemcpyHostToDevice, st));
  if (w.router_bias) {
    l->bias.alloc(NE);
    CUDA_OK(cudaMemcpyAsync(l->bias.get(), w.router_bias, NE * sizeof(float), cudaMemcpyHostToDevice, st));
  }
  // The codebooks, one after another (formats.h: grid_offset).
  l->grid.alloc(kGridWordsAll);
  static_assert(sizeof(kIq3sGrid) == 4 * grid_words(QT_IQ3_S) && sizeof(kIq3xxsGrid) == 4 * grid_words(QT_IQ3_XXS) && sizeof(kIq2sGrid) == 4 * grid_words(QT_IQ2_S),
                "the generated tables' sizes");
  CUDA_OK(cudaMemcpyAsync(l->grid.get() + grid_offset(QT_IQ3_S), kIq3sGrid, sizeof(kIq3sGrid), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(l->grid.get() + grid_offset(QT_IQ3_XXS), kIq3xxsGrid, sizeof(kIq3xxsGrid), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(l->grid.get() + grid_offset(QT_IQ2_S), kIq2sGrid, sizeof(kIq2sGrid), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaStreamSynchronize(st));

  const uint64_t gblk = (uint64_t)F * (E / block_values(c.gate_type)), dblk = (uint64_t)E * (F / block_values(c.down_type));
  l->gate_slice = gblk * block_bytes(c.gate_type), l->down_slice = dblk * block_bytes(c.down_type);
  upload_matrix(l->wg, c.gate_type, w.gate_exps, gblk, l->local, st);
  upload_matrix(l->wu, c.gate_type, w.up_exps, gblk, l->local, st);
  upload_matrix(l->wd, c.down_type, w.down_exps, dblk, l->local, st);
  if (l->has_shared) {
    upload_matrix(l->sg, c.shexp_gate_type, w.gate_shexp, (uint64_t)F * (E / block_values(c.shexp_gate_type)), 1, st);
    upload_matrix(l->su, c.shexp_gate_type, w.up_shexp, (uint64_t)F * (E / block_values(c.shexp_gate_type)), 1, st);
    upload_matrix(l->sd, c.shexp_down_type, w.down_shexp, (uint64_t)E * (F / block_values(c.shexp_down_type)), 1, st);
  }

  if (l->can_tensor) {
    // A quant slot's row is 32 bytes a decode group: 2 groups for gate and up (two matrices a stage), 4 for down.
    if (quants_by_copy(c.gate_type)) {
      l->wg_q = make_quants_map(l->wg.get(), E / 2, F, l->local, l->gate_slice, 64);
      l->wu_q = make_quants_map(l->wu.get(), E / 2, F, l->local, l->gate_slice, 64);
    }
    if (quants_by_copy(c.down_type)) l->wd_q = make_quants_map(l->wd.get(), F / 2, E, l->local, l->down_slice, 128);
    if (l->has_shared && quants_by_copy(c.shexp_gate_type)) {
      l->sg_q = make_quants_map(l->sg.get(), E / 2, F, 1, l->sg.bytes(), 64);
      l->su_q = make_quants_map(l->su.get(), E / 2, F, 1, l->su.bytes(), 64);
    }
    if (l->has_shared && quants_by_copy(c.shexp_down_type)) l->sd_q = make_quants_map(l->sd.get(), F / 2, E, 1, l->sd.bytes(), 128);
  }
  l->x.alloc((size_t)T * E), l->out.alloc((size_t)T * E);
  l->router_tensor = l->can_tensor && T > kRouterExactRows;
  l->rl.alloc((size_t)(l->router_tensor ? kRouterExactRows : T) * l->N), l->gate_parts.alloc((size_t)T * (E / 256));
  if (l->router_tensor) setup_router_tensor(l, w.router, w.router_bias, st);
  l->ids.alloc(A), l->w.alloc(A), l->gs.alloc(T), l->error.alloc(1);
  l->pack.alloc(A, NE, kChunkTokens * K);
  if (ep) {
    l->pack_local.alloc(R, l->local, kLocalChunk);
    l->ids_local.alloc(R);
  }
  l->h.alloc((R + T) * F), l->y.alloc(R * E);
  if (l->can_tensor) {
    const uint64_t rows = std::max<uint64_t>(R, kMapBoxRows);
    l->xg.alloc(rows * E);
    l->xg_map = make_rows_map(l->xg.get(), rows, E);
  }
  l->xq_routed.alloc(T, E, act_is_q8k(c.gate_type), l->can_tensor);
  l->hq_routed.alloc(R, F, act_is_q8k(c.down_type), l->can_tensor);
  if (l->has_shared) {
    l->s.alloc((size_t)T * E);
    l->shared_x_same = act_is_q8k(c.shexp_gate_type) == act_is_q8k(c.gate_type);
    if (!l->shared_x_same) l->xq_shared.alloc(T, E, act_is_q8k(c.shexp_gate_type), l->can_tensor);
    l->hq_shared.alloc(T, F, act_is_q8k(c.shexp_down_type), l->can_tensor);
  }
  CUDA_OK(cudaMemsetAsync(l->pack.counters.get(), 0, 8 * sizeof(uint32_t), st));
  CUDA_OK(cudaMemsetAsync(l->error.get(), 0, sizeof(uint32_t), st));
  for (int i = 0; i <= MOE_STAGES; i++) l->ev.push_back(std::make_unique<Event>());
  CUDA_OK(cudaStreamSynchronize(st));
}

// The tensor-core router product's operands and error bound. Each of the router's rows is scaled by the power of two
// that puts its largest magnitude in [1024, 2048), then split into f16 hi and lo parts (lo = f16(w - hi)): both parts
// are then normal f16 numbers for every weight within 2^-13 of the row's largest, and hi + lo holds 22 bits of w.
//
// The bound. An approximate logit differs from the fp32 sum in the exact order by (a) the dropped lo * lo products and
// the rounding of the lo parts, at most 2^-20 of sum |x_i w_i|; (b) the roundings of the accumulations, each taken as
// at most 2^-23 of the running sum, one per MMA of 16 values and three MMAs a step: 3 E / 16 of them; (c) the exact
// order's own roundings: chains of E / 8 fused multiply-adds at 2^-24 of the running sum each, then eight additions.
// sum |x_i w_i| <= |x| |w_e| (Cauchy-Schwarz), so eps = eps_rel |x| max_e |w_e| with eps_rel = (3 E / 16 + E / 8 + 16) 2^-23
// (2^-13.6 at E = 2048) covers all three in the worst case, where every rounding falls the same way; measured errors
// are some hundred times smaller, and the GPU tests hold them under a quarter of the bound. The bias adds one rounding
// of the biased logit, covered by eps_abs.
void setup_router_tensor(moe_layer *l, const float *router, const float *bias, cudaStream_t st) {
  const uint32_t E = l->E, NE = l->NE, T = l->Tmax;
  const uint64_t wrows = std::max<uint32_t>(NE, kRouterTileExperts), xrows = std::max<uint32_t>(T, kRouterTileRows);
  std::vector<__half> hi(wrows * E, __float2half_rn(0.0f)), lo(wrows * E, __float2half_rn(0.0f));
  std::vector<float> unscale(NE, 1.0f);
  double wn_max = 0.0;
  for (uint32_t e = 0; e < NE; e++) {
    const float *w = router + (size_t)e * E;
    float m = 0.0f;
    double n2 = 0.0;
    for (uint32_t i = 0; i < E; i++) m = std::max(m, std::fabs(w[i])), n2 += (double)w[i] * w[i];
    wn_max = std::max(wn_max, std::sqrt(n2));
    int ex = 0;
    if (m > 0.0f && std::isfinite(m)) std::frexp(m, &ex);
    ex = std::min(std::max(ex, -100), 100);
    const float s = std::ldexp(1.0f, 11 - ex);
    unscale[e] = std::ldexp(1.0f, ex - 11);
    for (uint32_t i = 0; i < E; i++) {
      const float v = w[i] * s;
      const __half h = __float2half_rn(v);
      hi[(size_t)e * E + i] = h;
      lo[(size_t)e * E + i] = __float2half_rn(v - __half2float(h));
    }
  }
  float bias_max = 0.0f;
  for (uint32_t e = 0; bias && e < NE; e++) bias_max = std::max(bias_max, std::fabs(bias[e]));
  l->router_eps_rel = (float)(std::ldexp(3.0 * E / 16 + E / 8 + 16, -23) * wn_max);
  l->router_eps_abs = std::ldexp(1.0f + bias_max, -20);
  l->rw_hi.alloc(hi.size()), l->rw_lo.alloc(lo.size()), l->rw_unscale.alloc(NE);
  CUDA_OK(cudaMemcpyAsync(l->rw_hi.get(), hi.data(), hi.size() * sizeof(__half), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(l->rw_lo.get(), lo.data(), lo.size() * sizeof(__half), cudaMemcpyHostToDevice, st));
  CUDA_OK(cudaMemcpyAsync(l->rw_unscale.get(), unscale.data(), NE * sizeof(float), cudaMemcpyHostToDevice, st));
  l->rx_hi.alloc(xrows * E), l->rx_lo.alloc(xrows * E);
  CUDA_OK(cudaMemsetAsync(l->rx_hi.get(), 0, xrows * E * sizeof(__half), st));
  CUDA_OK(cudaMemsetAsync(l->rx_lo.get(), 0, xrows * E * sizeof(__half), st));
  l->approx.alloc((size_t)T * NE), l->norm2_parts.alloc((size_t)T * (E / 256));
  l->rw_hi_map = make_rows_map(l->rw_hi.get(), wrows, E, 128);  // 128 experts a box: an item takes one or two
  l->rw_lo_map = make_rows_map(l->rw_lo.get(), wrows, E, 128);
  l->rx_hi_map = make_rows_map(l->rx_hi.get(), xrows, E, kRouterTileRows);
  l->rx_lo_map = make_rows_map(l->rx_lo.get(), xrows, E, kRouterTileRows);
  CUDA_OK(cudaStreamSynchronize(st));
}

// gate: with the rows' product with this vector wanted too (the shared expert's gate logit), its parts go to gate_parts.
void quantize_rows(moe_layer *l, const float *src, uint64_t rows, uint32_t Kv, const ActBuffers &dst, cudaStream_t st,
                   const float *gate = nullptr, float *gate_parts = nullptr, RouterSplit rs = RouterSplit{}) {
  const uint64_t nblk = rows * (Kv / 256);
  if (nblk == 0) return;
  const ActView v = dst.view();
  const unsigned grid = (unsigned)((nblk + 7) / 8);
  if (dst.q8k)
    launched(l, launch_kernel(l->ctx.pdl, k_quant_q8_K, dim3(grid), dim3(256), 0, st, src, nblk, (int8_t *)v.q, (float *)v.d, (int16_t *)v.bs, dst.h.get(),
                              gate, Kv / 256, gate_parts, rs),
             "quantize");
  else
    launched(l, launch_kernel(l->ctx.pdl, k_quant_q8_0, dim3(grid), dim3(256), 0, st, src, nblk, (int8_t *)v.q, (float *)v.d, dst.h.get(), gate, Kv / 256,
                              gate_parts, rs),
             "quantize");
}

// Whether a call of R expert rows keeps its experts' results in f16: when every expert takes the tile kernels, whose
// products are f16 products already. The down kernel then writes half the bytes and the combine reads half; the sum
// over a row's experts stays in f32.
bool results_f16(const moe_layer *l, uint32_t tm) { return l->can_tensor && tm == 1; }

// Rows a group's kernel takes at once, for groups that hold at most n rows.
int group_rows(uint64_t n) { return n > 4 ? 8 : n > 2 ? 4 : (int)n; }

// The most rows a group holds in a call of R expert rows over nexp experts. With no more rows than experts nearly every
// expert has one or two: groups of two keep the kernel's accumulators few and its occupancy up, and the odd expert
// with more rows is read again by its next group, out of L2. With more rows, groups of eight read an expert once.
uint32_t group_cap(uint64_t R, uint32_t nexp) { return R <= nexp ? 2 : kGroupMax; }

// Rows from which an expert goes to the tensor-core kernels in a call of R expert rows; 0: none does. With few rows in
// all, the step is bound by reading each expert once and the integer-dot kernels do that best; with many, every
// expert's rows fill tensor-core tiles better than groups of 8.
uint32_t tensor_min_for(const moe_layer *l, uint64_t R) {
  if (!l->can_tensor) return 0;
  if (l->cfg.tensor_min_rows) return l->cfg.tensor_min_rows;
  return R >= 1280 ? 1 : 16;
}

// With the default threshold and a short step, the pack may lower the threshold itself to as few as 1 row, as long as
// no more than this many experts then take the tile kernels (half the SMs: each expert is four gate/up items). 0: fixed,
// as in steps of a few rows, where two more launches would cost more than they could save.
uint32_t tensor_budget_for(const moe_layer *l, uint64_t R) {
  return l->can_tensor && !l->cfg.tensor_min_rows && R >= 64 && R < 1280 ? l->sms / 2 : 0;
}

// Quantise x, the router's logits and top-k, and the pack of the step's T * K assignments over every expert.
void stage_route(moe_layer *l, const float *x, uint32_t T, cudaStream_t st) {
  const uint32_t E = l->E, NE = l->NE, K = l->K, N = l->N;
  const uint64_t A = (uint64_t)T * K;
  // Steps of up to kRouterExactRows rows (and every step of a layer kept off the tensor cores) take the exact fp32
  // product; longer ones the tensor-core product, whose logits the top-k kernel treats as approximate.
  const bool approx = l->router_tensor && T > kRouterExactRows;
  mark(l, ST_QUANT, st);
  if (approx)
    quantize_rows(l, x, T, E, l->xq_routed, st, l->router.get() + (size_t)NE * E, l->gate_parts.get(),
                  RouterSplit{l->rx_hi.get(), l->rx_lo.get(), l->norm2_parts.get()});
  else
    quantize_rows(l, x, T, E, l->xq_routed, st);
  if (l->has_shared && !l->shared_x_same) quantize_rows(l, x, T, E, l->xq_shared, st);
  mark(l, ST_ROUTER, st);
  if (!approx) {
    // Steps of up to 2 rows stage only those (8 KB a row); longer ones 8 rows a pass.
    const uint32_t tm = T <= 2 ? T : 8;
    const size_t smem = (size_t)tm * kRouterPieces * (E / kRouterPieces + 4) * sizeof(float);
    if (!l->rows_attr_set) {
      const int most = (int)((size_t)8 * kRouterPieces * (E / kRouterPieces + 4) * sizeof(float));
      CUDA_OK(cudaFuncSetAttribute(k_router_logits_rows<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
      l->rows_attr_set = true;
    }
    const uint32_t warps = tm <= 2 ? 1 : 8;
    const dim3 grid((N + 4 * warps - 1) / (4 * warps), (T + tm - 1) / tm);
    const bool deep = (E / kRouterPieces) % 64 == 0;  // sixteen loads in flight a lane: a step of one row is all latency
    if (tm == 1 && deep)
      k_router_logits_rows<1, 16><<<grid, 32, smem, st>>>(x, T, E, l->router.get(), N, l->bias.get(), NE, l->rl.get());
    else if (tm == 1)
      k_router_logits_rows<1><<<grid, 32, smem, st>>>(x, T, E, l->router.get(), N, l->bias.get(), NE, l->rl.get());
    else if (tm == 2 && deep)
      k_router_logits_rows<2, 16><<<grid, 32, smem, st>>>(x, T, E, l->router.get(), N, l->bias.get(), NE, l->rl.get());
    else if (tm == 2)
      k_router_logits_rows<2><<<grid, 32, smem, st>>>(x, T, E, l->router.get(), N, l->bias.get(), NE, l->rl.get());
    else
      k_router_logits_rows<8><<<grid, 256, smem, st>>>(x, T, E, l->router.get(), N, l->bias.get(), NE, l->rl.get());
  } else {
    if (!l->router_attr_set) {
      CUDA_OK(cudaFuncSetAttribute(k_router_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRouterSmemBytes));
      l->router_attr_set = true;
    }
    // Items of 256 experts halve what is read of x again; items of 128 give a short step twice the CTAs, as long as
    // they still all run at once (8,192 rows: 128 items of 256 experts took 50 us, 256 items of 128 took 62).
    const uint32_t row_tiles = (T + kRouterTileRows - 1) / kRouterTileRows;
    const uint32_t ne_tile = 2 * row_tiles * ((NE + kRouterTileExperts - 1) / kRouterTileExperts) <= l->sms ? 128 : kRouterTileExperts;
    const RouterMmaArgs ra{T, E, NE, ne_tile, l->rw_unscale.get(), l->approx.get(), l->error.get()};
    const uint32_t items = row_tiles * ((NE + ne_tile - 1) / ne_tile);
    k_router_mma<<<std::min(items, l->sms), kRouterThreads, kRouterSmemBytes, st>>>(ra, l->rx_hi_map, l->rx_lo_map, l->rw_hi_map, l->rw_lo_map);
  }
  launched(l, cudaGetLastError(), "router logits");
  const uint32_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  // On one GPU the pack also lists the groups and big tiles of the experts' kernels; expert parallel, it only sorts.
  const uint32_t tm = l->local == NE ? tensor_min_for(l, A) : 0, budget = l->local == NE ? tensor_budget_for(l, A) : 0;
  l->last_tensor_min = tm;
  const uint32_t chunk_len = kChunkTokens * K;
  if (nchunks == 1 && NE <= 512) {
    // One chunk: top-k, scan and fill in one CTA (the pack stage then has no kernel of its own).
    launched(l, launch_kernel(l->ctx.pdl, k_router_topk_pack, dim3(1), dim3(32 * kChunkTokens), chunk_len * sizeof(int32_t), st, l->rl.get(), l->bias.get(),
                              T, NE, K, l->ids.get(), l->w.get(), l->gs.get(), tm, budget, group_cap(A, NE), l->pack.out(), l->pack.inv.get(),
                              l->pack.row_src.get()),
             "router top-k and pack");
    mark(l, ST_PACK, st);
  } else {
    if (approx) {
      const RouterApprox ap{l->approx.get(), x, l->router.get(), l->norm2_parts.get(), l->gate_parts.get(), E, E / 256,
                            l->router_eps_rel, l->router_eps_abs};
      k_router_topk_rows<<<(T + kTopkRowsPerCta - 1) / kTopkRowsPerCta, 32 * kTopkRowsPerCta, 0, st>>>(ap, l->bias.get(), T, NE, K, l->ids.get(),
                                                                                                  l->w.get(), l->gs.get());
      launched(l, cudaGetLastError(), "router top-k");
      k_chunk_hist<<<nchunks, 256, 0, st>>>(l->ids.get(), (uint32_t)A, chunk_len, NE, 0, l->pack.chunk_hist.get());
      launched(l, cudaGetLastError(), "chunk counts");
    } else {
      k_router_topk<<<nchunks, 32 * kChunkTokens, 0, st>>>(l->rl.get(), RouterApprox{}, l->bias.get(), T, NE, K, l->ids.get(), l->w.get(),
                                                          l->gs.get(), l->pack.chunk_hist.get());
      launched(l, cudaGetLastError(), "router top-k");
    }
    mark(l, ST_PACK, st);
    launch_pack(l, l->pack, PackJob{l->ids.get(), (uint32_t)A, chunk_len, nchunks, 0, tm, budget, group_cap(A, NE), K}, st);
  }
  l->last_T = T, l->last_pack = &l->pack;
}

constexpr uint64_t kGatherInKernelRows = 163840;  // expert rows from which the gate/up tile kernel gathers its rows itself

// The routed experts on the R rows a pack lists: gate/up and SwiGLU into h, h quantised, down into y (expert order).
// most: the most rows one expert can have (a step's tokens; in an expert-parallel call, not known below R).
// y16: the results in f16 (only with every expert on the tile kernels: the integer-dot kernels write f32).
// rows_in: when not 0, src holds that many rows and every one of them has R / rows_in places in expert order, pk.inv[row *
// (R / rows_in) + k] (a GPU's own step); 0: a row's places are not laid out so (rows that came from other GPUs).
// in_order: the caller has put the rows' f16 form in expert order already (l->xg).
void stage_experts(moe_layer *l, const ActSource &src, const PackBuffers &pk, uint64_t R, uint64_t most, uint32_t tm, void *y, bool y16,
                   cudaStream_t st, uint32_t rows_in = 0, bool in_order = false) {
  const uint32_t E = l->E, F = l->F, nexp = pk.nexp;
  const moe_layer_config &c = l->cfg;
  // The most groups and big tiles the rows can make: an expert below tm rows has (tm - 2) / 8 + 1 groups at most, and one
  // at or above it a tile per 256 rows and one more.
  const uint32_t gmax = group_cap(R, nexp);
  const int M = group_rows(std::min<uint64_t>(std::min<uint64_t>(gmax, most), tm ? std::min<uint64_t>(R, tm - 1) : R));
  const uint32_t max_groups =
      tm ? (tm > 1 ? (uint32_t)std::min<uint64_t>(R, (uint64_t)nexp * ((tm - 2) / gmax + 1)) : 0) : (uint32_t)std::min<uint64_t>(R, R / gmax + nexp);
  // The pack may have lowered the threshold to 1 (tensor_budget_for): the tile launches are sized for that.
  const uint32_t tm_low = tm && tensor_budget_for(l, R) ? 1 : tm;
  const uint32_t max_big = tm_low && R >= tm_low ? (uint32_t)(R / kTileN + std::min<uint64_t>(nexp, R / tm_low)) : 0;
  // With MOE_FLAG_GATHER_IN_KERNEL, long steps of a GPU's own rows: the gate/up tile kernel gathers the rows by index
  // itself (cp.async.bulk.tensor's tile::gather4 form, 32 copies of four rows a stage for a pair's CTA instead of two
  // boxes of 64) and no copy to expert order runs. The copies then set that kernel's pace (1.39 -> 1.85 ms at 32,768
  // rows): even with the 0.48 ms the copy took as a gather, 0.2 ms behind the 0.24 ms it takes as a scatter. Off by default.
  // (The same gather by the copy warp's own 16-byte asynchronous copies, cp.async, was slower still: 2.26 ms.)
  const bool gather_in_kernel = (l->cfg.flags & MOE_FLAG_GATHER_IN_KERNEL) && max_big && R >= kGatherInKernelRows &&
                                src.h == l->xq_routed.h.get() && src.act_row != nullptr;
  if (max_big) {
    // The rows in expert order first (the reference's p_moe_scatter, kernels/models/qwen4exp/prompt.cl:744-754): a tile's
    // rows are then one box after another for the kernel's copies. Part of the pack stage: the gate/up stage times the
    // product's own kernels.
    if (!gather_in_kernel && !in_order) {
      if (!rows_in) throw std::logic_error("rows neither in expert order nor with their places laid out");
      k_scatter_f16<<<rows_in, 256, 0, st>>>(src.h, pk.inv.get(), (uint32_t)(R / rows_in), E, l->xg.get());
      launched(l, cudaGetLastError(), "rows to expert order");
    }
  }
  mark(l, ST_GATE_UP, st);
  if (max_big) {
    ExpertTilesArgs a{};
    a.w0 = l->wg.get(), a.w1 = l->wu.get(), a.slice_bytes = l->gate_slice, a.K = E, a.R = F;
    a.qmap[0] = l->wg_q, a.qmap[1] = l->wu_q;
    a.tiles = pk.big.get(), a.ntiles = pk.counters.get() + 4;
    a.out = l->h.get(), a.out_stride = F, a.limit = c.swiglu_limit, a.error = l->error.get();
    if (gather_in_kernel) {
      a.gather_rows = src.act_row;
      launched(l, launch_tiles(c.gate_type, 2, a, l->xq_routed.h_row_map, max_big, l->grid.get(), l->ctx, st), "experts gate/up tiles");
    } else {
      launched(l, launch_tiles(c.gate_type, 2, a, l->xg_map, max_big, l->grid.get(), l->ctx, st), "experts gate/up tiles");
    }
  }
  if (max_groups) {
    ExpertRowsArgs a{};
    a.w0 = l->wg.get(), a.w1 = l->wu.get(), a.slice_bytes = l->gate_slice, a.K = E, a.R = F, a.rows_per_cta = 32;
    a.act = src.view, a.act_row = src.act_row;
    a.groups = pk.groups.get(), a.ngroups = pk.counters.get() + 1;
    a.out = l->h.get(), a.out_stride = F, a.limit = c.swiglu_limit;
    launched(l, launch_rows(c.gate_type, 2, a, M, max_groups, l->grid.get(), l->ctx, st), "experts gate/up");
  }
  mark(l, ST_DOWN, st);  // the down stage starts with its input's quantiser
  quantize_rows(l, l->h.get(), R, F, l->hq_routed, st);
  if (max_big) {
    ExpertTilesArgs a{};
    a.w0 = l->wd.get(), a.slice_bytes = l->down_slice, a.K = F, a.R = E;
    a.qmap[0] = l->wd_q;
    a.tiles = pk.big.get(), a.ntiles = pk.counters.get() + 4;
    a.out = y, a.out_stride = E, a.out_f16 = y16, a.error = l->error.get();
    launched(l, launch_tiles(c.down_type, 1, a, l->hq_routed.h_map, max_big, l->grid.get(), l->ctx, st), "experts down tiles");
  }
  if (max_groups) {
    ExpertRowsArgs a{};
    a.w0 = l->wd.get(), a.slice_bytes = l->down_slice, a.K = F, a.R = E, a.rows_per_cta = 128;
    a.act = l->hq_routed.view(), a.act_row = nullptr;
    a.groups = pk.groups.get(), a.ngroups = pk.counters.get() + 1;
    if (y16) throw std::logic_error("f16 results with experts on the integer-dot kernels");
    a.out = (float *)y, a.out_stride = E;
    launched(l, launch_rows(c.down_type, 1, a, M, max_groups, l->grid.get(), l->ctx, st), "experts down");
  }
}

// The shared expert on the step's T rows, into s. Its h rows sit after the routed experts' in h.
void stage_shared(moe_layer *l, uint32_t T, cudaStream_t st) {
  mark(l, ST_SHARED, st);
  if (!l->has_shared) return;
  const uint32_t E = l->E, F = l->F;
  const moe_layer_config &c = l->cfg;
  const ActBuffers &xs = l->shared_x_same ? l->xq_routed : l->xq_shared;
  float *hs = l->h.get() + l->Rmax * F;
  if (l->can_tensor && T >= (l->cfg.tensor_min_rows ? l->cfg.tensor_min_rows : 16)) {
    const uint32_t dense_tiles = (T + kTileN - 1) / kTileN;
    ExpertTilesArgs a{};
    a.w0 = l->sg.get(), a.w1 = l->su.get(), a.K = E, a.R = F, a.dense_rows = T;
    a.qmap[0] = l->sg_q, a.qmap[1] = l->su_q;
    a.out = hs, a.out_stride = F, a.limit = c.swiglu_limit, a.error = l->error.get();
    launched(l, launch_tiles(c.shexp_gate_type, 2, a, xs.h_map, dense_tiles, l->grid.get(), l->ctx, st), "shared gate/up tiles");
    quantize_rows(l, hs, T, F, l->hq_shared, st);
    ExpertTilesArgs b{};
    b.w0 = l->sd.get(), b.K = F, b.R = E, b.dense_rows = T;
    b.qmap[0] = l->sd_q;
    b.out = l->s.get(), b.out_stride = E, b.error = l->error.get();
    launched(l, launch_tiles(c.shexp_down_type, 1, b, l->hq_shared.h_map, dense_tiles, l->grid.get(), l->ctx, st), "shared down tiles");
    l->shared_on_tensor = true;
    return;
  }
  l->shared_on_tensor = false;
  const int M = group_rows(T);
  const uint32_t dense_groups = (T + M - 1) / M;
  ExpertRowsArgs a{};
  a.w0 = l->sg.get(), a.w1 = l->su.get(), a.K = E, a.R = F, a.rows_per_cta = 32;
  a.act = xs.view(), a.dense_rows = T, a.out = hs, a.out_stride = F, a.limit = c.swiglu_limit;
  launched(l, launch_rows(c.shexp_gate_type, 2, a, M, dense_groups, l->grid.get(), l->ctx, st), "shared gate/up");
  quantize_rows(l, hs, T, F, l->hq_shared, st);
  ExpertRowsArgs b{};
  b.w0 = l->sd.get(), b.K = F, b.R = E, b.rows_per_cta = 128;
  b.act = l->hq_shared.view(), b.dense_rows = T, b.out = l->s.get(), b.out_stride = E;
  launched(l, launch_rows(c.shexp_down_type, 1, b, M, dense_groups, l->grid.get(), l->ctx, st), "shared down");
}

template <class Y>
void stage_combine(moe_layer *l, const Y *y, uint32_t T, float *out, cudaStream_t st) {
  mark(l, ST_COMBINE, st);
  launched(l, launch_kernel(l->ctx.pdl, k_combine<Y>, dim3(T), dim3(256), 0, st, y, (const uint32_t *)l->pack.inv.get(), (const float *)l->w.get(),
                            (const float *)l->gs.get(), (const float *)(l->has_shared ? l->s.get() : nullptr), l->K, l->E, out, l->residual),
           "combine");
  mark(l, ST_COPIES, st);
}

constexpr uint32_t kGraphMaxRows = 64;
constexpr uint64_t kSharedInlineRows = 65536;  // expert rows from which the shared expert runs after the routed ones, not beside them

// The whole block on device buffers, queued on st: a GPU that holds every expert.
void forward_device(moe_layer *l, const float *x, uint32_t T, float *out, cudaStream_t st) {
  if (l->local != l->NE) throw BadArgument("this call needs every expert on the GPU; an expert-parallel layer goes stage by stage");
  const uint64_t A = (uint64_t)T * l->K;
  // Launch-bound steps (the ones that are also replayed from a graph): each kernel a programmatic dependent of the one
  // before it in its stream.
  l->ctx.pdl = T <= kGraphMaxRows && !l->profile && l->pdl_ok;
  struct PdlOff {
    LaunchCtx &c;
    ~PdlOff() { c.pdl = false; }
  } pdl_off{l->ctx};
  // The shared expert needs only the quantised rows: it runs on a second stream beside the routed experts and joins
  // before the combine. With per-stage timing on, it runs in line instead, so that its stage can be timed.
  // In long steps it runs in line after all: the routed kernels then fill the GPU for many rounds of items dealt to
  // their CTAs beforehand, and CTAs that start late because the shared expert's hold their SMs finish late (a step of
  // 32,768 rows measured 6 % slower with the two side by side than one after the other; 3,521 rows 5 % faster).
  const bool beside = l->has_shared && !l->profile && A < kSharedInlineRows;
  // (The quantiser of a short step, whose exact router reads x itself, was tried on the second stream as well, ahead of
  // the shared expert: 5 us slower at one row, 2 % faster on a stack of 48 layers of 32 rows; not kept.)
  stage_route(l, x, T, st);
  if (beside) {
    l->fork_ev->record(st);
    CUDA_OK(cudaStreamWaitEvent(l->aux->get(), l->fork_ev->get(), 0));
    stage_shared(l, T, l->aux->get());
    l->join_ev->record(l->aux->get());
  }
  const ActSource src{l->xq_routed.view(), l->xq_routed.h.get(), l->pack.row_src.get()};
  const bool y16 = results_f16(l, l->last_tensor_min);
  stage_experts(l, src, l->pack, A, T, l->last_tensor_min, l->y.get(), y16, st, T);
  if (beside)
    CUDA_OK(cudaStreamWaitEvent(st, l->join_ev->get(), 0));
  else
    stage_shared(l, T, st);
  if (y16)
    stage_combine<__half>(l, (const __half *)l->y.get(), T, out, st);
  else
    stage_combine<float>(l, l->y.get(), T, out, st);
  l->stats.calls++, l->stats.rows += T, l->stats.assignments += A;
}


// forward_device, replayed from a graph when the step is small and has been seen before with the same buffers.
void forward_step(moe_layer *l, const float *x, uint32_t T, float *out, cudaStream_t st) {
  if (l->profile || !l->graphs_ok || T > kGraphMaxRows || l->local != l->NE) return forward_device(l, x, T, out, st);
  moe_layer::StepGraph *g = nullptr;
  for (auto &c : l->graphs)
    if (c.T == T && c.x == x && c.res == l->residual && c.out == out && c.st == st) g = &c;
  if (g && g->exec) {
    CUDA_OK(cudaGraphLaunch(g->exec, st));
    l->stats.kernels += g->kernels, l->stats.calls++, l->stats.rows += T, l->stats.assignments += (uint64_t)T * l->K;
    l->last_T = T, l->last_pack = &l->pack, l->last_tensor_min = tensor_min_for(l, (uint64_t)T * l->K);
    return;
  }
  if (!g) {  // first sight: run it plainly (this also sets the kernels' attributes); record it the next time
    if (l->graphs.size() >= 16) {
      if (l->graphs.front().exec) cudaGraphExecDestroy(l->graphs.front().exec);
      l->graphs.erase(l->graphs.begin());
    }
    l->graphs.push_back(moe_layer::StepGraph{T, x, l->residual, out, st, nullptr, 0, 1});
    return forward_device(l, x, T, out, st);
  }
  const moe_layer_stats before = l->stats;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
  if (e == cudaSuccess) {
    try {
      forward_device(l, x, T, out, st);
    } catch (...) {
      cudaStreamEndCapture(st, &graph);
      if (graph) cudaGraphDestroy(graph);
      l->graphs_ok = false;
      l->stats = before;
      cudaGetLastError();
      return forward_device(l, x, T, out, st);
    }
    e = cudaStreamEndCapture(st, &graph);
  }
  if (e == cudaSuccess && graph) e = cudaGraphInstantiate(&g->exec, graph, 0);
  if (graph) cudaGraphDestroy(graph);
  if (e != cudaSuccess || !g->exec) {  // recording is an optimisation: without it the call still runs
    cudaGetLastError();
    g->exec = nullptr, l->graphs_ok = false, l->stats = before;
    return forward_device(l, x, T, out, st);
  }
  g->kernels = l->stats.kernels - before.kernels;
  l->stats = before;
  CUDA_OK(cudaGraphLaunch(g->exec, st));
  l->stats.kernels += g->kernels, l->stats.calls++, l->stats.rows += T, l->stats.assignments += (uint64_t)T * l->K;
}

// After the stream has drained: a kernel whose wait ran out left the error word set.
void check_device_error(moe_layer *l) {
  uint32_t e = 0;
  CUDA_OK(cudaMemcpy(&e, l->error.get(), sizeof(e), cudaMemcpyDeviceToHost));
  if (e) {
    CUDA_OK(cudaMemset(l->error.get(), 0, sizeof(e)));
    throw Timeout("a tensor-core kernel gave up waiting on a barrier; the call's results are not valid");
  }
}

void read_counters(moe_layer *l) {
  uint32_t c[8];
  CUDA_OK(cudaMemcpy(c, l->last_pack->counters.get(), sizeof(c), cudaMemcpyDeviceToHost));
  l->stats.last_tiles = c[0], l->stats.last_experts_hit = c[2];
  l->stats.last_tensor_rows = c[5] + (l->shared_on_tensor ? l->last_T : 0);
}

// The kernels read rows through 16-byte loads: a device pointer that is not 16-byte aligned is refused here, where the
// answer is a status, rather than found by a kernel, where it is a fault.
void need_aligned16(std::initializer_list<const void *> ps) {
  for (const void *p : ps)
    if ((uintptr_t)p & 15) throw BadArgument("device pointers must be 16-byte aligned");
}

template <class Fn>
moe_status guarded(moe_layer *l, Fn &&fn) {
  try {
    if (l) CUDA_OK(cudaSetDevice(l->cfg.device));
    fn();
    return MOE_OK;
  } catch (const BadArgument &e) {
    (l ? l->err : g_create_error) = e.what();
    return MOE_BAD_ARGUMENT;
  } catch (const Timeout &e) {
    (l ? l->err : g_create_error) = e.what();
    return MOE_TIMEOUT;
  } catch (const std::exception &e) {
    (l ? l->err : g_create_error) = e.what();
    return MOE_ERROR;
  }
}

}  // namespace

extern "C" {

MOE_API moe_status moe_layer_create(const moe_layer_config *config, const moe_layer_weights *weights, moe_layer **out) {
  if (!config || !weights || !out) {
    g_create_error = "config, weights and out are required";
    return MOE_BAD_ARGUMENT;
  }
  *out = nullptr;
  auto l = std::make_unique<moe_layer>();
  moe_layer *raw = l.get();
  const moe_status s = guarded(nullptr, [&] { create(raw, *config, *weights); });
  if (s == MOE_OK) *out = l.release();
  return s;
}

MOE_API void moe_layer_destroy(moe_layer *l) {
  if (!l) return;
  cudaSetDevice(l->cfg.device);
  if (l->stream) cudaStreamSynchronize(l->stream->get());
  if (l->aux) cudaStreamSynchronize(l->aux->get());
  if (l->copy_out) cudaStreamSynchronize(l->copy_out->get());
  for (auto &g : l->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  delete l;
}

MOE_API moe_status moe_layer_forward(moe_layer *l, const float *x, uint32_t T, float *out) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!x || !out || T == 0 || T > l->Tmax) throw BadArgument("x and out are required, and 1 <= T <= max_tokens");
    cudaStream_t st = l->stream->get();
    const size_t bytes = (size_t)T * l->E * sizeof(float);
    const uint32_t chunk = l->cfg.host_chunk_rows;
    if (chunk && T >= 2 * chunk && !l->profile && l->local == l->NE) {
      // Chunks of equal size, about host_chunk_rows each: chunk c's rows come in on one stream while chunk c - 1 is
      // computed on the layer's and chunk c - 2's results leave on a third.
      const uint32_t n = T / chunk, rows = (T + n - 1) / n;
      if (!l->copy_in) l->copy_in = std::make_unique<Stream>(), l->copy_out = std::make_unique<Stream>();
      while (l->in_done.size() < n) l->in_done.push_back(std::make_unique<Event>()), l->comp_done.push_back(std::make_unique<Event>());
      for (uint32_t c = 0; c < n; c++) {
        const uint32_t t0 = c * rows, tn = std::min(rows, T - t0);
        CUDA_OK(cudaMemcpyAsync(l->x.get() + (size_t)t0 * l->E, x + (size_t)t0 * l->E, (size_t)tn * l->E * sizeof(float), cudaMemcpyHostToDevice,
                                l->copy_in->get()));
        l->in_done[c]->record(l->copy_in->get());
      }
      for (uint32_t c = 0; c < n; c++) {
        const uint32_t t0 = c * rows, tn = std::min(rows, T - t0);
        CUDA_OK(cudaStreamWaitEvent(st, l->in_done[c]->get(), 0));
        forward_step(l, l->x.get() + (size_t)t0 * l->E, tn, l->out.get() + (size_t)t0 * l->E, st);
        l->comp_done[c]->record(st);
        CUDA_OK(cudaStreamWaitEvent(l->copy_out->get(), l->comp_done[c]->get(), 0));
        CUDA_OK(cudaMemcpyAsync(out + (size_t)t0 * l->E, l->out.get() + (size_t)t0 * l->E, (size_t)tn * l->E * sizeof(float), cudaMemcpyDeviceToHost,
                                l->copy_out->get()));
      }
      l->stats.h2d_bytes += bytes, l->stats.d2h_bytes += bytes;
      l->copy_out->wait(0);
      l->stream->wait(0);
      check_device_error(l);
      return;
    }
    CUDA_OK(cudaMemcpyAsync(l->x.get(), x, bytes, cudaMemcpyHostToDevice, st));
    forward_step(l, l->x.get(), T, l->out.get(), st);
    CUDA_OK(cudaMemcpyAsync(out, l->out.get(), bytes, cudaMemcpyDeviceToHost, st));
    if (l->profile) l->ev[MOE_STAGES]->record(st), l->ev_valid = true;
    l->stats.h2d_bytes += bytes, l->stats.d2h_bytes += bytes;
    l->stream->wait(0);
    check_device_error(l);
  });
}

MOE_API moe_status moe_layer_forward_device(moe_layer *l, const float *x_dev, uint32_t T, float *out_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!x_dev || !out_dev || T == 0 || T > l->Tmax) throw BadArgument("x and out are required, and 1 <= T <= max_tokens");
    need_aligned16({x_dev, out_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    forward_step(l, x_dev, T, out_dev, st);
    if (l->profile) l->ev[MOE_STAGES]->record(st), l->ev_valid = true;
  });
}

MOE_API moe_status moe_layer_forward_residual_device(moe_layer *l, const float *x_dev, uint32_t T, const float *residual_dev,
                                                     float *out_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!x_dev || !out_dev || !residual_dev || T == 0 || T > l->Tmax) throw BadArgument("x, residual and out are required, and 1 <= T <= max_tokens");
    need_aligned16({x_dev, residual_dev, out_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    l->residual = residual_dev;
    try {
      forward_step(l, x_dev, T, out_dev, st);
    } catch (...) {
      l->residual = nullptr;
      throw;
    }
    l->residual = nullptr;
    if (l->profile) l->ev[MOE_STAGES]->record(st), l->ev_valid = true;
  });
}

// ---------------------------------------------------------------------------------------------------------------
// Expert parallel, stage by stage. The caller moves the rows between GPUs (all-to-all) between the stages.

MOE_API moe_status moe_layer_route_device(moe_layer *l, const float *x_dev, uint32_t T, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!x_dev || T == 0 || T > l->Tmax) throw BadArgument("x is required, and 1 <= T <= max_tokens");
    need_aligned16({x_dev});
    stage_route(l, x_dev, T, stream ? (cudaStream_t)stream : l->stream->get());
    l->stats.calls++, l->stats.rows += T, l->stats.assignments += (uint64_t)T * l->K;
  });
}

MOE_API moe_status moe_layer_read_counts(moe_layer *l, uint32_t *cnt, void *stream) {
  if (!l || !cnt) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    CUDA_OK(cudaMemcpyAsync(cnt, l->pack.cnt.get(), l->NE * sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    Stream::wait_on(st, 0);
  });
}

MOE_API moe_status moe_layer_counts_device(moe_layer *l, uint32_t *cnt_dev, void *stream) {
  if (!l || !cnt_dev) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    CUDA_OK(cudaMemcpyAsync(cnt_dev, l->pack.cnt.get(), l->NE * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
  });
}

MOE_API moe_status moe_layer_received_ids_device(moe_layer *l, const uint32_t *cnt_all_dev, uint32_t world, int32_t *ids_dev, void *stream) {
  if (!l || !cnt_all_dev || !ids_dev || world == 0) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    k_received_ids<<<world * l->local, 128, 0, st>>>(cnt_all_dev, l->NE, l->cfg.expert_first, l->local, ids_dev);
    launched(l, cudaGetLastError(), "received ids");
  });
}

MOE_API uint32_t moe_layer_wire_row_bytes(const moe_layer *l) { return l ? wire_row_bytes(act_is_q8k(l->cfg.gate_type), l->E) : 0; }

MOE_API moe_status moe_layer_gather_rows_device(moe_layer *l, void *rows_dev, int32_t *ids_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!rows_dev || !ids_dev || l->last_T == 0) throw BadArgument("rows and ids are required, after moe_layer_route_device");
    need_aligned16({rows_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    const uint32_t A = l->last_T * l->K;
    k_gather_wire<<<(A + 7) / 8, 256, 0, st>>>(l->xq_routed.view(), l->E, l->xq_routed.q8k, l->pack.row_src.get(), l->pack.inv.get(),
                                             l->ids.get(), A, (uint8_t *)rows_dev, ids_dev);
    launched(l, cudaGetLastError(), "gather rows");
  });
}

MOE_API moe_status moe_layer_experts_device(moe_layer *l, const void *rows_dev, const int32_t *ids_dev, uint32_t R, void *y_dev,
                                            uint32_t y_f16, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->local == l->NE) throw BadArgument("this layer holds every expert: use moe_layer_forward_device");
    if (R > l->Rmax) throw BadArgument("more rows than max_expert_rows");
    if (R == 0) return;
    if (!rows_dev || !ids_dev || !y_dev) throw BadArgument("rows, ids and y are required");
    need_aligned16({rows_dev, y_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    const uint32_t E = l->E, nexp = l->local;
    const bool q8k = l->xq_routed.q8k;
    const uint32_t wb = wire_row_bytes(q8k, E), tm = tensor_min_for(l, R);
    // Sort the rows by expert among this GPU's experts: a stable pack, chunks of 512 entries.
    PackBuffers &pk = l->pack_local;
    const uint32_t nchunks = (R + kLocalChunk - 1) / kLocalChunk;
    k_chunk_hist<<<nchunks, 256, 0, st>>>(ids_dev, R, kLocalChunk, nexp, l->cfg.expert_first, pk.chunk_hist.get());
    launched(l, cudaGetLastError(), "local counts");
    launch_pack(l, pk, PackJob{ids_dev, R, kLocalChunk, nchunks, l->cfg.expert_first, tm, tensor_budget_for(l, R), group_cap(R, nexp), 1}, st);
    const uint8_t *wire = (const uint8_t *)rows_dev;
    const uint32_t dbytes = q8k ? E / 64 : E / 8;
    ActSource src{ActView{(const int8_t *)wire, (const float *)(wire + E), (const int16_t *)(wire + E + dbytes), wb, wb, wb}, nullptr,
                  pk.row_src.get()};
    if (tm) {
      // The rows' f16 form straight to their places in expert order (one place a row here).
      const uint64_t nblk = (uint64_t)R * (E / 256);
      k_wire_to_f16<<<(unsigned)((nblk + 7) / 8), 256, 0, st>>>(wire, E, q8k, nblk, l->xg.get(), 0, ids_dev, pk.inv.get(), 1, l->Rmax);
      launched(l, cudaGetLastError(), "wire rows to f16, in expert order");
    }
    l->last_pack = &pk;
    // The results stay f16 in between only when they also leave as f16 (f32 results are the bit-exact mode).
    const bool y16 = y_f16 && results_f16(l, tm);
    stage_experts(l, src, pk, R, R, tm, l->y.get(), y16, st, 0, true);
    if (y16)
      k_unpermute<__half, __half><<<R, 256, 0, st>>>((const __half *)l->y.get(), pk.inv.get(), E, (__half *)y_dev);
    else if (y_f16)
      k_unpermute<float, __half><<<R, 256, 0, st>>>(l->y.get(), pk.inv.get(), E, (__half *)y_dev);
    else
      k_unpermute<float, float><<<R, 256, 0, st>>>(l->y.get(), pk.inv.get(), E, (float *)y_dev);
    launched(l, cudaGetLastError(), "rows back in arrival order");
  });
}

// ---------------------------------------------------------------------------------------------------------------
// Expert parallel with one row per (token, GPU) on the way out and one weighted partial sum per (token, GPU) back.

MOE_API uint32_t moe_layer_dispatch_row_bytes(const moe_layer *l) { return l ? dispatch_row_bytes(act_is_q8k(l->cfg.gate_type), l->E) : 0; }

MOE_API moe_status moe_layer_dispatch_plan_device(moe_layer *l, uint32_t *totals_dev, void *stream) {
  if (!l || !totals_dev) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("after moe_layer_route_device");
    const uint32_t world = l->NE / l->local;
    if (l->local * world != l->NE || world > kMaxWorld || l->cfg.expert_first % l->local)
      throw BadArgument("the GPUs must hold equal contiguous ranges of the experts, eight GPUs at most");
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    const uint32_t T = l->last_T, nchunks = (T + kDestChunk - 1) / kDestChunk;
    if (!l->dest_pos.get()) {
      const uint32_t most = (l->Tmax + kDestChunk - 1) / kDestChunk;
      l->dest_pos.alloc((size_t)l->Tmax * kMaxWorld), l->dest_chunk_cnt.alloc(most * kMaxWorld), l->dest_chunk_asg.alloc(most * kMaxWorld);
      l->dest_totals.alloc(2 * kMaxWorld);
    }
    l->dest_world = world;
    k_dest_count<<<nchunks, kDestChunk, 0, st>>>(l->ids.get(), T, l->K, l->local, l->dest_chunk_cnt.get(), l->dest_chunk_asg.get());
    launched(l, cudaGetLastError(), "destination counts");
    k_dest_fill<<<nchunks, kDestChunk, 0, st>>>(l->ids.get(), T, l->K, l->local, l->dest_chunk_cnt.get(), l->dest_chunk_asg.get(), nchunks,
                                                l->dest_pos.get(), l->dest_totals.get());
    launched(l, cudaGetLastError(), "destination places");
    CUDA_OK(cudaMemcpyAsync(totals_dev, l->dest_totals.get(), 2 * kMaxWorld * sizeof(uint32_t), cudaMemcpyDeviceToDevice, st));
  });
}

MOE_API moe_status moe_layer_dispatch_rows_device(moe_layer *l, void *rows_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!rows_dev || l->last_T == 0 || !l->dest_world) throw BadArgument("rows are required, after moe_layer_dispatch_plan_device");
    need_aligned16({rows_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    const uint64_t pairs = (uint64_t)l->last_T * l->dest_world;
    k_dispatch_rows<<<(unsigned)((pairs + 7) / 8), 256, 0, st>>>(l->xq_routed.view(), l->E, l->xq_routed.q8k, l->ids.get(), l->w.get(),
                                                                l->dest_pos.get(), l->dest_totals.get(), l->last_T, l->K, l->local, l->dest_world,
                                                                (uint8_t *)rows_dev);
    launched(l, cudaGetLastError(), "rows by destination");
  });
}

MOE_API moe_status moe_layer_experts_partial_device(moe_layer *l, const void *rows_dev, uint32_t R, uint32_t assignments, void *y_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->local == l->NE) throw BadArgument("this layer holds every expert: use moe_layer_forward_device");
    if (R == 0) return;
    if (!rows_dev || !y_dev) throw BadArgument("rows and y are required");
    need_aligned16({rows_dev, y_dev});
    const uint64_t entries = (uint64_t)R * l->K;
    const uint64_t A = std::min<uint64_t>(assignments ? assignments : entries, entries);  // the rows' assignments: an upper bound will do
    if (entries > l->Rmax) throw BadArgument("more rows than max_expert_rows allows (rows x n_used entries)");
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    const uint32_t E = l->E, K = l->K, nexp = l->local;
    const bool q8k = l->xq_routed.q8k;
    const uint32_t wb = wire_row_bytes(q8k, E), wb2 = wb + kMetaBytes, tm = tensor_min_for(l, A);
    if (!l->w_local.get()) l->w_local.alloc(l->Rmax);
    const uint8_t *wire = (const uint8_t *)rows_dev;
    k_meta_unpack<<<(unsigned)((entries + 255) / 256), 256, 0, st>>>(wire, R, wb, K, l->cfg.expert_first, l->ids_local.get(), l->w_local.get());
    launched(l, cudaGetLastError(), "received lists");
    // Sort the entries by expert among this GPU's experts (entries with no expert fall out): row_src = the entry's row.
    PackBuffers &pk = l->pack_local;
    const uint32_t nchunks = (uint32_t)((entries + kLocalChunk - 1) / kLocalChunk);
    k_chunk_hist<<<nchunks, 256, 0, st>>>(l->ids_local.get(), (uint32_t)entries, kLocalChunk, nexp, l->cfg.expert_first, pk.chunk_hist.get());
    launched(l, cudaGetLastError(), "local counts");
    launch_pack(l, pk, PackJob{l->ids_local.get(), (uint32_t)entries, kLocalChunk, nchunks, l->cfg.expert_first, tm, tensor_budget_for(l, A),
                               group_cap(A, nexp), K}, st);
    const uint32_t dbytes = q8k ? E / 64 : E / 8;
    ActSource src{ActView{(const int8_t *)wire, (const float *)(wire + E), (const int16_t *)(wire + E + dbytes), wb2, wb2, wb2}, nullptr,
                  pk.row_src.get()};
    if (tm) {
      // The rows' f16 form straight to their places in expert order: a row is read once, as it came, and no copy of the
      // rows in their own order is made on the way.
      const uint64_t nblk = (uint64_t)R * (E / 256);
      k_wire_to_f16<<<(unsigned)((nblk + 7) / 8), 256, 0, st>>>(wire, E, q8k, nblk, l->xg.get(), wb2, l->ids_local.get(), pk.inv.get(), K, l->Rmax);
      launched(l, cudaGetLastError(), "wire rows to f16, in expert order");
    }
    l->last_pack = &pk;
    const bool y16 = results_f16(l, tm);
    stage_experts(l, src, pk, A, A, tm, l->y.get(), y16, st, 0, true);
    if (y16)
      k_combine_partial<__half><<<R, 256, 0, st>>>((const __half *)l->y.get(), pk.inv.get(), l->ids_local.get(), l->w_local.get(), K, E, (__half *)y_dev);
    else
      k_combine_partial<float><<<R, 256, 0, st>>>(l->y.get(), pk.inv.get(), l->ids_local.get(), l->w_local.get(), K, E, (__half *)y_dev);
    launched(l, cudaGetLastError(), "partial sums");
  });
}

MOE_API moe_status moe_layer_combine_partials_device(moe_layer *l, const void *back_dev, float *out_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!back_dev || !out_dev || l->last_T == 0 || !l->dest_world) throw BadArgument("the returned rows and out are required, after moe_layer_dispatch_plan_device");
    need_aligned16({back_dev, out_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    mark(l, ST_COMBINE, st);
    k_combine_home<<<l->last_T, 256, 0, st>>>((const __half *)back_dev, l->dest_pos.get(), l->dest_totals.get(), l->gs.get(),
                                             l->has_shared ? l->s.get() : nullptr, l->residual, l->dest_world, l->E, out_dev);
    launched(l, cudaGetLastError(), "combine of the GPUs' sums");
    mark(l, ST_COPIES, st);
    if (l->profile) l->ev[MOE_STAGES]->record(st), l->ev_valid = true;
  });
}

MOE_API moe_status moe_layer_shared_device(moe_layer *l, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("after moe_layer_route_device");
    stage_shared(l, l->last_T, stream ? (cudaStream_t)stream : l->stream->get());
  });
}

MOE_API moe_status moe_layer_combine_device(moe_layer *l, const void *y_dev, uint32_t y_f16, float *out_dev, void *stream) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!y_dev || !out_dev || l->last_T == 0) throw BadArgument("y and out are required, after moe_layer_route_device");
    need_aligned16({y_dev, out_dev});
    cudaStream_t st = stream ? (cudaStream_t)stream : l->stream->get();
    if (y_f16)
      stage_combine<__half>(l, (const __half *)y_dev, l->last_T, out_dev, st);
    else
      stage_combine<float>(l, (const float *)y_dev, l->last_T, out_dev, st);
    if (l->profile) l->ev[MOE_STAGES]->record(st), l->ev_valid = true;
  });
}

MOE_API moe_status moe_layer_read_config(const moe_layer *l, moe_layer_config *out) {
  if (!l || !out) return MOE_BAD_ARGUMENT;
  *out = l->cfg;
  out->expert_count = l->local, out->max_tokens = l->Tmax, out->max_expert_rows = (uint32_t)std::min<uint64_t>(l->Rmax, 0xFFFFFFFFu);
  return MOE_OK;
}

MOE_API moe_status moe_layer_sync(moe_layer *l, uint32_t timeout_ms) {
  if (!l) return MOE_BAD_ARGUMENT;
  return guarded(l, [&] {
    l->stream->wait(timeout_ms);
    check_device_error(l);
  });
}

MOE_API moe_status moe_layer_read_route(moe_layer *l, int32_t *ids, float *w, uint32_t *inv, moe_tile *tiles, uint32_t tiles_cap,
                                        uint32_t *ntiles) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("no call has run yet");
    cudaStream_t st = l->stream->get();
    const size_t A = (size_t)l->last_T * l->K;
    uint32_t counters[8];
    CUDA_OK(cudaMemcpyAsync(counters, l->pack.counters.get(), sizeof(counters), cudaMemcpyDeviceToHost, st));
    if (ids) CUDA_OK(cudaMemcpyAsync(ids, l->ids.get(), A * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    if (w) CUDA_OK(cudaMemcpyAsync(w, l->w.get(), A * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (inv) CUDA_OK(cudaMemcpyAsync(inv, l->pack.inv.get(), A * sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    l->stream->wait(0);
    if (tiles && tiles_cap) {
      static_assert(sizeof(moe_tile) == sizeof(MoeTile), "tile layout");
      const size_t n = std::min<size_t>(tiles_cap, counters[0]);
      CUDA_OK(cudaMemcpyAsync(tiles, l->pack.tiles.get(), n * sizeof(moe_tile), cudaMemcpyDeviceToHost, st));
      l->stream->wait(0);
    }
    if (ntiles) *ntiles = counters[0];
    read_counters(l);
  });
}

MOE_API moe_status moe_layer_read_groups(moe_layer *l, moe_group *groups, uint32_t cap, uint32_t *ngroups) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("no call has run yet");
    static_assert(sizeof(moe_group) == sizeof(MoeGroup), "group layout");
    l->stream->wait(0);
    uint32_t counters[8];
    CUDA_OK(cudaMemcpy(counters, l->pack.counters.get(), sizeof(counters), cudaMemcpyDeviceToHost));
    if (groups && cap)
      CUDA_OK(cudaMemcpy(groups, l->pack.groups.get(), std::min<size_t>(cap, counters[1]) * sizeof(moe_group), cudaMemcpyDeviceToHost));
    if (ngroups) *ngroups = counters[1];
  });
}

MOE_API moe_status moe_layer_read_quantized(moe_layer *l, uint32_t which, int8_t *codes, float *scales, int16_t *sums, uint32_t *is_q8k) {
  if (!l || which > 1) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("no call has run yet");
    if (which == 1 && l->local != l->NE) throw BadArgument("an expert-parallel layer's inner rows are those of the rows it received");
    l->stream->wait(0);
    const ActBuffers &b = which == 0 ? l->xq_routed : l->hq_routed;
    const uint64_t rows = which == 0 ? l->last_T : (uint64_t)l->last_T * l->K;
    if (codes) CUDA_OK(cudaMemcpy(codes, b.q.get(), rows * b.K, cudaMemcpyDeviceToHost));
    if (scales) CUDA_OK(cudaMemcpy(scales, b.d.get(), rows * (b.q8k ? b.K / 256 : b.K / 32) * sizeof(float), cudaMemcpyDeviceToHost));
    if (sums && b.q8k) CUDA_OK(cudaMemcpy(sums, b.bs.get(), rows * (b.K / 16) * sizeof(int16_t), cudaMemcpyDeviceToHost));
    if (is_q8k) *is_q8k = b.q8k;
  });
}

MOE_API moe_status moe_layer_read_logits(moe_layer *l, float *logits, uint32_t *approximate, float *eps_rel, float *eps_abs) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T == 0) throw BadArgument("no call has run yet");
    l->stream->wait(0);
    const bool approx = l->router_tensor && l->last_T > kRouterExactRows;
    if (logits) {
      if (approx)
        CUDA_OK(cudaMemcpy(logits, l->approx.get(), (size_t)l->last_T * l->NE * sizeof(float), cudaMemcpyDeviceToHost));
      else
        CUDA_OK(cudaMemcpy2D(logits, l->NE * sizeof(float), l->rl.get(), l->N * sizeof(float), l->NE * sizeof(float), l->last_T,
                             cudaMemcpyDeviceToHost));
    }
    if (approximate) *approximate = approx;
    if (eps_rel) *eps_rel = approx ? l->router_eps_rel : 0.0f;
    if (eps_abs) *eps_abs = approx ? l->router_eps_abs : 0.0f;
  });
}

MOE_API moe_status moe_layer_read_stats(moe_layer *l, moe_layer_stats *out) {
  if (!l || !out) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (l->last_T) {
      l->stream->wait(0);
      read_counters(l);
    }
    *out = l->stats;
  });
}

MOE_API moe_status moe_layer_stage_ms(moe_layer *l, float *ms) {
  if (!l || !ms) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    if (!l->profile || !l->ev_valid) throw BadArgument("the layer was not created with MOE_FLAG_PROFILE, or no call has run");
    CUDA_OK(cudaEventSynchronize(l->ev[MOE_STAGES]->get()));
    for (int i = 0; i < MOE_STAGES; i++) ms[i] = Event::ms(*l->ev[i], *l->ev[i + 1]);
  });
}

MOE_API moe_status moe_layer_set_profiling(moe_layer *l, uint32_t on) {
  if (!l) return MOE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(l->mu);
  return guarded(l, [&] {
    l->stream->wait(0);
    l->profile = on != 0, l->ev_valid = false;
  });
}

MOE_API void *moe_layer_stream(moe_layer *l) { return l ? (void *)l->stream->get() : nullptr; }

MOE_API const char *moe_last_error(const moe_layer *l) { return l ? l->err.c_str() : g_create_error.c_str(); }

MOE_API moe_status moe_to_runs(uint32_t type, const void *file_blocks, uint64_t nblocks, void *dst) {
  if (!type_known(type) || !file_blocks || !dst) return MOE_BAD_ARGUMENT;
  to_runs(type, (const uint8_t *)file_blocks, nblocks, (uint8_t *)dst);
  return MOE_OK;
}

MOE_API moe_status moe_from_runs(uint32_t type, const void *runs, uint64_t nblocks, void *dst) {
  if (!type_known(type) || !runs || !dst) return MOE_BAD_ARGUMENT;
  from_runs(type, (const uint8_t *)runs, nblocks, (uint8_t *)dst);
  return MOE_OK;
}

MOE_API uint32_t moe_abi_layout(moe_abi_row *table, uint32_t cap) {
  static const moe_abi_row rows[] = {
#define ROW(S, F) {#S "." #F, (uint32_t)offsetof(S, F), (uint32_t)sizeof(((S *)0)->F)}
      ROW(moe_layer_config, n_embd), ROW(moe_layer_config, n_ff), ROW(moe_layer_config, n_experts), ROW(moe_layer_config, n_used),
      ROW(moe_layer_config, gate_type), ROW(moe_layer_config, down_type), ROW(moe_layer_config, shexp_gate_type),
      ROW(moe_layer_config, shexp_down_type), ROW(moe_layer_config, expert_first), ROW(moe_layer_config, expert_count),
      ROW(moe_layer_config, max_tokens), ROW(moe_layer_config, device), ROW(moe_layer_config, swiglu_limit), ROW(moe_layer_config, flags),
      ROW(moe_layer_config, tensor_min_rows), ROW(moe_layer_config, max_expert_rows), ROW(moe_layer_config, host_chunk_rows),
      ROW(moe_layer_weights, router), ROW(moe_layer_weights, shexp_gate_inp), ROW(moe_layer_weights, router_bias),
      ROW(moe_layer_weights, gate_exps), ROW(moe_layer_weights, up_exps), ROW(moe_layer_weights, down_exps),
      ROW(moe_layer_weights, gate_shexp), ROW(moe_layer_weights, up_shexp), ROW(moe_layer_weights, down_shexp),
      ROW(moe_tile, expert), ROW(moe_tile, slot), ROW(moe_tile, start), ROW(moe_tile, count),
      ROW(moe_layer_stats, calls), ROW(moe_layer_stats, rows), ROW(moe_layer_stats, assignments), ROW(moe_layer_stats, kernels),
      ROW(moe_layer_stats, h2d_bytes), ROW(moe_layer_stats, d2h_bytes), ROW(moe_layer_stats, last_tiles),
      ROW(moe_layer_stats, last_experts_hit), ROW(moe_layer_stats, last_tensor_rows),
      ROW(moe_group, slot), ROW(moe_group, start), ROW(moe_group, n),
      ROW(moe_gguf_tensor, name), ROW(moe_gguf_tensor, type), ROW(moe_gguf_tensor, n_dims), ROW(moe_gguf_tensor, shape),
      ROW(moe_gguf_tensor, offset), ROW(moe_gguf_tensor, bytes),
      ROW(moe_abi_row, name), ROW(moe_abi_row, offset), ROW(moe_abi_row, size),
#undef ROW
      {"moe_layer_config", 0, (uint32_t)sizeof(moe_layer_config)},
      {"moe_layer_weights", 0, (uint32_t)sizeof(moe_layer_weights)},
      {"moe_tile", 0, (uint32_t)sizeof(moe_tile)},
      {"moe_group", 0, (uint32_t)sizeof(moe_group)},
      {"moe_gguf_tensor", 0, (uint32_t)sizeof(moe_gguf_tensor)},
      {"moe_layer_stats", 0, (uint32_t)sizeof(moe_layer_stats)},
      {"moe_abi_row", 0, (uint32_t)sizeof(moe_abi_row)},
  };
  const uint32_t n = (uint32_t)(sizeof(rows) / sizeof(rows[0]));
  if (table)
    for (uint32_t i = 0; i < n && i < cap; i++) table[i] = rows[i];
  return n;
}

}  // extern "C"
