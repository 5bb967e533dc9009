// moe_route_rows_static: the router for a few rows with no allocation anywhere on the way. Some callers of this
// library may not allocate when they route a step: an engine whose device memory was all shared out at load by a
// memory plan, so that nothing is left to ask for and asking could fail in the middle of a step; and a step loop that
// must never take the device-wide wait the allocator can bring. For them the scratch the router needs between its two
// kernels (the rows' logits, and the per-chunk expert counts its top-k kernel leaves) lives in one file-scope device
// array of fixed size, which every GPU that loads this library holds until the process ends.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "moe_layer.h"
#include "route_kernels.cuh"

using namespace moe;

namespace {

constexpr uint32_t kStaticRows = MOE_ROUTE_STATIC_MAX_ROWS, kStaticExperts = 512, kStaticEmbd = 4096;
constexpr uint32_t kLogitFloats = kStaticRows * (kStaticExperts + 1);
constexpr uint32_t kHistWords = ((kStaticRows + kChunkTokens - 1) / kChunkTokens) * kStaticExperts;

// The scratch: logits [rows][experts + 1], then the chunks' counts. About 136 KB per GPU. In host code this name is
// only a handle for the runtime; the kernels get the address cudaGetSymbolAddress gives for the current device.
static __device__ __align__(256) float g_route_scratch[kLogitFloats + kHistWords];

constexpr int kMaxDevices = 64;
float *g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mu;
thread_local std::string g_error;

// Once per device, with that device current: the scratch's device address, and the logits kernel's opt-in to the
// shared memory it needs. Neither allocates.
cudaError_t setup(int device, float **out) {
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_ptr[device]) {
    float *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void **)&p, g_route_scratch);
    if (e != cudaSuccess) return e;
    const int smem = (int)((size_t)8 * kRouterPieces * (kStaticEmbd / kRouterPieces + 4) * sizeof(float));
    e = cudaFuncSetAttribute(k_router_logits_rows<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[device] = p;
  }
  *out = g_scratch_ptr[device];
  return cudaSuccess;
}

moe_status fail(moe_status s, const std::string &m) {
  g_error = m;
  return s;
}

}  // namespace

extern "C" {

MOE_API const char *moe_route_rows_static_error(void) { return g_error.c_str(); }

MOE_API moe_status moe_route_rows_static(const float *x_dev, uint32_t T, uint32_t n_embd, const float *router_dev,
                                         const float *bias_dev, uint32_t n_experts, uint32_t n_used, int32_t *ids_dev,
                                         float *w_dev, float *gate_dev, void *stream) {
  if (!x_dev || !router_dev || !ids_dev || !w_dev || !gate_dev) return fail(MOE_BAD_ARGUMENT, "x, router, ids, w and gate are required");
  if (((uintptr_t)x_dev | (uintptr_t)router_dev) & 15)
    return fail(MOE_BAD_ARGUMENT, "x and router must be 16-byte aligned: the kernels read them through 16-byte loads");
  if (T == 0 || T > kStaticRows)
    return fail(MOE_BAD_ARGUMENT, "rows must be 1 .. " + std::to_string(kStaticRows) + ": the static scratch holds no more");
  if (n_experts == 0 || n_experts % 32 || n_experts > kStaticExperts)
    return fail(MOE_BAD_ARGUMENT, "n_experts must be a multiple of 32, at most " + std::to_string(kStaticExperts));
  if (n_embd == 0 || n_embd % 256 || n_embd > kStaticEmbd)
    return fail(MOE_BAD_ARGUMENT, "n_embd must be a multiple of 256, at most " + std::to_string(kStaticEmbd));
  if (n_used == 0 || n_used > 16 || n_used > n_experts) return fail(MOE_BAD_ARGUMENT, "n_used must be 1 .. 16 and at most n_experts");
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess && device >= kMaxDevices) return fail(MOE_BAD_ARGUMENT, "device ordinal past the table");
  float *scratch = nullptr;
  if (e == cudaSuccess) e = setup(device, &scratch);
  if (e != cudaSuccess) return fail(MOE_ERROR, std::string("set-up failed: ") + cudaGetErrorString(e));

  cudaStream_t st = (cudaStream_t)stream;
  const uint32_t N = n_experts + 1;
  float *rl = scratch;
  uint32_t *hist = (uint32_t *)(scratch + kLogitFloats);
  // Both regions are written in full for the rows of this call before they are read (every logit of rows < T; every
  // expert's count of every chunk), so the last call's contents need no clearing.
  const size_t smem = (size_t)8 * kRouterPieces * (n_embd / kRouterPieces + 4) * sizeof(float);
  k_router_logits_rows<8><<<dim3((N + 3) / 4, (T + 7) / 8), 32, smem, st>>>(x_dev, T, n_embd, router_dev, N, bias_dev, n_experts, rl);
  const uint32_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  k_router_topk<<<nchunks, 32 * kChunkTokens, 0, st>>>(rl, RouterApprox{}, nullptr, T, n_experts, n_used, ids_dev, w_dev, gate_dev, hist);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(MOE_ERROR, std::string("launch failed: ") + cudaGetErrorString(e));
  return MOE_OK;
}

}  // extern "C"
