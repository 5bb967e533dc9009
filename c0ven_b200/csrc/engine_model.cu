// The MoE-only model of the engine ABI (engine_model.h): embedding rows in, a stack of x <- x + moe_l(rmsnorm_l(x)) over
// the layers of include/moe_layer.h, greedy next tokens out. The kernels here are the little there is around the
// layers: the embedding gather, the RMS norm in front of each layer, and the arg-max over the vocabulary for the rows
// that end a run.
#include "engine_model.h"

#include <cuda_runtime.h>

#include <cmath>
#include <stdexcept>

#include "cuda_rt.h"
#include "gguf_file.h"
#include "moe_layer.h"

namespace moe {

namespace {

// x[r] = embd[tokens[r]]: one CTA per row, 16 bytes a thread.
__global__ void __launch_bounds__(256) k_embed_rows(const int32_t *__restrict__ tokens, const float *__restrict__ embd, uint32_t E,
                                                    float *__restrict__ x) {
  const uint64_t r = blockIdx.x;
  const float4 *src = (const float4 *)(embd + (uint64_t)tokens[r] * E);
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) ((float4 *)(x + r * E))[i] = __ldg(src + i);
}

// out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * g (g null: 1). One CTA of 256 threads per row.
__global__ void __launch_bounds__(256) k_rmsnorm(const float *__restrict__ x, const float *__restrict__ g, uint32_t E, float eps,
                                                 float *__restrict__ out) {
  __shared__ float part[8];
  const uint64_t r = blockIdx.x;
  const float4 *row = (const float4 *)(x + r * E);
  float s = 0.0f;
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    const float4 v = row[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (threadIdx.x % 32 == 0) part[threadIdx.x / 32] = s;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) tot += part[i];
  const float k = rsqrtf(tot / (float)E + eps);
  for (uint32_t i = threadIdx.x; i < E / 4; i += 256) {
    float4 v = row[i];
    const float4 w = g ? __ldg((const float4 *)g + i) : make_float4(1, 1, 1, 1);
    v.x *= k * w.x, v.y *= k * w.y, v.z *= k * w.z, v.w *= k * w.w;
    ((float4 *)(out + r * E))[i] = v;
  }
}

// The largest of W[v] . x[want[j]] over a chunk of kVocabChunk vocabulary rows, for every wanted row j: grid
// (chunks, wanted rows), a warp a vocabulary row at a time. best[j][chunk] = (value, id), ties to the lower id.
constexpr uint32_t kVocabChunk = 64;
__global__ void __launch_bounds__(256) k_vocab_best(const float *__restrict__ x, const uint32_t *__restrict__ want, const float *__restrict__ W,
                                                    uint32_t vocab, uint32_t E, float2 *__restrict__ best) {
  __shared__ float bv[8];
  __shared__ uint32_t bi[8];
  const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, v0 = blockIdx.x * kVocabChunk;
  const float4 *row = (const float4 *)(x + (uint64_t)want[blockIdx.y] * E);
  float mine = -INFINITY;
  uint32_t at = 0xFFFFFFFFu;
  for (uint32_t v = v0 + warp; v < min(v0 + kVocabChunk, vocab); v += 8) {
    const float4 *w = (const float4 *)(W + (uint64_t)v * E);
    float s = 0.0f;
    for (uint32_t i = lane; i < E / 4; i += 32) {
      const float4 a = row[i], b = __ldg(w + i);
      s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (s > mine || at == 0xFFFFFFFFu) mine = s, at = v;  // v ascends: a later equal value does not replace
  }
  if (lane == 0) bv[warp] = mine, bi[warp] = at;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = bv[0];
    uint32_t a = bi[0];
    for (int i = 1; i < 8; i++)
      if (bi[i] != 0xFFFFFFFFu && (a == 0xFFFFFFFFu || bv[i] > m || (bv[i] == m && bi[i] < a))) m = bv[i], a = bi[i];
    best[(uint64_t)blockIdx.y * gridDim.x + blockIdx.x] = make_float2(m, __uint_as_float(a));
  }
}

__global__ void __launch_bounds__(32) k_vocab_pick(const float2 *__restrict__ best, uint32_t chunks, int32_t *__restrict__ next) {
  const float2 *b = best + (uint64_t)blockIdx.x * chunks;
  float m = -INFINITY;
  uint32_t a = 0xFFFFFFFFu;
  for (uint32_t c = threadIdx.x; c < chunks; c += 32) {
    const uint32_t id = __float_as_uint(b[c].y);
    if (id != 0xFFFFFFFFu && (a == 0xFFFFFFFFu || b[c].x > m || (b[c].x == m && id < a))) m = b[c].x, a = id;
  }
  for (int off = 16; off > 0; off >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, off);
    const uint32_t oa = __shfl_xor_sync(0xffffffffu, a, off);
    if (oa != 0xFFFFFFFFu && (a == 0xFFFFFFFFu || om > m || (om == m && oa < a))) m = om, a = oa;
  }
  if (threadIdx.x == 0) next[blockIdx.x] = (int32_t)a;
}

std::vector<float> optional_vector(const GgufFile &g, const std::string &name, uint64_t n) {
  const GgufTensorInfo *t = g.find(name);
  if (!t) return {};
  if (!t->data || t->elements() != n) throw std::runtime_error(name + " is not a vector of " + std::to_string(n) + " values");
  return gguf_to_f32(*t);
}

}  // namespace

struct EngineModel::Buffers {
  Stream stream;
  DeviceBuffer<float> embd, out_w, out_norm, x, xn;
  std::vector<DeviceBuffer<float>> norms;  // one per layer; empty: no weight
  DeviceBuffer<int32_t> tokens, next;
  DeviceBuffer<uint32_t> want;
  DeviceBuffer<float2> best;
  int32_t *h_tokens = nullptr, *h_next = nullptr;  // pinned
  uint32_t *h_want = nullptr;
  uint32_t last_rows = 0;
  ~Buffers() {
    if (h_tokens) cudaFreeHost(h_tokens);
    if (h_next) cudaFreeHost(h_next);
    if (h_want) cudaFreeHost(h_want);
  }
};

EngineModel::EngineModel(const std::string &path, int device, uint32_t max_rows) : device_(device), max_rows_(max_rows) {
  CUDA_OK(cudaSetDevice(device));
  size_t free0 = 0, total = 0;
  CUDA_OK(cudaMemGetInfo(&free0, &total));
  if (moe_gguf_open(path.c_str(), &file_) != MOE_OK) throw std::runtime_error(moe_last_error(nullptr));
  try {
    GgufFile g(path);  // a second, short-lived view for the tensors the layers do not take
    const uint32_t nl = moe_gguf_layers(file_);
    if (nl == 0) throw std::runtime_error("the file does not say how many blocks it has (<architecture>.block_count)");
    const GgufTensorInfo &te = g.tensor("token_embd.weight");
    if (te.shape.size() != 2) throw std::runtime_error("token_embd.weight is not a matrix");
    n_embd_ = (uint32_t)te.shape[0], vocab_ = (uint32_t)te.shape[1];
    norm_eps_ = (float)g.get_float(g.get_string("general.architecture") + ".attention.layer_norm_rms_epsilon", 1e-6);
    buf_ = std::make_unique<Buffers>();
    cudaStream_t st = buf_->stream.get();
    auto upload = [&](DeviceBuffer<float> &dst, const std::vector<float> &v) {
      dst.alloc(v.size());
      CUDA_OK(cudaMemcpyAsync(dst.get(), v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice, st));
      CUDA_OK(cudaStreamSynchronize(st));
    };
    upload(buf_->embd, gguf_to_f32(te));
    if (const GgufTensorInfo *ow = g.find("output.weight")) {
      if (!ow->data || ow->shape.size() != 2 || ow->shape[0] != n_embd_ || ow->shape[1] != vocab_)
        throw std::runtime_error("output.weight does not have token_embd's shape");
      upload(buf_->out_w, gguf_to_f32(*ow));
    }
    const std::vector<float> on = optional_vector(g, "output_norm.weight", n_embd_);
    if (!on.empty()) upload(buf_->out_norm, on);
    buf_->norms.resize(nl);
    for (uint32_t i = 0; i < nl; i++) {
      moe_layer_config c{};
      c.max_tokens = max_rows, c.device = device;
      moe_layer *l = nullptr;
      if (moe_layer_create_from_gguf(file_, i, &c, &l) != MOE_OK) throw std::runtime_error("layer " + std::to_string(i) + ": " + moe_last_error(nullptr));
      layers_.push_back(l);
      moe_layer_config got{};
      moe_layer_read_config(l, &got);
      if (got.n_embd != n_embd_) throw std::runtime_error("layer " + std::to_string(i) + " is not as wide as token_embd");
      n_experts_ = got.n_experts;
      const std::vector<float> nw = optional_vector(g, "blk." + std::to_string(i) + ".ffn_norm.weight", n_embd_);
      if (!nw.empty()) upload(buf_->norms[i], nw);
    }
    buf_->x.alloc((size_t)max_rows * n_embd_), buf_->xn.alloc((size_t)max_rows * n_embd_);
    buf_->tokens.alloc(max_rows), buf_->next.alloc(max_rows), buf_->want.alloc(max_rows);
    buf_->best.alloc((size_t)max_rows * ((vocab_ + kVocabChunk - 1) / kVocabChunk));
    CUDA_OK(cudaMallocHost((void **)&buf_->h_tokens, max_rows * sizeof(int32_t)));
    CUDA_OK(cudaMallocHost((void **)&buf_->h_next, max_rows * sizeof(int32_t)));
    CUDA_OK(cudaMallocHost((void **)&buf_->h_want, max_rows * sizeof(uint32_t)));
    size_t free1 = 0;
    CUDA_OK(cudaMemGetInfo(&free1, &total));
    device_bytes_ = free0 > free1 ? free0 - free1 : 0;
  } catch (...) {
    for (moe_layer *l : layers_) moe_layer_destroy(l);
    layers_.clear();
    buf_.reset();
    moe_gguf_close(file_);
    throw;
  }
}

EngineModel::~EngineModel() {
  cudaSetDevice(device_);
  if (buf_) cudaStreamSynchronize(buf_->stream.get());
  for (moe_layer *l : layers_) moe_layer_destroy(l);
  buf_.reset();
  moe_gguf_close(file_);
}

void EngineModel::batch(const int32_t *tokens, uint32_t rows, const uint32_t *want, uint32_t nwant, int32_t *next, uint32_t timeout_ms) {
  if (rows == 0 || rows > max_rows_ || nwant > rows) throw BadArgument("a batch holds 1 .. max_rows rows");
  CUDA_OK(cudaSetDevice(device_));
  Buffers &b = *buf_;
  cudaStream_t st = b.stream.get();
  for (uint32_t r = 0; r < rows; r++) {
    if (tokens[r] < 0 || (uint32_t)tokens[r] >= vocab_) throw BadArgument("a token is outside the vocabulary");
    b.h_tokens[r] = tokens[r];
  }
  for (uint32_t i = 0; i < nwant; i++) b.h_want[i] = want[i];
  CUDA_OK(cudaMemcpyAsync(b.tokens.get(), b.h_tokens, rows * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  if (nwant) CUDA_OK(cudaMemcpyAsync(b.want.get(), b.h_want, nwant * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
  k_embed_rows<<<rows, 256, 0, st>>>(b.tokens.get(), b.embd.get(), n_embd_, b.x.get());
  CUDA_OK(cudaGetLastError());
  for (size_t i = 0; i < layers_.size(); i++) {
    k_rmsnorm<<<rows, 256, 0, st>>>(b.x.get(), b.norms[i].get(), n_embd_, norm_eps_, b.xn.get());
    CUDA_OK(cudaGetLastError());
    if (moe_layer_forward_residual_device(layers_[i], b.xn.get(), rows, b.x.get(), b.x.get(), st) != MOE_OK)
      throw std::runtime_error("layer " + std::to_string(i) + ": " + moe_last_error(layers_[i]));
  }
  b.last_rows = rows;
  if (nwant) {
    // The rows that end a run: the output norm, when the file has one, then the product with the output matrix (the
    // embedding itself when the file has no output.weight) and its arg-max.
    const float *h = b.x.get();
    if (b.out_norm.get()) {
      // Only the wanted rows matter, but norming every row keeps the kernel simple and rows are few against a layer's work.
      k_rmsnorm<<<rows, 256, 0, st>>>(b.x.get(), b.out_norm.get(), n_embd_, norm_eps_, b.xn.get());
      CUDA_OK(cudaGetLastError());
      h = b.xn.get();
    }
    const uint32_t chunks = (vocab_ + kVocabChunk - 1) / kVocabChunk;
    k_vocab_best<<<dim3(chunks, nwant), 256, 0, st>>>(h, b.want.get(), b.out_w.get() ? b.out_w.get() : b.embd.get(), vocab_, n_embd_, b.best.get());
    CUDA_OK(cudaGetLastError());
    k_vocab_pick<<<nwant, 32, 0, st>>>(b.best.get(), chunks, b.next.get());
    CUDA_OK(cudaGetLastError());
    CUDA_OK(cudaMemcpyAsync(b.h_next, b.next.get(), nwant * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  }
  b.stream.wait(timeout_ms);
  for (moe_layer *l : layers_)
    if (moe_layer_sync(l, timeout_ms) == MOE_TIMEOUT) throw Timeout(moe_last_error(l));
  for (uint32_t i = 0; i < nwant; i++) next[i] = b.h_next[i];
}

void EngineModel::read_hidden(float *dst, uint32_t rows) const {
  CUDA_OK(cudaSetDevice(device_));
  if (rows > buf_->last_rows) throw BadArgument("more rows than the last batch had");
  CUDA_OK(cudaMemcpy(dst, buf_->x.get(), (size_t)rows * n_embd_ * sizeof(float), cudaMemcpyDeviceToHost));
}

uint64_t EngineModel::kernels() const {
  uint64_t n = 0;
  for (moe_layer *l : layers_) {
    moe_layer_stats s{};
    if (moe_layer_read_stats(l, &s) == MOE_OK) n += s.kernels;
  }
  return n;
}

}  // namespace moe

extern "C" {

MOE_API moe_status moe_rmsnorm_rows_device(const float *x_dev, const float *weight_dev, uint32_t T, uint32_t n_embd, float eps, float *out_dev,
                                           void *stream) {
  if (!x_dev || !out_dev || T == 0 || n_embd == 0 || n_embd % 4 || (((uintptr_t)x_dev | (uintptr_t)out_dev | (uintptr_t)weight_dev) & 15))
    return MOE_BAD_ARGUMENT;
  moe::k_rmsnorm<<<T, 256, 0, (cudaStream_t)stream>>>(x_dev, weight_dev, n_embd, eps, out_dev);
  return cudaGetLastError() == cudaSuccess ? MOE_OK : MOE_ERROR;
}

}  // extern "C"
