// The thin device layer under the MoE layer: one device's buffers, streams and events, with every
// CUDA error turned into an exception the C ABI catches. It stands where the reference has core/ze (Runtime, List,
// EventPool: core/ze/ze.h:50-217) and offers only what this path uses. Waits are polls against a deadline, never an
// unbounded synchronise (the reference's list timeout, core/ze/ze.cpp:549-560).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <thread>

namespace moe {

struct CudaFailure : std::runtime_error {
  cudaError_t code;
  CudaFailure(cudaError_t c, const std::string &what) : std::runtime_error(what), code(c) {}
};
struct Timeout : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct BadArgument : std::runtime_error {
  using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t e, const char *what, const char *file, int line) {
  if (e != cudaSuccess)
    throw CudaFailure(e, std::string(what) + ": " + cudaGetErrorString(e) + " (" + file + ":" + std::to_string(line) + ")");
}
#define CUDA_OK(call) ::moe::cuda_check((call), #call, __FILE__, __LINE__)

// What a launch helper needs to know about the device it launches on; the layer finds it once, at create.
struct LaunchCtx {
  int device = 0;
  uint32_t sms = 148;
  bool pdl = false;  // launch-bound steps: kernels are launched as programmatic dependents of the one before (launch_kernel)
};

#if defined(__CUDACC__)
// For kernels that may be launched as programmatic dependents: the first lets the kernel after this one be scheduled
// (it then waits where this one waits), the second waits until the kernels before have completed and their writes are
// visible. Both do nothing in a kernel launched the ordinary way. They stand at a kernel's top, before it reads or
// writes anything another kernel touches.
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_predecessors() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// kernel<<<grid, block, smem, st>>>(args...), as a programmatic dependent of the stream's last kernel when pdl is set:
// it may be scheduled while that kernel still runs, which takes the launch's latency out of a chain of short kernels.
template <class... KArgs, class... Args>
inline cudaError_t launch_kernel(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute at{};
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = pdl ? &at : nullptr, cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// A kernel's opt-in to more than 48 KB of dynamic shared memory holds per device: `done` has a bit per device ordinal
// (one static word per kernel instantiation), so the attribute is set on a kernel's first launch on a device and not
// again. Ordinals past 31 set it every time.
template <class Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, size_t bytes, std::atomic<uint32_t> &done, int device) {
  const uint32_t bit = device >= 0 && device < 32 ? 1u << device : 0u;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && bit) done.fetch_or(bit, std::memory_order_release);
  return e;
}

// Device memory of n elements of T, freed with its owner.
template <class T>
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  DeviceBuffer(const DeviceBuffer &) = delete;
  DeviceBuffer &operator=(const DeviceBuffer &) = delete;
  DeviceBuffer(DeviceBuffer &&o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr, o.n_ = 0; }
  ~DeviceBuffer() { release(); }
  void alloc(size_t n) {
    release();
    if (n == 0) return;
    CUDA_OK(cudaMalloc((void **)&p_, n * sizeof(T)));
    n_ = n;
  }
  void release() {
    if (p_) cudaFree(p_);
    p_ = nullptr, n_ = 0;
  }
  T *get() const { return p_; }
  size_t size() const { return n_; }
  size_t bytes() const { return n_ * sizeof(T); }

 private:
  T *p_ = nullptr;
  size_t n_ = 0;
};

class Stream {
 public:
  Stream() { CUDA_OK(cudaStreamCreateWithFlags(&s_, cudaStreamNonBlocking)); }
  Stream(const Stream &) = delete;
  ~Stream() {
    if (s_) cudaStreamDestroy(s_);
  }
  cudaStream_t get() const { return s_; }
  // Waits until the stream's work is done, polling; throws Timeout after timeout_ms.
  void wait(uint32_t timeout_ms) const { wait_on(s_, timeout_ms); }
  static void wait_on(cudaStream_t s, uint32_t timeout_ms) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms ? timeout_ms : 60000);
    for (unsigned spins = 0;; spins++) {
      const cudaError_t e = cudaStreamQuery(s);
      if (e == cudaSuccess) return;
      if (e != cudaErrorNotReady) cuda_check(e, "cudaStreamQuery", __FILE__, __LINE__);
      if (std::chrono::steady_clock::now() > deadline) throw Timeout("the stream's work did not finish in time");
      if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }

 private:
  cudaStream_t s_ = nullptr;
};

class Event {
 public:
  Event() { CUDA_OK(cudaEventCreate(&e_)); }
  Event(const Event &) = delete;
  ~Event() {
    if (e_) cudaEventDestroy(e_);
  }
  void record(cudaStream_t s) { CUDA_OK(cudaEventRecord(e_, s)); }
  cudaEvent_t get() const { return e_; }
  static float ms(const Event &a, const Event &b) {
    float v = 0;
    CUDA_OK(cudaEventElapsedTime(&v, a.e_, b.e_));
    return v;
  }

 private:
  cudaEvent_t e_ = nullptr;
};

}  // namespace moe
