// File blocks -> the runs layout the kernels read, on the host (the role of the reference's core/load/runs.cpp:12-41).
#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>
#include <vector>

#include "formats.h"

namespace moe {

void to_runs(uint32_t t, const uint8_t *src, uint64_t n, uint8_t *dst) {
  const uint32_t bb = block_bytes(t), nf = nfields(t);
  for (uint32_t f = 0; f < nf; f++) {
    const Field fd = field(t, f);
    uint8_t *run = dst + run_offset(t, f, n);
    const uint8_t *from = src + fd.offset;
    for (uint64_t k = 0; k < n; k++) std::memcpy(run + k * fd.size, from + k * bb, fd.size);
  }
}

void from_runs(uint32_t t, const uint8_t *src, uint64_t n, uint8_t *dst) {
  const uint32_t bb = block_bytes(t), nf = nfields(t);
  for (uint32_t f = 0; f < nf; f++) {
    const Field fd = field(t, f);
    const uint8_t *run = src + run_offset(t, f, n);
    for (uint64_t k = 0; k < n; k++) std::memcpy(dst + k * bb + fd.offset, run + k * fd.size, fd.size);
  }
}

void to_runs_slices(uint32_t t, const uint8_t *src, uint64_t n, uint64_t nslices, uint8_t *dst, unsigned threads) {
  const uint64_t sb = n * block_bytes(t);
  threads = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(threads, nslices));
  std::atomic<uint64_t> next{0};
  auto work = [&] {
    for (uint64_t s; (s = next.fetch_add(1)) < nslices;) to_runs(t, src + s * sb, n, dst + s * sb);
  };
  std::vector<std::thread> pool;
  for (unsigned i = 1; i < threads; i++) pool.emplace_back(work);
  work();
  for (auto &th : pool) th.join();
}

}  // namespace moe
