// The twenty engine_* symbols of include/engine_abi.h over the MoE-only model (engine_model.h). The shape is the
// reference's (core/api/engine_api.cpp): callers queue plans; one engine thread runs them in order and is the only
// thread that touches the GPU while a plan may run (docs/adr/0077-one-thread-uses-the-cards.md); events and timing
// records are read by snapshot. What differs is the hand-off to the device: a plan's prompt pieces and decode rows
// become ONE packed ragged batch with a run table, one device program, where the reference runs windows, a chunk and
// a step one after another (engine_api.cpp:651-931).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "cuda_rt.h"
#include "engine_abi.h"
#include "engine_model.h"

using namespace moe;

namespace {

constexpr int32_t kNoToken = -1;
constexpr size_t kMaxQueuedPlans = 64, kTimingRing = 4096;
constexpr uint32_t kStepTimeoutMs = 60000;
std::atomic<int> g_stuck{0};
thread_local std::string g_open_error;

uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Slot {
  bool used = false, done = false;
  engine_settings settings{};
  std::vector<int32_t> prompt, tokens;  // tokens: what the slot has been fed so far, prompt included
  uint32_t fed = 0, generated = 0;
  int32_t next = kNoToken;
  engine_slot_stats stats{};
};

struct Checkpoint {
  bool full = false;
  std::vector<int32_t> tokens;
};

struct Plan {
  engine_step_plan p{};
  std::vector<engine_page_change> pages;
};

}  // namespace

struct engine_ctx {
  engine_config config{};
  std::string model_path;
  engine_info info{};
  std::unique_ptr<EngineModel> model;  // null while asleep
  std::vector<Slot> slots;
  std::vector<Checkpoint> checkpoints;
  std::vector<uint32_t> mapped;  // pages mapped per slot, as the queued plans leave them

  std::mutex mu;
  std::condition_variable work_cv, event_cv, idle_cv;
  std::deque<Plan> queue;
  std::deque<engine_event> events;
  std::deque<engine_timing> timing;
  engine_stats stats{};
  uint64_t opened_ns = 0, plans_done = 0;
  bool running = false, stop = false;
  std::thread thread;
  std::string err;

  // The last batch, for engine_read_batch.
  std::vector<BatchRun> last_runs;
  uint32_t last_rows = 0;

  void emit(engine_event ev) {
    events.push_back(ev);
    event_cv.notify_all();
  }
  void record(engine_timing t) {
    if (timing.size() == kTimingRing) timing.pop_front();
    timing.push_back(t);
  }
  // The slot's token for position pos; ends the request when it must (core/api/engine_api.cpp:323-339). Under mu.
  void emit_token(uint32_t s, int32_t tok, uint32_t pos) {
    Slot &sl = slots[s];
    sl.next = tok, sl.generated++;
    emit({ENGINE_EVENT_TOKEN, s, tok, pos});
    bool stop_tok = false;
    for (uint32_t i = 0; i < sl.settings.n_stop && i < ENGINE_MAX_STOP; i++) stop_tok |= sl.settings.stop[i] == tok;
    if (stop_tok || sl.generated >= sl.settings.max_tokens) {
      sl.done = true;
      emit({ENGINE_EVENT_DONE, s, tok, stop_tok ? (uint32_t)ENGINE_DONE_STOP : (uint32_t)ENGINE_DONE_LENGTH});
    } else if (pos >= info.max_ctx) {
      sl.done = true;
      emit({ENGINE_EVENT_DONE, s, tok, ENGINE_DONE_CONTEXT});
    }
  }
  void run_plan(const Plan &plan, uint32_t seq);
  void loop();
};

// One plan, one packed ragged batch. Runs on the engine thread.
void engine_ctx::run_plan(const Plan &plan, uint32_t seq) {
  struct Part {
    uint32_t slot, n, pos0, row0;
    bool piece;
  };
  std::vector<Part> parts;
  std::vector<int32_t> tokens;
  {
    std::lock_guard<std::mutex> lk(mu);
    const uint32_t cap = info.prompt_chunk;
    std::vector<bool> taken(slots.size(), false);
    for (uint32_t i = 0; i < plan.p.npieces && i < ENGINE_MAX_PROMPT_PIECES; i++) {
      const engine_prompt_piece &pi = plan.p.pieces[i];
      if (pi.slot >= slots.size() || taken[pi.slot]) continue;
      Slot &sl = slots[pi.slot];
      if (!sl.used || sl.done || sl.fed >= sl.prompt.size()) continue;  // released, or nothing left to read
      uint32_t n = (uint32_t)sl.prompt.size() - sl.fed;
      if (pi.tokens) n = std::min(n, pi.tokens);
      n = std::min<uint32_t>(n, cap - (uint32_t)tokens.size());
      if (n == 0) continue;
      parts.push_back({pi.slot, n, sl.fed, (uint32_t)tokens.size(), true});
      tokens.insert(tokens.end(), sl.prompt.begin() + sl.fed, sl.prompt.begin() + sl.fed + n);
      taken[pi.slot] = true;
    }
    for (uint32_t i = 0; i < plan.p.nslots && i < ENGINE_MAX_STEP_SLOTS; i++) {
      const uint32_t s = plan.p.slots[i];
      if (s >= slots.size() || taken[s] || tokens.size() >= cap) continue;
      Slot &sl = slots[s];
      if (!sl.used || sl.done) continue;
      if (sl.fed >= info.max_ctx) {
        sl.done = true;
        emit({ENGINE_EVENT_DONE, s, kNoToken, ENGINE_DONE_CONTEXT});
        continue;
      }
      const int32_t tok = sl.fed < sl.prompt.size() ? sl.prompt[sl.fed] : sl.next;
      parts.push_back({s, 1, sl.fed, (uint32_t)tokens.size(), false});
      tokens.push_back(tok);
      taken[s] = true;
    }
  }
  if (parts.empty()) return;
  // A run's last row gives a token when the run takes the slot to its prompt's end or past it.
  std::vector<uint32_t> want;
  std::vector<size_t> want_part;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (size_t i = 0; i < parts.size(); i++)
      if (parts[i].pos0 + parts[i].n >= slots[parts[i].slot].prompt.size()) want.push_back(parts[i].row0 + parts[i].n - 1), want_part.push_back(i);
  }
  std::vector<int32_t> next(want.size(), kNoToken);
  const uint64_t t0 = now_ns();
  model->batch(tokens.data(), (uint32_t)tokens.size(), want.data(), (uint32_t)want.size(), next.data(), kStepTimeoutMs);
  const uint64_t t1 = now_ns();

  std::lock_guard<std::mutex> lk(mu);
  last_runs.clear();
  last_rows = (uint32_t)tokens.size();
  uint32_t decode_rows = 0;
  for (const Part &pa : parts) last_runs.push_back({pa.n, pa.pos0, pa.slot, pa.row0});
  for (size_t i = 0; i < parts.size(); i++) {
    const Part &pa = parts[i];
    Slot &sl = slots[pa.slot];
    if (pa.piece) {
      record({ENGINE_TIMING_PROMPT, seq, pa.n, 0, t0, t1});
      stats.prompt_chunks++, stats.prompt_rows += pa.n, stats.prompt_ns += t1 - t0;
    } else {
      decode_rows++;
    }
    if (!sl.used) continue;  // released while the batch ran
    sl.tokens.insert(sl.tokens.end(), tokens.begin() + pa.row0, tokens.begin() + pa.row0 + pa.n);
    const bool own = !pa.piece && pa.pos0 >= sl.prompt.size();  // the row was one of the slot's own tokens
    sl.fed = pa.pos0 + pa.n;
    if (sl.fed <= sl.prompt.size() && (pa.piece || sl.fed % 512 == 0 || sl.fed == sl.prompt.size()))
      emit({ENGINE_EVENT_PROMPT, pa.slot, kNoToken, sl.fed});
    if (own) sl.stats.steps++;
    const auto w = std::find(want_part.begin(), want_part.end(), i);
    if (w != want_part.end() && !sl.done) emit_token(pa.slot, next[w - want_part.begin()], sl.fed);
  }
  if (decode_rows) {
    record({ENGINE_TIMING_DECODE, seq, decode_rows, 0, t0, t1});
    stats.steps++, stats.step_rows += decode_rows, stats.step_ns += t1 - t0;
  }
  stats.experts_cached = model->n_experts();
}

void engine_ctx::loop() {
  for (;;) {
    Plan plan;
    {
      std::unique_lock<std::mutex> lk(mu);
      work_cv.wait(lk, [&] { return stop || !queue.empty(); });
      if (stop && queue.empty()) return;
      plan = std::move(queue.front());
    }
    const uint64_t t0 = now_ns();
    const uint32_t seq = (uint32_t)(plans_done + 1);
    bool failed = false;
    std::string what;
    try {
      if (!model) throw std::runtime_error("the engine is asleep");
      run_plan(plan, seq);
    } catch (const Timeout &e) {
      g_stuck = 1, failed = true, what = e.what();
    } catch (const std::exception &e) {
      failed = true, what = e.what();
    }
    std::lock_guard<std::mutex> lk(mu);
    queue.pop_front();
    plans_done++;
    stats.plans++, stats.busy_ns += now_ns() - t0;
    if (failed) {
      err = what;
      emit({ENGINE_EVENT_ERROR, 0, kNoToken, ENGINE_ERROR});
    }
    emit({ENGINE_EVENT_STEP, 0, kNoToken, (uint32_t)plans_done});
    if (queue.empty()) idle_cv.notify_all();
  }
}

namespace {

template <class Fn>
engine_status guarded(engine_ctx *e, Fn &&fn) {
  try {
    return fn();
  } catch (const BadArgument &x) {
    (e ? e->err : g_open_error) = x.what();
    return ENGINE_BAD_ARGUMENT;
  } catch (const Timeout &x) {
    (e ? e->err : g_open_error) = x.what();
    return ENGINE_TIMEOUT;
  } catch (const std::exception &x) {
    (e ? e->err : g_open_error) = x.what();
    return ENGINE_ERROR;
  }
}

void fill_info(engine_ctx *e, double seconds) {
  engine_info &i = e->info;
  std::memset(&i, 0, sizeof(i));
  i.api_version = ENGINE_API_VERSION, i.cards = 1;
  i.slots = (uint32_t)e->slots.size(), i.max_ctx = e->config.max_ctx;
  i.experts_per_layer = e->model->n_experts(), i.vocab = e->model->vocab();
  i.device_bytes[0] = e->model->device_bytes();
  i.load_seconds = seconds;
  i.prompt_chunk = e->model->max_rows(), i.checkpoints = (uint32_t)e->checkpoints.size();
  i.max_step_rows = e->model->max_rows();
  i.pages_per_slot = (e->config.max_ctx + 3) / 4;
  i.kv_pages = e->config.kv_pages ? e->config.kv_pages : i.slots * i.pages_per_slot;
}

// Waits until the engine thread has run every queued plan. Under lk.
void drain(engine_ctx *e, std::unique_lock<std::mutex> &lk) { e->idle_cv.wait(lk, [&] { return e->queue.empty(); }); }

// A plan's page changes against the rules of engine_abi.h, counting the changes of the plans queued before it.
void check_pages(engine_ctx *e, const engine_step_plan &p) {
  std::vector<uint32_t> mapped = e->mapped;
  for (uint32_t i = 0; i < p.npages; i++) {
    const engine_page_change &c = p.pages[i];
    if (c.slot >= e->slots.size()) throw BadArgument("a page change names slot " + std::to_string(c.slot) + ", past the engine's slots");
    if (c.logical > mapped[c.slot]) throw BadArgument("a page change leaves a gap in slot " + std::to_string(c.slot) + "'s pages");
    if (c.page == ENGINE_NO_PAGE) {
      mapped[c.slot] = c.logical;
      continue;
    }
    if (c.page >= e->info.kv_pages || c.logical >= e->info.pages_per_slot) throw BadArgument("a page change names a page past the pool or the slot's context");
    if (c.cells > 3 || (c.cells && c.source >= e->info.kv_pages)) throw BadArgument("a page change copies more than 3 cells, or from a page past the pool");
    mapped[c.slot] = std::max(mapped[c.slot], c.logical + 1);
  }
  e->mapped = mapped;
}

}  // namespace

extern "C" {

ENGINE_API engine_status engine_open(const engine_config *config, engine_info *info, engine_ctx **out) {
  if (!config || !out || !config->model_path) {
    g_open_error = "config, its model_path and out are required";
    return ENGINE_BAD_ARGUMENT;
  }
  *out = nullptr;
  auto e = std::make_unique<engine_ctx>();
  engine_ctx *raw = e.get();
  const engine_status s = guarded(nullptr, [&]() -> engine_status {
    raw->config = *config;
    raw->model_path = config->model_path;
    engine_config &c = raw->config;
    c.model_path = raw->model_path.c_str();
    if (!c.slots) c.slots = 1;
    if (!c.max_ctx) c.max_ctx = 32768;
    if (c.max_ctx % 4) throw BadArgument("max_ctx must be a multiple of 4");
    if (c.max_cards > 1) throw BadArgument("this engine runs its layers on one GPU: max_cards is 0 or 1");
    const bool set = c.flags & ENGINE_CONFIG_PROMPT_SET;
    if (!c.prompt_chunk && !set) c.prompt_chunk = 4352;
    if (c.prompt_chunk % 64) throw BadArgument("prompt_chunk must be a multiple of 64");
    if (!c.prompt_chunk) c.prompt_chunk = 64;  // the prompt path "off": pieces still ride in the batch, 64 rows at most
    const auto t0 = std::chrono::steady_clock::now();
    raw->model = std::make_unique<EngineModel>(raw->model_path, 0, c.prompt_chunk);
    raw->slots.resize(c.slots);
    raw->mapped.assign(c.slots, 0);
    raw->checkpoints.resize(c.checkpoints);
    fill_info(raw, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    raw->opened_ns = now_ns();
    raw->running = true;
    raw->thread = std::thread([raw] { raw->loop(); });
    return ENGINE_OK;
  });
  if (s != ENGINE_OK) return s;
  if (info) *info = raw->info;
  *out = e.release();
  return ENGINE_OK;
}

ENGINE_API engine_status engine_admit(engine_ctx *e, uint32_t slot, const engine_settings *settings, const int32_t *prompt, uint32_t n_prompt) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  return guarded(e, [&]() -> engine_status {
    if (!e->model) throw std::runtime_error("the engine is asleep");
    if (!settings || !prompt || n_prompt == 0 || slot >= e->slots.size()) throw BadArgument("a slot of the engine, settings and a prompt are required");
    if (settings->min_p < 0.0f || settings->min_p > 1.0f) throw BadArgument("min_p must be in [0, 1]");
    if (settings->penalty_last_n && settings->penalty_repeat <= 0.0f) throw BadArgument("a penalty needs penalty_repeat above 0");
    if (n_prompt >= e->config.max_ctx) throw BadArgument("the prompt does not fit the context");
    for (uint32_t i = 0; i < n_prompt; i++)
      if (prompt[i] < 0 || (uint32_t)prompt[i] >= e->model->vocab()) throw BadArgument("a prompt token is outside the vocabulary");
    Slot &sl = e->slots[slot];
    if (sl.used) {
      e->err = "slot " + std::to_string(slot) + " is in use";
      return ENGINE_BUSY;
    }
    sl = Slot{};
    sl.used = true, sl.settings = *settings;
    sl.prompt.assign(prompt, prompt + n_prompt);
    e->mapped[slot] = 0;
    return ENGINE_OK;
  });
}

ENGINE_API engine_status engine_admit_images(engine_ctx *e, uint32_t slot, const engine_image *images, uint32_t n) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  if (slot >= e->slots.size() || !e->slots[slot].used) return e->err = "the slot is not admitted", ENGINE_BAD_ARGUMENT;
  if (n == 0) return ENGINE_OK;
  (void)images;
  return e->err = "this model has no image encoder (image_tokens_max is 0)", ENGINE_BAD_ARGUMENT;
}

ENGINE_API engine_status engine_release(engine_ctx *e, uint32_t slot) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  if (slot >= e->slots.size()) return e->err = "no such slot", ENGINE_BAD_ARGUMENT;
  e->slots[slot] = Slot{};
  return ENGINE_OK;
}

ENGINE_API engine_status engine_submit(engine_ctx *e, const engine_step_plan *plan) {
  if (!e || !plan) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  return guarded(e, [&]() -> engine_status {
    if (!e->model) throw std::runtime_error("the engine is asleep");
    if (plan->nslots > ENGINE_MAX_STEP_SLOTS || plan->npieces > ENGINE_MAX_PROMPT_PIECES) throw BadArgument("too many decode slots or prompt pieces");
    if (plan->npages && !plan->pages) throw BadArgument("npages without pages");
    if (e->queue.size() >= kMaxQueuedPlans) {
      e->err = "the plan queue is full";
      return ENGINE_BUSY;
    }
    check_pages(e, *plan);
    Plan p;
    p.p = *plan;
    p.pages.assign(plan->pages, plan->pages + plan->npages);  // submit copies the changes
    p.p.pages = nullptr;
    e->queue.push_back(std::move(p));
    e->work_cv.notify_one();
    return ENGINE_OK;
  });
}

ENGINE_API engine_status engine_poll(engine_ctx *e, engine_event *buf, uint32_t cap, uint32_t *n) {
  if (!e || !n || (cap && !buf)) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  uint32_t k = 0;
  while (k < cap && !e->events.empty()) buf[k++] = e->events.front(), e->events.pop_front();
  *n = k;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_wait(engine_ctx *e, uint32_t timeout_ms) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  return e->event_cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !e->events.empty(); }) ? ENGINE_OK : ENGINE_TIMEOUT;
}

ENGINE_API engine_status engine_checkpoint(engine_ctx *e, uint32_t slot, uint32_t id) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  drain(e, lk);
  if (!e->model) return e->err = "the engine is asleep", ENGINE_ERROR;
  if (slot >= e->slots.size() || !e->slots[slot].used || id >= e->checkpoints.size())
    return e->err = "an admitted slot and a checkpoint id below config.checkpoints are required", ENGINE_BAD_ARGUMENT;
  e->checkpoints[id] = Checkpoint{true, e->slots[slot].tokens};
  e->stats.checkpoints_taken++;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_restore(engine_ctx *e, uint32_t slot, uint32_t id) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  drain(e, lk);
  if (!e->model) return e->err = "the engine is asleep", ENGINE_ERROR;
  if (slot >= e->slots.size() || !e->slots[slot].used || id >= e->checkpoints.size() || !e->checkpoints[id].full)
    return e->err = "an admitted slot and a full checkpoint are required", ENGINE_BAD_ARGUMENT;
  Slot &sl = e->slots[slot];
  const std::vector<int32_t> &ck = e->checkpoints[id].tokens;
  if (ck.size() > sl.prompt.size() || !std::equal(ck.begin(), ck.end(), sl.prompt.begin()))
    return e->err = "the checkpoint's tokens are not a prefix of the slot's prompt", ENGINE_BAD_ARGUMENT;
  sl.tokens = ck, sl.fed = (uint32_t)ck.size();
  e->stats.restores++;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_drop(engine_ctx *e, uint32_t id) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  if (id >= e->checkpoints.size()) return e->err = "no such checkpoint", ENGINE_BAD_ARGUMENT;
  e->checkpoints[id] = Checkpoint{};
  return ENGINE_OK;
}

ENGINE_API engine_status engine_read_timing(engine_ctx *e, engine_timing *buf, uint32_t cap, uint32_t *n) {
  if (!e || !n || (cap && !buf)) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  uint32_t k = 0;
  while (k < cap && !e->timing.empty()) buf[k++] = e->timing.front(), e->timing.pop_front();
  *n = k;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_read_stats(engine_ctx *e, engine_stats *out) {
  if (!e || !out) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  *out = e->stats;
  out->up_ns = now_ns() - e->opened_ns;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_read_slot_stats(engine_ctx *e, uint32_t slot, engine_slot_stats *out) {
  if (!e || !out) return ENGINE_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lk(e->mu);
  if (slot >= e->slots.size() || !e->slots[slot].used) return e->err = "the slot is not admitted", ENGINE_BAD_ARGUMENT;
  *out = e->slots[slot].stats;
  return ENGINE_OK;
}

ENGINE_API engine_status engine_sleep(engine_ctx *e) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  drain(e, lk);
  if (!e->model) return ENGINE_OK;
  for (const Slot &s : e->slots)
    if (s.used) return e->err = "a slot is admitted", ENGINE_BUSY;
  e->model.reset();
  for (Checkpoint &c : e->checkpoints) c = Checkpoint{};
  return ENGINE_OK;
}

ENGINE_API engine_status engine_wake(engine_ctx *e, engine_info *info) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  drain(e, lk);
  const engine_status s = guarded(e, [&]() -> engine_status {
    if (!e->model) {
      const auto t0 = std::chrono::steady_clock::now();
      e->model = std::make_unique<EngineModel>(e->model_path, 0, e->config.prompt_chunk);
      fill_info(e, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
    }
    return ENGINE_OK;
  });
  if (s == ENGINE_OK && info) *info = e->info;
  return s;
}

ENGINE_API const char *engine_last_error(const engine_ctx *e) { return e ? e->err.c_str() : g_open_error.c_str(); }

ENGINE_API void engine_close(engine_ctx *e) {
  if (!e) return;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->stop = true;
    e->work_cv.notify_all();
  }
  if (e->thread.joinable()) e->thread.join();
  delete e;
}

ENGINE_API int engine_queue_stuck(void) { return g_stuck.load(); }

ENGINE_API engine_status engine_cards(engine_card *cards, uint32_t cap, uint32_t *n) {
  if (!n) return ENGINE_BAD_ARGUMENT;
  return guarded(nullptr, [&]() -> engine_status {
    int count = 0;
    CUDA_OK(cudaGetDeviceCount(&count));
    for (int d = 0; cards && d < count && (uint32_t)d < cap; d++) {
      cudaDeviceProp p{};
      CUDA_OK(cudaGetDeviceProperties(&p, d));
      engine_card &c = cards[d];
      std::memset(&c, 0, sizeof(c));
      std::strncpy(c.name, p.name, sizeof(c.name) - 1);
      std::snprintf(c.pci, sizeof(c.pci), "%04x:%02x:%02x.0", p.pciDomainID, p.pciBusID, p.pciDeviceID);
      c.memory = p.totalGlobalMem;
      int dev_id = 0;
      if (cudaDeviceGetAttribute(&dev_id, cudaDevAttrPciDeviceId, d) == cudaSuccess) c.device_id = (uint32_t)dev_id;
      c.ip_version = (uint32_t)p.major << 8 | (uint32_t)p.minor;
      c.xe_cores = (uint32_t)p.multiProcessorCount;
      c.pcie_gen = -1, c.pcie_width = -1, c.pcie_bytes_per_s = -1;
    }
    *n = (uint32_t)count;
    return ENGINE_OK;
  });
}

ENGINE_API engine_status engine_read_batch(engine_ctx *e, float *hidden, uint32_t rows_cap, uint32_t *rows, engine_batch_run *runs,
                                           uint32_t runs_cap, uint32_t *nruns) {
  if (!e) return ENGINE_BAD_ARGUMENT;
  std::unique_lock<std::mutex> lk(e->mu);
  drain(e, lk);
  return guarded(e, [&]() -> engine_status {
    if (!e->model) throw std::runtime_error("the engine is asleep");
    if (rows) *rows = e->last_rows;
    if (nruns) *nruns = (uint32_t)e->last_runs.size();
    if (hidden) e->model->read_hidden(hidden, std::min(rows_cap, e->last_rows));
    for (uint32_t i = 0; runs && i < runs_cap && i < e->last_runs.size(); i++)
      runs[i] = engine_batch_run{e->last_runs[i].n, e->last_runs[i].pos0, e->last_runs[i].slot, e->last_runs[i].row0};
    return ENGINE_OK;
  });
}

ENGINE_API uint32_t engine_abi_layout(engine_abi_row *table, uint32_t cap) {
#define ROW(S, F) {#S "." #F, (uint32_t)offsetof(S, F), (uint32_t)sizeof(((S *)nullptr)->F)}
#define SIZE(S) {#S, 0, (uint32_t)sizeof(S)}
#define R2(S, A, B) ROW(S, A), ROW(S, B)
#define R4(S, A, B, C, D) R2(S, A, B), R2(S, C, D)
  static const engine_abi_row rows[] = {
      R4(engine_config, model_path, slots, max_ctx, max_cards), R4(engine_config, experts_per_layer, cpu_threads, flags, reserve_bytes),
      R4(engine_config, prompt_chunk, checkpoints, routing_profile, mtp_dir), R4(engine_config, draft_max, draft_min_p, vision_path, kv_pages),
      R2(engine_config, kv_resident_cells, ngram_huge_bytes), SIZE(engine_config),
      R4(engine_info, api_version, cards, slots, max_ctx), R4(engine_info, experts_per_layer, vocab, device_bytes, arena_bytes),
      R4(engine_info, load_seconds, prompt_chunk, checkpoints, max_step_rows), R4(engine_info, drafting, image_tokens_max, kv_pages, pages_per_slot),
      R4(engine_info, host_read_bytes_per_s, loader_threads, ngram_in_ram, loader_bytes_per_s),
      R4(engine_info, ngram_read_us, copy_bytes_per_s, expert_budget, fetch_rows), R2(engine_info, decode_weight, ngram_cache_rows),
      ROW(engine_info, ngram_huge_bytes), SIZE(engine_info),
      R4(engine_settings, temperature, top_k, top_p, max_tokens), R4(engine_settings, seed, n_stop, stop, min_p),
      R4(engine_settings, penalty_last_n, penalty_repeat, penalty_freq, penalty_present), SIZE(engine_settings),
      R4(engine_page_change, slot, logical, page, source), ROW(engine_page_change, cells), SIZE(engine_page_change),
      R2(engine_prompt_piece, slot, tokens), SIZE(engine_prompt_piece),
      R4(engine_step_plan, nslots, slots, npieces, pieces), R4(engine_step_plan, npages, pages, kv_free, window_rows), SIZE(engine_step_plan),
      R4(engine_event, kind, slot, token, value), SIZE(engine_event),
      R4(engine_timing, kind, plan, rows, misses), R2(engine_timing, start_ns, end_ns), SIZE(engine_timing),
      R4(engine_stats, up_ns, plans, busy_ns, prompt_chunks), R4(engine_stats, prompt_rows, prompt_ns, window_pieces, window_rows),
      R4(engine_stats, window_ns, steps, step_rows, step_ns), R4(engine_stats, step_misses, step_layers_missed, undrafted_steps, rounds),
      R4(engine_stats, round_rows, round_ns, round_misses, round_layers_missed), R4(engine_stats, layer_runs, layer_drafts, layer_accepted, layer_ns),
      R4(engine_stats, lookup_runs, lookup_drafts, lookup_accepted, lookup_ns), R4(engine_stats, swap_rounds, swaps, swap_ns, stalls),
      R4(engine_stats, checkpoints_taken, restores, ngram_rows, ngram_hits), R4(engine_stats, ngram_reads, experts_cached, experts_floor, idle_rounds),
      R4(engine_stats, reading_steps, reading_rounds, draft_passes, draft_ns),
      R4(engine_stats, layer_drafts_1, layer_drafts_2, layer_drafts_3, layer_drafts_4), R4(engine_stats, layer_drafts_5, layer_drafts_6, layer_drafts_7, layer_accepted_1),
      R4(engine_stats, layer_accepted_2, layer_accepted_3, layer_accepted_4, layer_accepted_5), R2(engine_stats, layer_accepted_6, layer_accepted_7),
      R4(engine_stats, layer_stop_max, layer_stop_share, layer_stop_p, layer_stop_choice), SIZE(engine_stats),
      R4(engine_slot_stats, steps, rounds, drafts, accepted), R2(engine_slot_stats, lookup_rounds, lookup_drafts), ROW(engine_slot_stats, lookup_accepted),
      SIZE(engine_slot_stats),
      R4(engine_image, first, grid_h, grid_w, frames), ROW(engine_image, pixels), SIZE(engine_image),
      R4(engine_card, name, pci, memory, device_id), R4(engine_card, ip_version, xe_cores, pcie_gen, pcie_width), R2(engine_card, reserved, pcie_bytes_per_s),
      SIZE(engine_card),
      R2(engine_abi_row, name, offset), ROW(engine_abi_row, size), SIZE(engine_abi_row),
  };
#undef R4
#undef R2
#undef SIZE
#undef ROW
  const uint32_t n = (uint32_t)(sizeof(rows) / sizeof(rows[0]));
  for (uint32_t i = 0; table && i < n && i < cap; i++) table[i] = rows[i];
  return n;
}

}  // extern "C"
