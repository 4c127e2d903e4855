// Token-window data loader of the host runtime (see oil_host.h): windows of seq + 1 tokens over a
// token array, optional window-level shuffle per epoch, batches assembled by a worker thread into a
// bounded ring so that the training loop only copies a finished batch (into pinned memory when the
// caller passes pinned buffers). Role of the reference's DataLoader with its prefetch thread and
// bounded queue (src/trainer.cpp:91-238); unlike it, shuffling permutes windows, not single tokens.
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "oil_host.h"

struct OilLoader {
  std::vector<int32_t> tokens;
  int batch = 0, seq = 0, prefetch = 2;
  bool shuffle = false;
  uint64_t seed = 0;
  int64_t n_windows = 0, n_batches = 0;
  std::vector<int64_t> order;

  // ring of prepared batches: ids then targets, batch * seq each
  std::vector<std::vector<int32_t>> ring;
  int64_t produced = 0, consumed = 0;   // batch counters of the current epoch
  std::mutex mu;
  std::condition_variable cv_space, cv_data;
  std::thread worker;
  bool stop = false;

  void run() {
    for (;;) {
      int64_t b;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_space.wait(lk, [&] { return stop || (produced < n_batches && produced - consumed < prefetch); });
        if (stop) return;
        b = produced;
      }
      std::vector<int32_t>& slot = ring[(size_t)(b % prefetch)];
      const int64_t per = (int64_t)batch * seq;
      for (int i = 0; i < batch; ++i) {
        const int64_t w = order[(size_t)(b * batch + i)];
        const int32_t* src = tokens.data() + w * seq;
        std::memcpy(slot.data() + (int64_t)i * seq, src, sizeof(int32_t) * (size_t)seq);
        std::memcpy(slot.data() + per + (int64_t)i * seq, src + 1, sizeof(int32_t) * (size_t)seq);
      }
      {
        std::lock_guard<std::mutex> lk(mu);
        ++produced;
      }
      cv_data.notify_one();
    }
  }

  void halt() {
    {
      std::lock_guard<std::mutex> lk(mu);
      stop = true;
    }
    cv_space.notify_all();
    cv_data.notify_all();
    if (worker.joinable()) worker.join();
    stop = false;
  }
};

namespace {
// splitmix64: the seeding function of the runtime's RNG, used here as the shuffle generator
inline uint64_t splitmix64(uint64_t& x) {
  uint64_t z = (x += 0x9E3779B97F4A7C15ULL);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
}  // namespace

extern "C" {

OilLoader* oil_loader_create(const int32_t* tokens, int64_t n_tokens, int batch, int seq, int shuffle, uint64_t seed,
                             int prefetch) {
  if (!tokens || n_tokens < 2 || batch < 1 || seq < 1) return nullptr;
  auto* L = new OilLoader;
  L->tokens.assign(tokens, tokens + n_tokens);
  L->batch = batch;
  L->seq = seq;
  L->prefetch = prefetch < 1 ? 1 : prefetch;
  L->shuffle = shuffle != 0;
  L->seed = seed;
  L->n_windows = (n_tokens - 1) / seq;
  L->n_batches = L->n_windows / batch;   // full batches only
  L->ring.assign((size_t)L->prefetch, std::vector<int32_t>((size_t)2 * batch * seq));
  oil_loader_reset(L, 0);
  return L;
}

int64_t oil_loader_num_batches(const OilLoader* L) { return L ? L->n_batches : 0; }

void oil_loader_reset(OilLoader* L, int epoch) {
  if (!L) return;
  L->halt();
  L->order.resize((size_t)L->n_windows);
  for (int64_t i = 0; i < L->n_windows; ++i) L->order[(size_t)i] = i;
  if (L->shuffle) {   // Fisher-Yates, deterministic in (seed, epoch)
    uint64_t s = L->seed * 0x9E3779B97F4A7C15ULL + (uint64_t)epoch + 1;
    for (int64_t i = L->n_windows - 1; i > 0; --i) {
      const int64_t j = (int64_t)(splitmix64(s) % (uint64_t)(i + 1));
      std::swap(L->order[(size_t)i], L->order[(size_t)j]);
    }
  }
  L->produced = L->consumed = 0;
  L->worker = std::thread([L] { L->run(); });
}

// Copies the next batch into ids_out / targets_out (batch * seq int32 each). Returns 1, or 0 when the
// epoch is over.
int oil_loader_next(OilLoader* L, int32_t* ids_out, int32_t* targets_out) {
  if (!L || !ids_out || !targets_out) return 0;
  const int64_t per = (int64_t)L->batch * L->seq;
  {
    std::unique_lock<std::mutex> lk(L->mu);
    if (L->consumed >= L->n_batches) return 0;
    L->cv_data.wait(lk, [&] { return L->produced > L->consumed; });
  }
  const std::vector<int32_t>& slot = L->ring[(size_t)(L->consumed % L->prefetch)];
  std::memcpy(ids_out, slot.data(), sizeof(int32_t) * (size_t)per);
  std::memcpy(targets_out, slot.data() + per, sizeof(int32_t) * (size_t)per);
  {
    std::lock_guard<std::mutex> lk(L->mu);
    ++L->consumed;
  }
  L->cv_space.notify_one();
  return 1;
}

void oil_loader_free(OilLoader* L) {
  if (!L) return;
  L->halt();
  delete L;
}

}  // extern "C"
