#include "pool.h"

#include <cstdlib>
#include <cstring>
#include <sched.h>

namespace blh {

// spins on the generation word before a worker parks (BLOOMERY_SPIN; blh_pool_set_spin)
static std::atomic<int> g_spin{[] {
  if (const char* e = std::getenv("BLOOMERY_SPIN")) { int v = std::atoi(e); if (v >= 0) return v; }
  return 20000;
}()};
static std::atomic<int> g_pin{-1};   // -1: follow BLOOMERY_PIN, 0 / 1: set by blh_pool_set_pin

static int default_threads() {
  if (const char* e = std::getenv("BLOOMERY_THREADS")) {
    int v = std::atoi(e);
    if (v > 0) return v;
  }
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) == 0) {
    int c = CPU_COUNT(&set);
    if (c > 0) return c;
  }
  unsigned h = std::thread::hardware_concurrency();
  return h ? (int)h : 1;
}

Pool& Pool::instance() {
  static Pool p(default_threads());
  return p;
}

Pool::Pool(int n_threads) { start(n_threads); }
Pool::~Pool() { stop(); }

void Pool::start(int n_threads) {
  quit_ = false;
  for (int i = 1; i < n_threads; ++i) workers_.emplace_back([this, i] { worker_loop(i); });
}

void Pool::stop() {
  {
    std::lock_guard<std::mutex> g(mu_);
    quit_ = true;
    generation_.fetch_add(1);
  }
  cv_.notify_all();
  for (auto& t : workers_) t.join();
  workers_.clear();
}

void Pool::resize(int n_threads) {
  std::lock_guard<std::mutex> g(call_mu_);
  stop();
  start(n_threads < 1 ? 1 : n_threads);
}

void Pool::run_chunks() {
  for (;;) {
    int b = cursor_.fetch_add(grain_);
    if (b >= n_) break;
    int e = b + grain_ < n_ ? b + grain_ : n_;
    (*fn_)(b, e);
  }
}

void Pool::worker_loop(int idx) {
  const char* pin = std::getenv("BLOOMERY_PIN");
  const int forced = g_pin.load();
  if (forced == 1 || (forced < 0 && (!pin || std::strcmp(pin, "0") != 0))) {
    cpu_set_t allowed;
    CPU_ZERO(&allowed);
    if (sched_getaffinity(0, sizeof(allowed), &allowed) == 0) {
      int want = idx % CPU_COUNT(&allowed), seen = 0;
      for (int c = 0; c < CPU_SETSIZE; ++c)
        if (CPU_ISSET(c, &allowed)) {
          if (seen++ == want) {
            cpu_set_t one;
            CPU_ZERO(&one);
            CPU_SET(c, &one);
            pthread_setaffinity_np(pthread_self(), sizeof(one), &one);
            break;
          }
        }
    }
  }
  uint64_t seen_gen = 0;
  for (;;) {
    // spin, then park
    int spins = 0;
    while (generation_.load(std::memory_order_acquire) == seen_gen) {
      if (++spins > g_spin.load(std::memory_order_relaxed)) {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return generation_.load() != seen_gen; });
        break;
      }
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    }
    seen_gen = generation_.load(std::memory_order_acquire);
    if (quit_.load()) return;
    run_chunks();
    pending_.fetch_sub(1, std::memory_order_acq_rel);
  }
}

void Pool::parallel_for(int n, int grain, const std::function<void(int, int)>& fn) {
  if (n <= 0) return;
  if (workers_.empty() || n <= grain) { fn(0, n); return; }
  std::lock_guard<std::mutex> g(call_mu_);
  n_ = n; grain_ = grain < 1 ? 1 : grain; fn_ = &fn;
  cursor_.store(0);
  pending_.store((int)workers_.size());
  {
    std::lock_guard<std::mutex> lk(mu_);
    generation_.fetch_add(1, std::memory_order_release);
  }
  cv_.notify_all();
  run_chunks();
  while (pending_.load(std::memory_order_acquire) > 0) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  }
  fn_ = nullptr;
}

}  // namespace blh

extern "C" {
int blh_pool_size() { return blh::Pool::instance().size(); }
void blh_pool_resize(int n) { blh::Pool::instance().resize(n); }
void blh_pool_set_spin(int spins) { blh::g_spin.store(spins < 0 ? 0 : spins); }
// takes effect for workers started afterwards (call before blh_pool_resize)
void blh_pool_set_pin(int on) { blh::g_pin.store(on ? 1 : 0); }
}
