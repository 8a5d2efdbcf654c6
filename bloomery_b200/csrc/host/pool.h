// Resident worker pool: workers spin briefly on a generation word, then park on a
// condition variable; work is split into contiguous chunks claimed by an atomic cursor.
// Counterpart of crates/threads (lib.rs:1-33: resident pinned workers, spin then park,
// affinity-mask aware).  Affinity: each worker is pinned to one CPU of the process's
// allowed set when BLOOMERY_PIN is not "0".
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace blh {

class Pool {
 public:
  static Pool& instance();
  explicit Pool(int n_threads);
  ~Pool();
  int size() const { return (int)workers_.size() + 1; }
  // run fn(begin, end) over [0, n) in chunks of `grain`; the caller takes part
  void parallel_for(int n, int grain, const std::function<void(int, int)>& fn);
  void resize(int n_threads);

 private:
  void worker_loop(int idx);
  void run_chunks();
  void start(int n_threads);
  void stop();
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::atomic<uint64_t> generation_{0};
  std::atomic<int> cursor_{0};
  std::atomic<int> pending_{0};
  std::atomic<bool> quit_{false};
  int n_ = 0, grain_ = 1;
  const std::function<void(int, int)>* fn_ = nullptr;
  std::mutex call_mu_;
};

}  // namespace blh
