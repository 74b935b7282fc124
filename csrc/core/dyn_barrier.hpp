// Generation-counted barrier whose membership can shrink while threads wait, with a leader section
// run by the last arriver before anyone is released (parameter_server/src/synchronization/
// dyn_barrier.rs:6-107). BarrierSync relies on it so that a worker that finishes early never
// deadlocks the ones still training (synchronization/barrier.rs:30-38).
#pragma once
#include <condition_variable>
#include <functional>
#include <mutex>

namespace ono {

class DynBarrier {
 public:
  explicit DynBarrier(size_t size) : size_(size) {}

  // Blocks until `size` participants arrived; the last one runs `leader` first. Returns true for
  // the leader.
  bool wait_with(const std::function<void()>& leader) {
    std::unique_lock<std::mutex> lk(mu_);
    const size_t gen = generation_;
    ++arrived_;
    if (arrived_ >= size_) {
      release(leader);
      return true;
    }
    cv_.wait(lk, [&] { return generation_ != gen; });
    return false;
  }

  // A participant leaves for good: the expected count drops by one, and if everyone else is already
  // waiting they are released (the leader section runs on the leaving thread).
  void leave(const std::function<void()>& leader) {
    std::unique_lock<std::mutex> lk(mu_);
    if (size_ > 0) --size_;
    if (size_ > 0 && arrived_ >= size_) release(leader);
  }

  size_t size() const {
    std::lock_guard<std::mutex> lk(mu_);
    return size_;
  }

 private:
  void release(const std::function<void()>& leader) {
    if (leader) leader();
    arrived_ = 0;
    ++generation_;
    cv_.notify_all();
  }
  mutable std::mutex mu_;
  std::condition_variable cv_;
  size_t size_, arrived_ = 0, generation_ = 0;
};

}  // namespace ono
