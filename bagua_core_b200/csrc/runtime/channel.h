// Thread-safe channels used by the scheduler.
//
//  * `EventChannel` — one-shot completion flag handed out per scheduled bucket
//    (reference: bagua-core-internal/src/events.rs:5-31).  The wait loops on a
//    predicate, so a spurious wake-up cannot release a waiter early (the reference
//    tests the flag with a single `if`).
//  * `Channel<T>`   — MPMC queue, optionally bounded.  A bounded channel blocks the
//    sender when full, which is how back-pressure reaches `mark_communication_ready`
//    (reference: flume::bounded in bagua-core-internal/src/lib.rs:84-100).
#pragma once

#include <condition_variable>
#include <deque>
#include <optional>

#include "../common.h"

namespace bagua {

class EventChannel {
 public:
  explicit EventChannel(std::string name) : state_(std::make_shared<State>()) { state_->name = std::move(name); }

  void finish() const {
    {
      std::lock_guard<std::mutex> g(state_->mu);
      state_->finished = true;
    }
    state_->cv.notify_all();
  }
  void fail(const std::string& err) const {
    {
      std::lock_guard<std::mutex> g(state_->mu);
      state_->error = err;
      state_->finished = true;
    }
    state_->cv.notify_all();
  }
  // Blocks until finish()/fail(); returns the error text ("" when none).
  std::string wait() const {
    std::unique_lock<std::mutex> lk(state_->mu);
    state_->cv.wait(lk, [&] { return state_->finished; });
    return state_->error;
  }
  // Returns false on timeout.
  bool wait_for(std::chrono::milliseconds d) const {
    std::unique_lock<std::mutex> lk(state_->mu);
    return state_->cv.wait_for(lk, d, [&] { return state_->finished; });
  }
  bool finished() const {
    std::lock_guard<std::mutex> g(state_->mu);
    return state_->finished;
  }
  const std::string& name() const { return state_->name; }

 private:
  struct State {
    std::string name;
    std::mutex mu;
    std::condition_variable cv;
    bool finished = false;
    std::string error;
  };
  std::shared_ptr<State> state_;
};

template <typename T>
class Channel {
 public:
  // cap == 0 → unbounded
  explicit Channel(size_t cap = 0) : cap_(cap) {}

  // Blocks while full.  Returns false if the channel was closed.
  bool send(T v) {
    std::unique_lock<std::mutex> lk(mu_);
    not_full_.wait(lk, [&] { return closed_ || cap_ == 0 || q_.size() < cap_; });
    if (closed_) return false;
    q_.push_back(std::move(v));
    lk.unlock();
    not_empty_.notify_one();
    return true;
  }
  // Blocks while empty.  nullopt once closed and drained.
  std::optional<T> recv() {
    std::unique_lock<std::mutex> lk(mu_);
    not_empty_.wait(lk, [&] { return closed_ || !q_.empty(); });
    if (q_.empty()) return std::nullopt;
    T v = std::move(q_.front());
    q_.pop_front();
    lk.unlock();
    not_full_.notify_one();
    return v;
  }
  std::optional<T> try_recv() {
    std::unique_lock<std::mutex> lk(mu_);
    if (q_.empty()) return std::nullopt;
    T v = std::move(q_.front());
    q_.pop_front();
    lk.unlock();
    not_full_.notify_one();
    return v;
  }
  // 0 = got a value, 1 = timed out, 2 = closed
  int recv_timeout(std::chrono::milliseconds d, T* out) {
    std::unique_lock<std::mutex> lk(mu_);
    if (!not_empty_.wait_for(lk, d, [&] { return closed_ || !q_.empty(); })) return 1;
    if (q_.empty()) return 2;
    *out = std::move(q_.front());
    q_.pop_front();
    lk.unlock();
    not_full_.notify_one();
    return 0;
  }
  void close() {
    {
      std::lock_guard<std::mutex> g(mu_);
      closed_ = true;
    }
    not_empty_.notify_all();
    not_full_.notify_all();
  }
  size_t size() const {
    std::lock_guard<std::mutex> g(mu_);
    return q_.size();
  }
  size_t capacity() const { return cap_; }

 private:
  const size_t cap_;
  mutable std::mutex mu_;
  std::condition_variable not_empty_, not_full_;
  std::deque<T> q_;
  bool closed_ = false;
};

}  // namespace bagua
