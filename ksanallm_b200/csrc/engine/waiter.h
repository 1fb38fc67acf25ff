// Blocking primitives of the request path (the counterparts of the reference's Waiter and of the queue behind its
// StreamingIterator, src/ksana_llm/utils/waiter.h and src/ksana_llm/endpoints/streaming/streaming_iterator.cpp):
//  * Waiter: "this request is finished" - set once by the engine's loop thread, awaited by the thread that serves the
//    client;
//  * StreamChannel: the per-step outputs of a streaming request, pushed by the loop thread and popped by the serving
//    thread, closed by the engine when the request ends.
// Both block on a condition variable with the interpreter lock released, so a server thread that waits for tokens
// costs the loop thread nothing. Items of a channel are opaque handles (the binding stores Python objects).
#pragma once
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <utility>

namespace ksana {

class Waiter {
 public:
  void Set() {
    {
      std::lock_guard<std::mutex> g(mu_);
      set_ = true;
    }
    cv_.notify_all();
  }
  void Clear() {
    std::lock_guard<std::mutex> g(mu_);
    set_ = false;
  }
  bool IsSet() {
    std::lock_guard<std::mutex> g(mu_);
    return set_;
  }
  // timeout_ms < 0: no limit. Returns whether the waiter is set.
  bool Wait(long long timeout_ms) {
    std::unique_lock<std::mutex> lk(mu_);
    if (timeout_ms < 0) {
      cv_.wait(lk, [this] { return set_; });
      return true;
    }
    return cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [this] { return set_; });
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  bool set_ = false;
};

template <typename T>
class StreamChannel {
 public:
  void Put(T item) {
    {
      std::lock_guard<std::mutex> g(mu_);
      items_.push_back(std::move(item));
    }
    cv_.notify_one();
  }
  // Pops the oldest item into *out. timeout_ms < 0: no limit. False when the time ran out with nothing queued.
  bool Get(T* out, long long timeout_ms) {
    std::unique_lock<std::mutex> lk(mu_);
    auto ready = [this] { return !items_.empty(); };
    if (timeout_ms < 0) cv_.wait(lk, ready);
    else if (!cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), ready)) return false;
    *out = std::move(items_.front());
    items_.pop_front();
    return true;
  }
  size_t Size() {
    std::lock_guard<std::mutex> g(mu_);
    return items_.size();
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<T> items_;
};

}  // namespace ksana
