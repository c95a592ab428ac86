// Fixed thread pool with a FIFO of tasks, and a count-down latch.
//
// The shard runs checkpoint save / load and table migration on a single
// background thread so that training calls never block on them, the same
// division of labour as the reference's AsyncTaskQueue / ThreadBarrier
// (kraken/common/async_task_queue.cc:13-52, kraken/common/thread_barrier.h:20-40).
#pragma once

#include <condition_variable>
#include <cstddef>
#include <deque>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace kb {

class Latch {
 public:
  explicit Latch(size_t count) : count_(count) {}
  void Release() {
    std::lock_guard<std::mutex> g(mu_);
    if (count_ > 0 && --count_ == 0) cv_.notify_all();
  }
  void Wait() {
    std::unique_lock<std::mutex> g(mu_);
    cv_.wait(g, [this] { return count_ == 0; });
  }
  // Returns false when the timeout expired first.
  bool WaitFor(double seconds) {
    std::unique_lock<std::mutex> g(mu_);
    return cv_.wait_for(g, std::chrono::duration<double>(seconds), [this] { return count_ == 0; });
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  size_t count_;
};

class TaskQueue {
 public:
  explicit TaskQueue(size_t threads = 1) {
    for (size_t i = 0; i < threads; ++i) workers_.emplace_back([this] { Run(); });
  }
  ~TaskQueue() { Stop(); }

  void Enqueue(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) return;
      tasks_.push_back(std::move(fn));
      ++pending_;
    }
    cv_.notify_one();
  }
  // Blocks until every task enqueued so far has finished.
  void Drain() {
    std::unique_lock<std::mutex> g(mu_);
    idle_.wait(g, [this] { return pending_ == 0; });
  }
  size_t Pending() {
    std::lock_guard<std::mutex> g(mu_);
    return pending_;
  }
  void Stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_)
      if (t.joinable()) t.join();
  }

 private:
  void Run() {
    for (;;) {
      std::function<void()> fn;
      {
        std::unique_lock<std::mutex> g(mu_);
        cv_.wait(g, [this] { return stop_ || !tasks_.empty(); });
        if (tasks_.empty()) return;  // stop requested and nothing left
        fn = std::move(tasks_.front());
        tasks_.pop_front();
      }
      try {
        fn();
      } catch (...) {
        // A failed background task must not take the process down; the
        // submitter observes failure through its own result object.
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        if (--pending_ == 0) idle_.notify_all();
      }
    }
  }

  std::mutex mu_;
  std::condition_variable cv_, idle_;
  std::deque<std::function<void()>> tasks_;
  std::vector<std::thread> workers_;
  size_t pending_ = 0;
  bool stop_ = false;
};

}  // namespace kb
