// Rank-agreed termination for expert-parallel stepping inside one process.
//
// Under expert parallelism every GPU takes part in every layer of every decode step: a
// GPU that has finished its own sequences still owns experts that the others' tokens are
// routed to.  The reference lets a home thread leave its step loop as soon as its own
// batch is done (getp-csrc/getp_run.cpp:942-943) while the owners' rendezvous counts on
// every home (getp-csrc/expert.cpp:145-171) - a latent hang once the GPUs' request lists
// differ in length.  Here the threads agree before each step: each one says whether it
// still has work, all of them learn whether anybody has, and they all step (the idle ones
// with an empty batch) or all stop.
//
// Plain C++17, no CUDA: a counting barrier on a mutex and a condition variable.  The cost
// is one wake-up per decode step, microseconds against a step of milliseconds.
#ifndef GPTOSS_STEP_AGREEMENT_H
#define GPTOSS_STEP_AGREEMENT_H

#include <condition_variable>
#include <mutex>

namespace gptoss_host {

class StepAgreement {
 public:
  explicit StepAgreement(int participants) : n_(participants) {}

  // Called by every participant before each step with "I still have work".  Returns
  // whether ANY participant has: true = everybody runs one more step, false = everybody
  // stops.  All participants get the same answer for the same round.
  bool another_step(bool have_work) {
    std::unique_lock<std::mutex> lk(m_);
    const long long round = round_;
    any_ = any_ || have_work;
    if (++arrived_ == n_) {
      decision_ = any_;
      any_ = false;
      arrived_ = 0;
      ++round_;
      cv_.notify_all();
      return decision_;
    }
    cv_.wait(lk, [&] { return round_ != round || failed_; });
    return failed_ ? false : decision_;
  }

  // A participant that cannot go on (an error it is about to report) releases the others:
  // every pending and future another_step() returns false.
  void fail() {
    std::lock_guard<std::mutex> lk(m_);
    failed_ = true;
    cv_.notify_all();
  }

  bool failed() {
    std::lock_guard<std::mutex> lk(m_);
    return failed_;
  }

 private:
  const int n_;
  std::mutex m_;
  std::condition_variable cv_;
  int arrived_ = 0;
  long long round_ = 0;
  bool any_ = false, decision_ = false, failed_ = false;
};

}  // namespace gptoss_host

#endif  // GPTOSS_STEP_AGREEMENT_H
