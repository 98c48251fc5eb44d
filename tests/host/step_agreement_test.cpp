// CPU test of the rank-agreed termination used under expert parallelism
// (gpt-oss_b200/host/step_agreement.h): host threads with different amounts of work must
// all make the same number of steps - the longest one's - and stop together; a failing
// participant releases the others.
// usage: step_agreement_test  (prints "ok" and exits 0, or a message and exits 1)
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "../../gpt-oss_b200/host/step_agreement.h"

static int run_case(const std::vector<int> &work) {
  const int n = static_cast<int>(work.size());
  gptoss_host::StepAgreement agree(n);
  std::vector<int> steps(n, 0), idle_steps(n, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < n; r++)
    th.emplace_back([&, r]() {
      int left = work[r];
      while (agree.another_step(left > 0)) {
        steps[r]++;
        if (left > 0)
          left--;
        else
          idle_steps[r]++;
        if ((steps[r] + r) % 7 == 0) std::this_thread::yield();
      }
    });
  for (auto &t : th) t.join();
  int longest = 0;
  for (int w : work) longest = w > longest ? w : longest;
  for (int r = 0; r < n; r++) {
    if (steps[r] != longest || idle_steps[r] != longest - work[r]) {
      std::fprintf(stderr, "rank %d of %d: %d steps (%d idle), expected %d (%d idle)\n", r, n,
                   steps[r], idle_steps[r], longest, longest - work[r]);
      return 1;
    }
  }
  return 0;
}

int main() {
  if (run_case({5, 5}) || run_case({0, 9}) || run_case({1000, 3, 0, 517}) ||
      run_case({0, 0, 0}) || run_case({1, 2, 3, 4, 5, 6, 7, 8}))
    return 1;
  // a participant that gives up releases the ones that wait for it
  {
    gptoss_host::StepAgreement agree(3);
    std::atomic<int> released{0};
    std::vector<std::thread> th;
    for (int r = 0; r < 2; r++)
      th.emplace_back([&]() {
        while (agree.another_step(true)) {
        }
        released++;
      });
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
    agree.fail();  // the third participant never arrives
    for (auto &t : th) t.join();
    if (released != 2 || !agree.failed()) {
      std::fprintf(stderr, "fail() did not release the waiting threads\n");
      return 1;
    }
  }
  std::puts("ok");
  return 0;
}
