// warm_up / inference / finish of the getp mode on B200: the host side of the engine,
// C++17, no CUDA in this file - it drives the extern "C" layer of
// include/gptoss_decode_b200.h.
//
// Takes the place of getp-csrc/getp_run.cpp of the reference, with its behaviour at the
// boundary:
//   warm_up    one engine per GPU, every weight converted and uploaded once, all device
//              memory allocated for the largest batch (getp_run.cpp:413-446).  With more
//              than one GPU and 128 experts - or GETP_FORCE_EP set, the reference's own
//              switch - the experts are sharded over the GPUs (expert e on GPU e % n,
//              getp_run.cpp:426-432, expert.cpp:1176-1231) and everything else is
//              replicated; otherwise every GPU holds the whole model.
//   inference  prompts encoded with the host program's tokenizer; requests split evenly
//              over the GPUs, one host thread per GPU; one decode step per iteration for
//              every running sequence of the GPU; greedy (argmax) decoding; tok_gens row
//              i = generated ids terminated by -1; returns the number of generated tokens
//              (getp_run.cpp:457-499, :896-1009, :1011-1074).  A row that ends is given to
//              the next waiting request at once (continuous batching); GPTOSS_GETP_STATIC=1
//              keeps the reference's static batches, where finished sequences stay in
//              place as inactive rows until the whole batch is done.  The generated
//              tokens are the same either way.
//   finish     frees everything (getp_run.cpp:448-455)
// Under expert parallelism the GPUs step in lock step: before every decode step the
// threads agree on whether anybody still has work (step_agreement.h), and a GPU that has
// run out of requests keeps stepping with an empty batch, because its experts still
// serve the others' tokens.  (The reference's thread leaves its loop, getp_run.cpp:942,
// and the owners then wait for it forever, expert.cpp:145-171.)
// Errors end the process with a message on stderr, as the reference does
// (getp-csrc/common/defines.h:94-102).
//
// Environment: GPTOSS_GETP_GPUS (default: all sm_100 devices), GPTOSS_GETP_BATCH
// (sequences per GPU batch; default 896, or 768 with 128 experts, the reference's
// MAX_BATCH_SIZE / MAX_BATCH_SIZE_120B, defines.h:30-31), GETP_FORCE_EP (expert
// parallelism also with fewer than 128 experts, getp_run.cpp:426), GPTOSS_GETP_STATIC
// (1 = the reference's static batches instead of continuous batching).
#include "getp_abi.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "../../include/gptoss_decode_b200.h"
#include "step_agreement.h"

namespace {

// Ids that end a sequence (getp_run.cpp:977) and the step limit per request
// (getp_run.cpp:463).
constexpr int kEosA = 199999, kEosB = 200002;
constexpr int kMaxSteps = 1024;

struct Sequence {
  std::vector<int> prompt;
  int *out = nullptr;  // the request's row of tok_gens
  int out_cap = 0;     // ids that fit before the terminator
  int pos = 0, token = 0, generated = 0;
};

struct Device {
  gptoss_decode_t *engine = nullptr;
  int batch = 0;
};

std::vector<Device> g_devices;
bool g_expert_parallel = false;

[[noreturn]] void die(const char *what, const char *detail) {
  std::fprintf(stderr, "getp (B200): %s: %s\n", what, detail ? detail : "");
  std::exit(EXIT_FAILURE);
}

int env_int(const char *name, int fallback) {
  const char *v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : fallback;
}

// One GPU's share of the requests.  The GPU's rows are slots: a request takes a free slot,
// decodes there one position per step, and gives the slot back when it ends; the next
// waiting request starts in it at position 0 in the following step (continuous batching:
// a row's KV-cache slot simply starts over).  With `static_batches` the reference's
// schedule is kept instead: a new batch starts only when every sequence of the previous
// one has ended (getp_run.cpp:896-1009), finished sequences idling as inactive rows.
// The tokens a request generates are the same either way - rows do not see each other.
// `agree` (expert parallelism) makes the GPUs step together; without it the GPU runs on
// its own.
long long run_on_device(Device &dev, const Config &cfg, Sequence *seqs, int count,
                        gptoss_host::StepAgreement *agree, bool static_batches) {
  long long total = 0;
  const int slots = dev.batch;
  std::vector<int> tokens(slots), pos(slots), next(slots);
  std::vector<Sequence *> row(slots, nullptr);
  int next_request = 0, running = 0, rows_in_use = 0;
  auto retire = [&](int i) {
    Sequence &s = *row[i];
    const int n = std::min(s.generated, s.out_cap);
    s.out[n] = -1;
    total += n;
    row[i] = nullptr;
    running--;
  };
  while (true) {
    // hand free slots to waiting requests
    if (static_batches) {
      if (running == 0 && next_request < count) {
        rows_in_use = std::min(slots, count - next_request);
        for (int i = 0; i < rows_in_use; i++) row[i] = &seqs[next_request++];
        running = rows_in_use;
      }
    } else {
      for (int i = 0; i < slots && next_request < count; i++) {
        if (!row[i]) {
          row[i] = &seqs[next_request++];
          running++;
          rows_in_use = std::max(rows_in_use, i + 1);
        }
      }
      while (rows_in_use > 0 && !row[rows_in_use - 1]) rows_in_use--;
    }
    const bool have_work = running > 0;
    if (agree ? !agree->another_step(have_work) : !have_work) break;
    int rows;
    if (have_work) {
      rows = rows_in_use;
      for (int i = 0; i < rows; i++) {
        tokens[i] = row[i] ? row[i]->token : -1;
        pos[i] = row[i] ? row[i]->pos : -1;
      }
    } else {
      // nothing of its own left: one inactive row, so that this GPU's experts still
      // take part in the step the others are making
      rows = 1;
      tokens[0] = -1;
      pos[0] = -1;
    }
    if (gptoss_decode_step(dev.engine, tokens.data(), pos.data(), rows, next.data(), nullptr) !=
        GPTOSS_OK) {
      if (agree) agree->fail();
      die("decode step", gptoss_decode_last_error(dev.engine));
    }
    if (!have_work) continue;
    for (int i = 0; i < rows; i++) {
      if (!row[i]) continue;
      Sequence &s = *row[i];
      s.pos++;
      int tok;
      if (s.pos < static_cast<int>(s.prompt.size())) {
        tok = s.prompt[s.pos];  // still feeding the prompt
      } else {
        tok = next[i];
        if (s.generated < s.out_cap) s.out[s.generated] = tok;
        s.generated++;
      }
      s.token = tok;
      const bool eos = tok == kEosA || tok == kEosB;
      // also stop where the caller's output row or the KV cache would overflow
      // (the reference checks neither)
      if (eos || s.pos + 1 >= kMaxSteps || s.pos + 1 >= cfg.seq_len || s.generated >= s.out_cap)
        retire(i);
    }
  }
  return total;
}

}  // namespace

void warm_up(Transformer *transformer, Tokenizer *) {
  const Config &cfg = transformer->config;
  const auto t0 = std::chrono::steady_clock::now();
  int n_gpus = gptoss_decode_device_count();
  if (n_gpus <= 0) die("warm_up", "no sm_100 GPU visible (there is no CPU fallback)");
  n_gpus = std::min(n_gpus, std::max(1, env_int("GPTOSS_GETP_GPUS", n_gpus)));
  const int batch = std::max(1, env_int("GPTOSS_GETP_BATCH", cfg.n_experts >= 128 ? 768 : 896));
  // the reference's rule (getp_run.cpp:426); at most 8 GPUs share the experts here
  g_expert_parallel = n_gpus > 1 && (cfg.n_experts == 128 || std::getenv("GETP_FORCE_EP") != nullptr);
  if (g_expert_parallel && (n_gpus > 8 || cfg.n_experts % n_gpus != 0))
    die("warm_up", "expert parallelism needs 2..8 GPUs that divide the expert count");
  static_assert(sizeof(Config) == sizeof(gptoss_model_config_t), "checkpoint header layout");
  static_assert(sizeof(TransformerWeights) == sizeof(gptoss_model_weights_t), "weight table layout");
  gptoss_model_config_t mc;
  std::memcpy(&mc, &cfg, sizeof(mc));
  gptoss_model_weights_t mw;
  std::memcpy(&mw, &transformer->weights, sizeof(mw));
  g_devices.assign(n_gpus, Device());
  std::vector<std::thread> workers;
  std::vector<std::string> errors(n_gpus);
  for (int d = 0; d < n_gpus; d++) {
    workers.emplace_back([&, d]() {
      Device &dev = g_devices[d];
      dev.batch = batch;
      const int rc = g_expert_parallel
                         ? gptoss_decode_create_ep(&mc, batch, d, d, n_gpus, &dev.engine)
                         : gptoss_decode_create(&mc, batch, d, &dev.engine);
      if (rc != GPTOSS_OK) {
        errors[d] = std::string("create: ") + gptoss_decode_last_error(nullptr);
        return;
      }
      // under expert parallelism only this GPU's experts are converted and uploaded
      if (gptoss_decode_load_weights(dev.engine, &mw) != GPTOSS_OK)
        errors[d] = std::string("weights: ") + gptoss_decode_last_error(dev.engine);
    });
  }
  for (auto &w : workers) w.join();
  for (int d = 0; d < n_gpus; d++)
    if (!errors[d].empty()) die("warm_up", errors[d].c_str());
  if (g_expert_parallel) {
    std::vector<gptoss_moe_t *> moes(n_gpus);
    for (int d = 0; d < n_gpus; d++) moes[d] = gptoss_decode_moe(g_devices[d].engine);
    if (gptoss_moe_ep_init_local(moes.data(), n_gpus) != GPTOSS_OK) {
      const char *text = gptoss_moe_last_error(nullptr);
      for (int d = 0; d < n_gpus; d++)
        if (*gptoss_moe_last_error(moes[d])) text = gptoss_moe_last_error(moes[d]);
      die("warm_up (expert parallelism)", text);
    }
  }
  const double sec =
      std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::printf("getp (B200): %d GPU(s), batch %d per GPU, %s, warm-up %.2f s\n", n_gpus, batch,
              g_expert_parallel ? "experts sharded over the GPUs" : "one replica per GPU", sec);
}

long long inference(Transformer *transformer, Tokenizer *tokenizer, Sampler *, Requests *requests) {
  if (g_devices.empty()) die("inference", "warm_up has not run");
  const Config &cfg = transformer->config;
  const int n = requests->num_reqs;
  if (n <= 0) return 0;
  std::vector<Sequence> seqs(n);
  const size_t text_stride = static_cast<size_t>(requests->max_token_len) * (requests->max_seq_len + 1);
  for (int i = 0; i < n; i++) {
    Sequence &s = seqs[i];
    const char *text = requests->str_reqs + i * text_stride;
    s.out = requests->tok_gens + static_cast<size_t>(i) * (requests->max_seq_len + 1);
    s.out_cap = requests->max_seq_len;
    s.prompt.resize(std::strlen(text) + 3);
    int count = 0;
    encode(tokenizer, text, -1, -1, s.prompt.data(), &count, cfg.initial_context_length);
    if (count < 1) die("inference", "a request encoded to no tokens");
    s.prompt.resize(count);
    s.token = s.prompt[0];
  }
  // contiguous, near-equal shares, the first (n % gpus) one request longer
  const int gpus = static_cast<int>(g_devices.size());
  std::vector<long long> totals(gpus, 0);
  std::vector<std::thread> workers;
  std::unique_ptr<gptoss_host::StepAgreement> agree;
  if (g_expert_parallel) agree.reset(new gptoss_host::StepAgreement(gpus));
  const bool static_batches = env_int("GPTOSS_GETP_STATIC", 0) != 0;
  int start = 0;
  for (int d = 0; d < gpus; d++) {
    const int share = n / gpus + (d < n % gpus ? 1 : 0);
    // under expert parallelism a GPU without requests still steps with the others
    if (share > 0 || g_expert_parallel)
      workers.emplace_back([&, d, start, share]() {
        totals[d] = run_on_device(g_devices[d], cfg, seqs.data() + start, share, agree.get(),
                                  static_batches);
      });
    start += share;
  }
  for (auto &w : workers) w.join();
  long long total = 0;
  for (long long t : totals) total += t;
  return total;
}

void finish(Transformer *, Tokenizer *) {
  // every thread of inference() has been joined: all streams are idle, which is what
  // engines that read each other's memory need before any of them is destroyed
  for (Device &d : g_devices) gptoss_decode_destroy(d.engine);
  g_devices.clear();
  g_expert_parallel = false;
}
