// Test host for the getp entry points: plays the part of the reference's main() + getp()
// (run.cpp:1239-1241, getp-csrc/getp_eval.cpp:105-154) around warm_up / inference /
// finish, with two stand-ins for what is not available offline:
//   * the tokenizer: prompts are lines of decimal token ids, and encode() parses them
//     (the reference's tokenizer needs the o200k vocabulary file);
//   * the checkpoint reader: the .bin image is mapped and the weight table filled in the
//     file's tensor order (run.cpp:207-248).
// usage: getp_harness model.bin requests.txt output.txt [steps]
//   requests.txt: first line = number of requests, then one prompt per line
//   output.txt:   one line per request, the generated ids separated by spaces
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "../../gpt-oss_b200/host/getp_abi.h"

void encode(Tokenizer *, const char *text, int, int, int *out, int *n_out, int max_tokens) {
  int n = 0;
  const char *p = text;
  while (*p && n < max_tokens) {
    char *end = nullptr;
    const long v = std::strtol(p, &end, 10);
    if (end == p) break;
    out[n++] = static_cast<int>(v);
    p = end;
  }
  *n_out = n;
}

int main(int argc, char **argv) {
  if (argc < 4) {
    std::fprintf(stderr, "usage: %s model.bin requests.txt output.txt [steps]\n", argv[0]);
    return 2;
  }
  Transformer tr;
  std::memset(&tr, 0, sizeof(tr));
  tr.fd = open(argv[1], O_RDONLY);
  struct stat st;
  if (tr.fd < 0 || fstat(tr.fd, &st) != 0) {
    std::perror(argv[1]);
    return 1;
  }
  tr.file_size = st.st_size;
  void *image = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, tr.fd, 0);
  if (image == MAP_FAILED) {
    std::perror("mmap");
    return 1;
  }
  tr.data = static_cast<float *>(image);
  std::memcpy(&tr.config, image, sizeof(Config));
  const Config &c = tr.config;
  const size_t V = c.vocab_size, H = c.hidden_dim, L = c.n_layers, D = c.head_dim, E = c.n_experts;
  const size_t IM = c.intermediate_dim, dq = c.n_attn_heads * D, dqkv = dq + 2 * c.n_kv_heads * D;
  float *p = tr.data + sizeof(Config) / sizeof(float);
  TransformerWeights &w = tr.weights;
  w.token_embedding_table = p; p += V * H;
  w.out = p;                   p += V * H;
  w.rms_attn_w = p;            p += L * H;
  w.rms_ffn_w = p;             p += L * H;
  w.rms_out_w = p;             p += H;
  w.w_qkv = p;                 p += L * dqkv * H;
  w.b_qkv = p;                 p += L * dqkv;
  w.w_o = p;                   p += L * H * dq;
  w.b_o = p;                   p += L * H;
  w.attn_sinks = p;            p += L * c.n_attn_heads;
  w.w_router = p;              p += L * E * H;
  w.b_router = p;              p += L * E;
  w.w_mlp1 = p;                p += L * E * 2 * IM * H;
  w.b_mlp1 = p;                p += L * E * 2 * IM;
  w.w_mlp2 = p;                p += L * E * H * IM;
  w.b_mlp2 = p;                p += L * E * H;
  if (static_cast<size_t>(reinterpret_cast<char *>(p) - static_cast<char *>(image)) !=
      static_cast<size_t>(st.st_size)) {
    std::fprintf(stderr, "checkpoint size does not match its header\n");
    return 1;
  }

  int steps = argc > 4 ? std::atoi(argv[4]) : 0;
  if (steps <= 0 || steps > c.seq_len) steps = c.seq_len;
  std::ifstream in(argv[2]);
  std::string line;
  if (!std::getline(in, line)) {
    std::fprintf(stderr, "cannot read %s\n", argv[2]);
    return 1;
  }
  Requests reqs;
  reqs.num_reqs = std::atoi(line.c_str());
  reqs.max_token_len = 16;  // bytes reserved per token of request text
  reqs.max_seq_len = steps;
  const size_t stride = static_cast<size_t>(reqs.max_token_len) * (steps + 1);
  std::vector<char> text(stride * reqs.num_reqs, 0);
  std::vector<int> gens(static_cast<size_t>(steps + 1) * reqs.num_reqs, 0);
  reqs.str_reqs = text.data();
  reqs.tok_gens = gens.data();
  for (int i = 0; i < reqs.num_reqs && std::getline(in, line); i++) {
    if (line.size() >= stride) {
      std::fprintf(stderr, "request %d too long\n", i);
      return 1;
    }
    std::memcpy(text.data() + i * stride, line.data(), line.size());
  }

  Tokenizer tok;
  std::memset(&tok, 0, sizeof(tok));
  tok.max_token_length = reqs.max_token_len;
  Sampler sampler;
  std::memset(&sampler, 0, sizeof(sampler));
  warm_up(&tr, &tok);
  const long long generated = inference(&tr, &tok, &sampler, &reqs);
  std::printf("generated %lld tokens\n", generated);
  std::ofstream out(argv[3]);
  for (int i = 0; i < reqs.num_reqs; i++) {
    const int *g = gens.data() + static_cast<size_t>(i) * (steps + 1);
    for (int j = 0; g[j] >= 0; j++) out << (j ? " " : "") << g[j];
    out << '\n';
  }
  finish(&tr, &tok);
  munmap(image, st.st_size);
  close(tr.fd);
  return 0;
}
