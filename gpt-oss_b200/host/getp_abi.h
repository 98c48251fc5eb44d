// Types that cross the getp entry points, laid out as the host program defines them.
//
// The reference builds its getp engine into the host program as one translation unit,
// so warm_up / inference / finish see the program's own Transformer, Tokenizer, Sampler
// and Requests (run.cpp:26-120, :765-778; tokenizer.hpp:11-29; getp-csrc/getp_eval.cpp:9-15).
// A separately compiled engine needs the same layouts; they are restated here field for
// field.  A host that already has these definitions in scope defines
// GPTOSS_GETP_HOST_TYPES before including this header and keeps its own.
#ifndef GPTOSS_GETP_ABI_H
#define GPTOSS_GETP_ABI_H

#include <sys/types.h>

#ifndef GPTOSS_GETP_HOST_TYPES

// run.cpp:26-46: model shape; also the 60-byte header of the .bin file
typedef struct {
  int vocab_size;
  int hidden_dim;
  int n_experts;
  int experts_per_token;
  int intermediate_dim;
  int n_layers;
  int head_dim;
  int n_attn_heads;
  int n_kv_heads;
  int seq_len;
  int initial_context_length;
  float rope_theta;
  float rope_scaling_factor;
  int sliding_window;
  float swiglu_limit;
} Config;

// run.cpp:48-84: fp32 tensors, pointers into the mapped checkpoint
typedef struct {
  float *token_embedding_table;
  float *rms_attn_w;
  float *rms_ffn_w;
  float *w_qkv;
  float *w_o;
  float *b_qkv;
  float *b_o;
  float *attn_sinks;
  float *w_router;
  float *b_router;
  float *w_mlp1;
  float *w_mlp2;
  float *b_mlp1;
  float *b_mlp2;
  float *rms_out_w;
  float *out;
} TransformerWeights;

// run.cpp:86-111: the CPU path's activation buffers; the engine never touches them
typedef struct {
  float *x, *t, *tb, *tb2, *router_score, *topk_v;
  int *topk_i;
  float *mlp1_out, *gate, *up, *gate_up, *e_agg, *qkv, *q, *k, *v, *att, *logits;
  float *key_cache, *value_cache, *mask;
} RunState;

// run.cpp:113-120
typedef struct {
  Config config;
  TransformerWeights weights;
  RunState state;
  int fd;
  float *data;
  ssize_t file_size;
} Transformer;

// tokenizer.hpp:11-29
typedef struct {
  const char *str;
  int len;
  int id;
} TokenIndex;
typedef struct {
  char **vocab;
  int *lengths;
  float *scores;
  int vocab_size;
  int max_token_length;
  TokenIndex *sorted_vocab;
  int byte_tokens[256];
  unsigned char byte_pieces[512];
} Tokenizer;

// run.cpp:765-778
typedef struct {
  float prob;
  int index;
} ProbIndex;
typedef struct {
  int vocab_size;
  ProbIndex *probindex;
  float temperature;
  float topp;
  unsigned long long rng_state;
} Sampler;

// getp-csrc/getp_eval.cpp:9-15; row i of str_reqs has max_token_len * (max_seq_len + 1)
// bytes, row i of tok_gens max_seq_len + 1 ints (getp_eval.cpp:35-41)
typedef struct {
  int num_reqs;
  int max_token_len;
  int max_seq_len;
  char *str_reqs;
  int *tok_gens;
} Requests;

#endif  // GPTOSS_GETP_HOST_TYPES

// The host program's tokenizer (tokenizer.hpp:47-48); the engine only encodes prompts.
void encode(Tokenizer *t, const char *text, int bos_id, int eos_id, int *out, int *n_out,
            int max_tokens);

// The three entry points the host's getp() calls (getp-csrc/getp_eval.cpp:100-103, :124-146).
void warm_up(Transformer *transformer, Tokenizer *tokenizer);
void finish(Transformer *transformer, Tokenizer *tokenizer);
long long inference(Transformer *transformer, Tokenizer *tokenizer, Sampler *sampler,
                    Requests *requests);

#endif  // GPTOSS_GETP_ABI_H
