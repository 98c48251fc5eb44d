// Harness around the reference's own CPU code.  TEST INFRASTRUCTURE ONLY.
//
// oracle/Makefile generates oracle/_ref/run_cpu_part.inc at build time from
// the reference tree (run.cpp up to, not including, the getp engine includes
// at run.cpp:1121, minus the one profiler include at run.cpp:22) and compiles
// this file around it, so `matmul`, `topk`, `softmax`, `rmsnorm`, `forward`
// and `build_transformer` below are the reference's unmodified functions.
// Nothing from the reference is stored in this repository.
//
// The glue in ref_moe_layer re-states the per-token MoE section of forward()
// (run.cpp:662-750) with the layer's tensors passed in directly instead of
// being read out of a Transformer, so layer-only inputs can be fed.
#define PROFILE_SCOPE(name)
#define PROFILER_PRINT_SUMMARY()
#include "_ref/run_cpu_part.inc"
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// One MoE block over T tokens, token by token, through the reference's own
// matmul/topk/softmax.  t [T,H] post-norm input; x [T,H] residual, updated in
// place; optional taps as in the oracle.
__attribute__((visibility("default"))) int
ref_moe_layer(const float *t, float *x, const int *pos, int T, int H, int IM, int E, int K,
              const float *w_router, const float *b_router, const float *w_mlp1,
              const float *b_mlp1, const float *w_mlp2, const float *b_mlp2, float swiglu_limit,
              float *logits_out, int *topk_i_out, float *topk_v_out, float *e_agg_out) {
  float *router_score = (float *)malloc(sizeof(float) * E);
  float *topk_v = (float *)malloc(sizeof(float) * K);
  int *topk_i = (int *)malloc(sizeof(int) * K);
  float *mlp1_out = (float *)malloc(sizeof(float) * 2 * IM);
  float *gate_up = (float *)malloc(sizeof(float) * IM);
  float *tb2 = (float *)malloc(sizeof(float) * H);
  float *e_agg = (float *)malloc(sizeof(float) * H);
  for (int tok = 0; tok < T; tok++) {
    if (pos && pos[tok] < 0) continue;
    float *tv = const_cast<float *>(t) + (size_t)tok * H;
    matmul(router_score, tv, const_cast<float *>(w_router), H, E);            // run.cpp:666
    for (int i = 0; i < E; i++) router_score[i] += b_router[i];               // run.cpp:669-671
    topk(topk_v, topk_i, router_score, E, K);                                 // run.cpp:673
    softmax(topk_v, K);                                                       // run.cpp:676
    memset(e_agg, 0, sizeof(float) * H);                                      // run.cpp:679
    for (int e = 0; e < E; e++) {                                             // run.cpp:680
      float expert_w = 0;
      int in_topk = 0;
      for (int idx = 0; idx < K; idx++) {
        if (topk_i[idx] == e) {
          in_topk = 1;
          expert_w = topk_v[idx];
          break;
        }
      }
      if (!in_topk) continue;
      float *w1 = const_cast<float *>(w_mlp1) + (size_t)e * 2 * IM * H;
      const float *b1 = b_mlp1 + (size_t)e * 2 * IM;
      matmul(mlp1_out, tv, w1, H, 2 * IM);                                    // run.cpp:698
      for (int i = 0; i < 2 * IM; i++) mlp1_out[i] += b1[i];
      const float alpha = 1.702f;
      for (int i = 0; i < IM; i++) {                                          // run.cpp:703-725
        float val = mlp1_out[2 * i];
        float up_val = mlp1_out[2 * i + 1];
        if (val > swiglu_limit) val = swiglu_limit;
        if (up_val > swiglu_limit) up_val = swiglu_limit;
        if (up_val < -swiglu_limit) up_val = -swiglu_limit;
        val *= (1.0f / (1.0f + expf(-alpha * val)));
        val *= (up_val + 1.0f);
        gate_up[i] = val;
      }
      float *w2 = const_cast<float *>(w_mlp2) + (size_t)e * H * IM;
      const float *b2 = b_mlp2 + (size_t)e * H;
      matmul(tb2, gate_up, w2, IM, H);                                        // run.cpp:733
      for (int i = 0; i < H; i++) tb2[i] += b2[i];
      for (int i = 0; i < H; i++) e_agg[i] += tb2[i] * expert_w;              // run.cpp:740-742
    }
    if (logits_out) memcpy(logits_out + (size_t)tok * E, router_score, sizeof(float) * E);
    if (topk_i_out) memcpy(topk_i_out + (size_t)tok * K, topk_i, sizeof(int) * K);
    if (topk_v_out) memcpy(topk_v_out + (size_t)tok * K, topk_v, sizeof(float) * K);
    if (e_agg_out) memcpy(e_agg_out + (size_t)tok * H, e_agg, sizeof(float) * H);
    if (x)
      for (int i = 0; i < H; i++) x[(size_t)tok * H + i] += e_agg[i];         // run.cpp:747-749
  }
  free(router_score); free(topk_v); free(topk_i); free(mlp1_out); free(gate_up); free(tb2);
  free(e_agg);
  return 0;
}

// rmsnorm of the reference over a batch (run.cpp:321-334).
__attribute__((visibility("default"))) void ref_rmsnorm_rows(float *o, const float *x,
                                                             const float *w, int T, int H) {
  for (int tok = 0; tok < T; tok++)
    rmsnorm(o + (size_t)tok * H, const_cast<float *>(x) + (size_t)tok * H,
            const_cast<float *>(w), H);
}

// Whole model through the reference's forward() (run.cpp:529-758), one token at
// a time as generate() does (run.cpp:965-979): tokens[0..n_prompt) are forced,
// then greedy.  out_tokens gets n_prompt-1+n_gen next-token ids (one per
// forward call); taps of the LAST layer's MoE state after the last call are
// copied out when the pointers are non-null.
__attribute__((visibility("default"))) int
ref_model_decode(const char *bin_path, const int *tokens, int n_prompt, int n_steps,
                 int *out_tokens, float *last_logits) {
  Transformer tr;
  build_transformer(&tr, const_cast<char *>(bin_path));
  int token = tokens[0];
  for (int pos = 0; pos < n_steps; pos++) {
    float *logits = forward(&tr, token, pos);
    int next;
    if (pos < n_prompt - 1) {
      next = tokens[pos + 1];
    } else {
      next = sample_argmax(logits, tr.config.vocab_size);
    }
    out_tokens[pos] = sample_argmax(logits, tr.config.vocab_size);
    if (last_logits && pos == n_steps - 1)
      memcpy(last_logits, logits, sizeof(float) * tr.config.vocab_size);
    token = next;
  }
  free_transformer(&tr);
  return 0;
}

// Teacher-forced logits of the whole model: forward() (run.cpp:536-766) on
// tokens[pos] at pos = 0..n-1, the fp32 logits of every call copied to
// logits_out [n, vocab_size].
__attribute__((visibility("default"))) int
ref_model_logits(const char *bin_path, const int *tokens, int n, float *logits_out) {
  Transformer tr;
  build_transformer(&tr, const_cast<char *>(bin_path));
  const size_t V = tr.config.vocab_size;
  for (int pos = 0; pos < n; pos++) {
    float *logits = forward(&tr, tokens[pos], pos);
    memcpy(logits_out + (size_t)pos * V, logits, sizeof(float) * V);
  }
  free_transformer(&tr);
  return 0;
}

__attribute__((visibility("default"))) int ref_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
}
