/*
 * CPU oracle for the GPT-OSS MoE block.  TEST INFRASTRUCTURE ONLY: this file is
 * the checker for the CUDA path (tests, the smoke check and the CPU-baseline
 * timing leg of the benchmark).  The product library never links or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference CPU forward pass
 * (pmatuan/gpt-oss, run.cpp):
 *   rmsnorm      run.cpp:321-334   (double sum of squares, eps 1e-5, sqrtf)
 *   softmax      run.cpp:336-354   (double max/sum, expf in float)
 *   matmul       run.cpp:356-369   (float products, double accumulator)
 *   topk         run.cpp:388-420   (descending by value)
 *   MoE section  run.cpp:659-750   (router+bias, top-k, softmax over the
 *                                   selected, interleaved gate/up, one-sided
 *                                   gate clamp, two-sided up clamp, alpha
 *                                   1.702, (up+1), down+bias, weighted sum in
 *                                   ascending expert order, residual add)
 *
 * Parity pin: checked bit-for-bit against the reference's own compiled code
 * (oracle/_ref, built by oracle/Makefile from the reference tree) by
 * tests/test_oracle_golden.py on the committed fixtures under tests/golden/.
 *
 * Multiply-add contraction: the reference is C++ built with -O3 for an
 * FMA-capable CPU (its Makefile:31-33), where GCC's default -ffp-contract=fast
 * fuses the one float multiply-add of the path, `e_agg[i] += tb2[i] * expert_w`
 * (run.cpp:741), into an fma.  This file is compiled with -ffp-contract=off and
 * spells that fma out, so it matches the reference build bit for bit and does
 * not depend on the compiler's choice.  No other expression of the path has the
 * a*b+c form in a single precision (matmul and rmsnorm widen the float product
 * to double before adding).
 *
 * Tie order: the reference sorts with qsort(), whose order on equal keys is
 * unspecified; this restatement puts the lower expert index first, which is
 * what the reference's GPU kernel does (getp-csrc/utility/utility.cpp:305-337).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* run.cpp:321-334 */
ORACLE_API void oracle_rmsnorm(float *o, const float *x, const float *weight, int size) {
  double ss = 0.0f;
  for (int j = 0; j < size; j++) ss += x[j] * x[j];
  ss /= size;
  ss += 1e-5f;
  ss = 1.0f / sqrtf(ss);
  for (int j = 0; j < size; j++) o[j] = weight[j] * (ss * x[j]);
}

/* run.cpp:336-354 */
ORACLE_API void oracle_softmax(float *x, int size) {
  double max_val = x[0];
  for (int i = 1; i < size; i++)
    if (x[i] > max_val) max_val = x[i];
  double sum = 0.0f;
  for (int i = 0; i < size; i++) {
    x[i] = expf(x[i] - max_val);
    sum += x[i];
  }
  for (int i = 0; i < size; i++) x[i] /= sum;
}

/* run.cpp:356-369; one output row, so callers can parallelise over rows or
 * over tokens without changing any sum's order. */
static inline float dot_row(const float *w, const float *x, int n) {
  double val = 0.0f;
  for (int j = 0; j < n; j++) val += w[j] * x[j];
  return (float)val;
}

ORACLE_API void oracle_matmul(float *xout, const float *x, const float *w, int n, int d) {
  for (int i = 0; i < d; i++) xout[i] = dot_row(w + (size_t)i * n, x, n);
}

/* run.cpp:388-420; selection by repeated strict-greater scan == stable
 * descending sort, i.e. lower index first among equal values. */
ORACLE_API void oracle_topk(float *topk_values, int *topk_indices, const float *score, int n_experts,
                            int k) {
  uint8_t taken[1024];
  memset(taken, 0, sizeof(taken));
  for (int r = 0; r < k; r++) {
    int best = -1;
    for (int e = 0; e < n_experts; e++) {
      if (taken[e]) continue;
      if (best < 0 || score[e] > score[best]) best = e;
    }
    taken[best] = 1;
    topk_values[r] = score[best];
    topk_indices[r] = best;
  }
}

/* run.cpp:711-725 */
static inline float swiglu_ref(float val, float up_val, float limit) {
  const float alpha = 1.702f;
  if (val > limit) val = limit;
  if (up_val > limit) up_val = limit;
  if (up_val < -limit) up_val = -limit;
  val *= (1.0f / (1.0f + expf(-alpha * val)));
  val *= (up_val + 1.0f);
  return val;
}

/*
 * Router part only (run.cpp:662-676): logits, top-k indices, softmaxed weights.
 * t [T,H] is the post-norm input.  Rows with pos[t] < 0 are skipped (the GPU
 * engine's inactive-row convention, getp-csrc/utility/utility.cpp:281) and
 * their outputs are left untouched.
 */
ORACLE_API int oracle_router(const float *t, const int *pos, int T, int H, int E, int K,
                             const float *w_router, const float *b_router, float *logits,
                             int *topk_i, float *topk_v) {
  if (E > 1024 || K > E || K <= 0) return 1;
#pragma omp parallel for schedule(static)
  for (int tok = 0; tok < T; tok++) {
    if (pos && pos[tok] < 0) continue;
    float *lg = logits + (size_t)tok * E;
    for (int e = 0; e < E; e++) lg[e] = dot_row(w_router + (size_t)e * H, t + (size_t)tok * H, H);
    for (int e = 0; e < E; e++) lg[e] += b_router[e];
    oracle_topk(topk_v + (size_t)tok * K, topk_i + (size_t)tok * K, lg, E, K);
    oracle_softmax(topk_v + (size_t)tok * K, K);
  }
  return 0;
}

/*
 * Whole block for a batch of tokens (run.cpp:662-750 applied per token):
 *   x[tok] += sum over selected experts e (ascending e) of
 *             w_e * (W2[e] . swiglu(W1[e] . t[tok] + b1[e]) + b2[e])
 * All tensors fp32.  w_mlp1 [E,2*IM,H] has gate rows at even and up rows at odd
 * indices; w_mlp2 [E,H,IM].  Optional taps (may be NULL): logits [T,E],
 * topk_i/topk_v [T,K], e_agg [T,H] (the block output before the residual add).
 * Experts are the outer loop so each expert's weights are streamed once; every
 * per-token sum still runs in the reference's order.
 */
ORACLE_API int oracle_moe_layer(const float *t, float *x, const int *pos, int T, int H, int IM, int E,
                                int K, const float *w_router, const float *b_router,
                                const float *w_mlp1, const float *b_mlp1, const float *w_mlp2,
                                const float *b_mlp2, float swiglu_limit, float *logits_out,
                                int *topk_i_out, float *topk_v_out, float *e_agg_out) {
  if (E > 1024 || K > E || K <= 0) return 1;
  float *logits = logits_out ? logits_out : (float *)malloc((size_t)T * E * sizeof(float));
  int *topk_i = topk_i_out ? topk_i_out : (int *)malloc((size_t)T * K * sizeof(int));
  float *topk_v = topk_v_out ? topk_v_out : (float *)malloc((size_t)T * K * sizeof(float));
  float *e_agg = e_agg_out ? e_agg_out : (float *)malloc((size_t)T * H * sizeof(float));
  if (!logits || !topk_i || !topk_v || !e_agg) return 2;

  oracle_router(t, pos, T, H, E, K, w_router, b_router, logits, topk_i, topk_v);
  memset(e_agg, 0, (size_t)T * H * sizeof(float));

  for (int e = 0; e < E; e++) {
    const float *w1 = w_mlp1 + (size_t)e * 2 * IM * H;
    const float *b1 = b_mlp1 + (size_t)e * 2 * IM;
    const float *w2 = w_mlp2 + (size_t)e * H * IM;
    const float *b2 = b_mlp2 + (size_t)e * H;
#pragma omp parallel
    {
      float *act = (float *)malloc((size_t)IM * sizeof(float));
#pragma omp for schedule(dynamic, 1)
      for (int tok = 0; tok < T; tok++) {
        if (pos && pos[tok] < 0) continue;
        float expert_w = 0.f;
        int in_topk = 0;
        for (int idx = 0; idx < K; idx++) {
          if (topk_i[(size_t)tok * K + idx] == e) {
            in_topk = 1;
            expert_w = topk_v[(size_t)tok * K + idx];
            break;
          }
        }
        if (!in_topk) continue;
        const float *tv = t + (size_t)tok * H;
        for (int j = 0; j < IM; j++) {
          float gate = dot_row(w1 + (size_t)(2 * j) * H, tv, H);
          float up = dot_row(w1 + (size_t)(2 * j + 1) * H, tv, H);
          gate += b1[2 * j];
          up += b1[2 * j + 1];
          act[j] = swiglu_ref(gate, up, swiglu_limit);
        }
        float *agg = e_agg + (size_t)tok * H;
        for (int i = 0; i < H; i++) {
          float y = dot_row(w2 + (size_t)i * IM, act, IM);
          y += b2[i];
          agg[i] = fmaf(y, expert_w, agg[i]);
        }
      }
      free(act);
    }
  }

  if (x) {
#pragma omp parallel for schedule(static)
    for (int tok = 0; tok < T; tok++) {
      if (pos && pos[tok] < 0) continue;
      for (int i = 0; i < H; i++) x[(size_t)tok * H + i] += e_agg[(size_t)tok * H + i];
    }
  }
  if (!logits_out) free(logits);
  if (!topk_i_out) free(topk_i);
  if (!topk_v_out) free(topk_v);
  if (!e_agg_out) free(e_agg);
  return 0;
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
