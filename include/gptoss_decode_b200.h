/*
 * gptoss_decode_b200.h - C ABI of the batched greedy decode step around the MoE block.
 *
 * One call = one token for each of up to max_batch sequences: embedding gather,
 * and per layer RMSNorm, QKV projection + bias, YaRN rotary embedding, KV-cache
 * append, attention over the cache with a per-head sink logit (128-token sliding
 * window on even layers), output projection + bias + residual, RMSNorm, the MoE
 * block (gptoss_moe_b200.h), then the final RMSNorm, the logits and their argmax.
 * It replaces gpu_forward_device_batch of the reference's getp engine
 * (getp-csrc/getp_run.cpp:501-894) and computes what forward() computes for one
 * sequence (run.cpp:536-766), for every row of the batch.
 *
 * The QKV and attention-output projections and the logits run on the library's
 * tcgen05 CTA-pair kernel (the grouped GEMM of the MoE block with one group: bias in
 * the epilogue, bf16 output; fp32 output for the logits, which the argmax needs in
 * fp32).  Shapes that kernel does not take (projection rows that are not multiples of
 * 8 elements, a vocabulary that is not a multiple of 4) fall back to cuBLAS, loaded
 * with dlopen on first need.  Activations between kernels: the residual stream, the normalised
 * rows and the projection outputs are bf16, q and the logits fp32, the KV cache bf16.
 */
#ifndef GPTOSS_DECODE_B200_H
#define GPTOSS_DECODE_B200_H

#include "gptoss_moe_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The reference's Config, which is also the header of the .bin checkpoint
 * (run.cpp:26-46): 15 four-byte fields in this order. */
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
} gptoss_model_config_t;

/* The reference's TransformerWeights (run.cpp:48-84): fp32 tensors on the host,
 * normally pointers into the mmap of the .bin file.  Shapes as in run.cpp:207-248. */
typedef struct {
  const float *token_embedding_table; /* [V, H] */
  const float *rms_attn_w;            /* [L, H] */
  const float *rms_ffn_w;             /* [L, H] */
  const float *w_qkv;                 /* [L, (Hq + 2 Hkv) D, H], rows q | k | v */
  const float *w_o;                   /* [L, H, Hq D] */
  const float *b_qkv;                 /* [L, (Hq + 2 Hkv) D] */
  const float *b_o;                   /* [L, H] */
  const float *attn_sinks;            /* [L, Hq] */
  const float *w_router;              /* [L, E, H] */
  const float *b_router;              /* [L, E] */
  const float *w_mlp1;                /* [L, E, 2 IM, H], gate rows even, up rows odd */
  const float *w_mlp2;                /* [L, E, H, IM] */
  const float *b_mlp1;                /* [L, E, 2 IM] */
  const float *b_mlp2;                /* [L, E, H] */
  const float *rms_out_w;             /* [H] */
  const float *out;                   /* [V, H] unembedding */
} gptoss_model_weights_t;

typedef struct gptoss_decode gptoss_decode_t;

/* Number of visible CUDA devices of compute capability 10.x (0 when there is none or
 * no driver). */
int gptoss_decode_device_count(void);

/* Allocates everything for max_batch sequences of up to cfg->seq_len positions on
 * `device` (KV cache: L * max_batch * seq_len * Hkv * D * 2 bf16).  No CPU
 * fallback: fails unless the device is sm_100. */
int gptoss_decode_create(const gptoss_model_config_t *cfg, int max_batch, int device,
                         gptoss_decode_t **out);
/* The same with the experts sharded over ep_size ranks (expert e on rank e % ep_size,
 * everything else replicated; getp-csrc/expert.cpp:709-1018).  After creation every
 * rank calls gptoss_moe_ep_init(gptoss_decode_moe(h), id); the ranks then step in lock
 * step, each on its own batch. */
int gptoss_decode_create_ep(const gptoss_model_config_t *cfg, int max_batch, int device,
                            int ep_rank, int ep_size, gptoss_decode_t **out);
int gptoss_decode_destroy(gptoss_decode_t *h);
/* Error text of the last failed call on this handle (or of the last failed create
 * when h is NULL). */
const char *gptoss_decode_last_error(const gptoss_decode_t *h);

/* Converts and uploads every tensor (fp32 host -> bf16 device, biases and norm
 * scales stay fp32); replaces init_device_context (getp_run.cpp:150-302). */
int gptoss_decode_load_weights(gptoss_decode_t *h, const gptoss_model_weights_t *w);
/* The same from the address of the first tensor of a .bin image (file base + 60
 * bytes), tensors in the file's order (memory_map_weights, run.cpp:207-248). */
int gptoss_decode_load_bin(gptoss_decode_t *h, const float *first_tensor);

/* One tensor at a time, for models too large for a host image: name = a field of
 * gptoss_model_weights_t outside the MoE block ("token_embedding_table", "out",
 * "rms_out_w"; per layer "w_qkv", "b_qkv", "w_o", "b_o", "attn_sinks", "rms_attn_w",
 * "rms_ffn_w"), src = that tensor (one layer of it) as fp32 on the host, or on the
 * device as bf16 (weights) / fp32 (biases, scales, sinks).  The MoE tensors go through
 * gptoss_moe_load_layer_* on gptoss_decode_moe(h). */
int gptoss_decode_set_tensor(gptoss_decode_t *h, const char *name, int layer, const void *src,
                             int on_device, int is_bf16);
/* Writes K and V (bf16 device arrays [n_rows, n_pos, Hkv * D], K already rotated) into
 * the cache of `layer` for rows row0.. and positions pos0..: a context without running
 * the prompt (benchmarks with synthetic contexts). */
int gptoss_decode_set_kv(gptoss_decode_t *h, int layer, int row0, int n_rows, int pos0, int n_pos,
                         const void *k_dev, const void *v_dev);
/* The reverse: copies that region of the cache out (moving a sequence to another row or
 * another engine). */
int gptoss_decode_get_kv(gptoss_decode_t *h, int layer, int row0, int n_rows, int pos0, int n_pos,
                         void *k_dev, void *v_dev);

/* One step.  tokens[i] / pos[i]: the token to feed to batch row i and its position
 * (host arrays); pos[i] < 0 marks a row that does no work (its cache is untouched
 * and next[i] = -1), the reference's inactive-row rule.  Row i owns KV-cache slot
 * i; a sequence starts over simply by feeding pos 0 again.  next[i] receives the
 * argmax of the row's logits (lowest index among equals, sample_argmax,
 * run.cpp:780-791).  Synchronises the stream before returning. */
int gptoss_decode_step(gptoss_decode_t *h, const int *tokens, const int *pos, int batch,
                       int *next, void *stream);
/* fp32 logits [vocab_size] of batch row `row` from the last step. */
int gptoss_decode_get_logits(gptoss_decode_t *h, int row, float *logits_host);
/* The MoE engine inside (for its options, taps and stage timers). */
gptoss_moe_t *gptoss_decode_moe(gptoss_decode_t *h);

#ifdef __cplusplus
}
#endif
#endif /* GPTOSS_DECODE_B200_H */
