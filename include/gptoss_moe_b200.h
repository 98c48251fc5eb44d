/*
 * C ABI of the B200 (sm_100a) GPT-OSS MoE engine.
 *
 * This is the boundary a host program binds to replace the MoE section of the
 * reference's batched ("getp") engine.  Plain C types only: device and host
 * pointers are void* / typed pointers, a CUDA stream is passed as void*
 * (cudaStream_t), every call returns 0 on success or a negative GPTOSS_E_* code
 * and gptoss_moe_last_error() gives the text.  There is no CPU fallback: every
 * compute entry point fails with GPTOSS_E_CUDA when no sm_100 device is usable.
 * A handle is used by one host thread at a time (the reference drives one
 * engine per GPU from one thread, getp_run.cpp:1038-1063); different handles are
 * independent.
 *
 * Citations are file:line in the reference project (pmatuan/gpt-oss).
 */
#ifndef GPTOSS_MOE_B200_H
#define GPTOSS_MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GPTOSS_OK 0
#define GPTOSS_E_INVALID (-1)   /* bad argument / unsupported shape            */
#define GPTOSS_E_CUDA (-2)      /* CUDA runtime or driver error                */
#define GPTOSS_E_CAPACITY (-3)  /* more tokens than the engine was created for */
#define GPTOSS_E_DEVICE (-4)    /* a kernel reported a status (bounded wait ran
                                   out, index out of range); see
                                   gptoss_moe_device_status()                  */
#define GPTOSS_E_STATE (-5)     /* call order (weights not loaded, EP not set
                                   up)                                         */
#define GPTOSS_E_COMM (-6)      /* NCCL error                                  */

#define GPTOSS_MAX_TOPK 8

typedef struct gptoss_moe gptoss_moe_t;

/* Expert weight storage on the device. */
enum { GPTOSS_WEIGHTS_BF16 = 0, GPTOSS_WEIGHTS_MXFP4 = 1 };
/* Grouped-GEMM implementation.  TCGEN05 is the product path; SIMT is a slow
 * CUDA-core kernel kept only so tests can cross-check the tensor-core path on
 * the GPU at sizes the CPU oracle cannot reach.  It is never selected
 * automatically. */
enum { GPTOSS_GEMM_TCGEN05 = 0, GPTOSS_GEMM_SIMT = 1, GPTOSS_GEMM_PAIR = 2 };
/* GPTOSS_GEMM_PAIR: the tcgen05 kernel on CTA pairs (cta_group::2) with the
 * weights as the M operand and token tiles of up to 256 as N. */

/*
 * Shape of one engine.  Field meanings follow the reference's Config
 * (run.cpp:26-46): hidden_dim, intermediate_dim, n_experts,
 * experts_per_token, n_layers, swiglu_limit.  max_tokens plays the role of
 * MAX_BATCH_SIZE (getp-csrc/common/defines.h:30-31): all device workspaces are
 * allocated once for it (getp_run.cpp:39-143).  ep_rank / ep_size select expert
 * parallelism: expert e lives on rank e % ep_size with local id e / ep_size
 * (getp-csrc/expert.cpp:18, :1191-1213); ep_size <= 1 means all experts local.
 */
typedef struct {
  int hidden_dim;
  int intermediate_dim;
  int n_experts;
  int experts_per_token;
  int n_layers;
  int max_tokens;
  float swiglu_limit;
  int ep_rank;
  int ep_size;
  int weight_format; /* GPTOSS_WEIGHTS_* */
  int device;        /* CUDA device ordinal */
} gptoss_moe_config_t;

/* Replaces init_device_context's MoE allocations (getp_run.cpp:43-68,
 * :126-143) and init_device_context_ep (expert.cpp:709). */
int gptoss_moe_create(const gptoss_moe_config_t *cfg, gptoss_moe_t **out);
/* Replaces cleanup in finish() (getp_run.cpp:315-411, expert.cpp:1234). */
int gptoss_moe_destroy(gptoss_moe_t *h);
/* Text of the last error on this handle (or of the last failed create when h
 * is NULL).  Valid until the next call on the same thread. */
const char *gptoss_moe_last_error(const gptoss_moe_t *h);

/*
 * Weight upload for one layer from the fp32 tensors of the .bin file
 * (run.cpp:237-248: w_router [E,H], b_router [E], w_mlp1 [E,2*IM,H] with gate
 * rows even / up rows odd, b_mlp1 [E,2*IM], w_mlp2 [E,H,IM], b_mlp2 [E,H]),
 * host pointers.  Weights are rounded to bf16 (round-to-nearest-even, as
 * copy_fp32_to_bf16_device does, getp-csrc/utility/utility.cpp:417-556);
 * biases stay fp32.  Under expert parallelism only the experts this rank owns
 * are uploaded (expert.cpp:895-930, :971-1009); pointers still address the full
 * [E,...] tensors.
 */
int gptoss_moe_load_layer_f32(gptoss_moe_t *h, int layer, const float *w_router,
                              const float *b_router, const float *w_mlp1, const float *b_mlp1,
                              const float *w_mlp2, const float *b_mlp2);
/*
 * Same tensors already in bf16 (uint16 bit patterns), biases fp32.
 * on_device != 0: all pointers are device pointers on the engine's device and
 * are copied device-to-device.  Full [E,...] tensors as above.
 */
int gptoss_moe_load_layer_bf16(gptoss_moe_t *h, int layer, const void *w_router,
                               const float *b_router, const void *w_mlp1, const float *b_mlp1,
                               const void *w_mlp2, const float *b_mlp2, int on_device);
/*
 * Expert weights as MXFP4 (engine created with GPTOSS_WEIGHTS_MXFP4): blocks are
 * packed e2m1 codes, two per byte, low nibble = even element
 * (export_model_bin/gpt-oss-120b/export_model_bin.py:80-97, :126-131), scales
 * are e8m0 bytes (value 2^(s-127)), one per 32 consecutive elements of the
 * contraction dimension.  w_mlp1_blocks [E,2*IM,H/2], w_mlp1_scales
 * [E,2*IM,H/32], w_mlp2_blocks [E,H,IM/2], w_mlp2_scales [E,H,IM/32]; router in
 * bf16, biases fp32.  The reference stores such checkpoints dequantised; this
 * format has no counterpart file in the reference.
 */
int gptoss_moe_load_layer_mxfp4(gptoss_moe_t *h, int layer, const void *w_router_bf16,
                                const float *b_router, const uint8_t *w_mlp1_blocks,
                                const uint8_t *w_mlp1_scales, const float *b_mlp1,
                                const uint8_t *w_mlp2_blocks, const uint8_t *w_mlp2_scales,
                                const float *b_mlp2, int on_device);

/*
 * One MoE block on device buffers; replaces the MoE section of
 * gpu_forward_device_batch (getp_run.cpp:697-852: router, top-k + softmax,
 * count / scan / build assignments, mlp1, mlp2, slot reduce, residual add) and,
 * when the engine was set up for expert parallelism, gpu_forward_device_batch_ep
 * (expert.cpp:1366-1607).
 *   t   bf16 [n_tokens, H]  post-norm input (the reference's d_t)
 *   x   bf16 [n_tokens, H]  residual stream, updated in place: x += MoE(t)
 *   pos i32  [n_tokens] or NULL; rows with pos < 0 are skipped and their x is
 *       left untouched (matmul.cpp:955, utility.cpp:281)
 * All work is enqueued on `stream`; the call does not synchronise unless expert
 * parallelism needs the per-peer row counts on the host.
 */
int gptoss_moe_forward(gptoss_moe_t *h, int layer, const void *t, void *x, const int *pos,
                       int n_tokens, void *stream);
/*
 * Same block with HOST buffers: copies t, x (and pos) to the device, runs the
 * block, copies x back and waits.  This is the call a host engine that keeps
 * activations in host memory makes per layer.
 */
int gptoss_moe_forward_host(gptoss_moe_t *h, int layer, const void *t_host, void *x_host,
                            const int *pos_host, int n_tokens);

/*
 * The same for callers that stream batch after batch: submit returns once the
 * copies and kernels are queued; up to three submissions are in flight, each in
 * its own staging buffers, so the host->device copy of one batch, the kernels of
 * the previous one and the device->host copy of the one before run at the same
 * time (one stream per direction and one for the kernels).  x_host is valid
 * after gptoss_moe_forward_host_wait(h, ticket); t_host, x_host and pos_host must
 * stay untouched until then.  A fourth submit waits for the oldest.  All experts
 * local, or expert parallel over the peer-memory transport (every rank then makes
 * the same sequence of submits).  While submissions are in flight the handle's workspaces are theirs:
 * wait for every ticket before calling gptoss_moe_forward or the stage entry points
 * on the same handle (gptoss_moe_forward_host does that wait itself).  t_host may be NULL once gptoss_moe_load_ffn_norm gave the layer the
 * scale of the RMSNorm that precedes the block in the model (run.cpp:664): the
 * normalised input is then computed on the device from x, and only x crosses the
 * bus in each direction.  No counterpart in the reference, whose host loop copies, computes
 * and copies back in turn (getp_run.cpp:956-961).
 */
int gptoss_moe_forward_host_submit(gptoss_moe_t *h, int layer, const void *t_host, void *x_host,
                                   const int *pos_host, int n_tokens, int *ticket);
int gptoss_moe_forward_host_wait(gptoss_moe_t *h, int ticket);
/* fp32 [H] scale of the ffn RMSNorm of `layer` (rms_ffn_w, run.cpp:52, :664), host
 * pointer; only needed for submits with t_host == NULL. */
int gptoss_moe_load_ffn_norm(gptoss_moe_t *h, int layer, const float *scale_host);

/* The stages of gptoss_moe_forward, individually (same order). */
/* router linear + bias + top-k + softmax (matmul.cpp:945, utility.cpp:274). */
int gptoss_moe_route(gptoss_moe_t *h, int layer, const void *t, const int *pos, int n_tokens,
                     void *stream);
/* histogram, prefix sum, scatter into per-expert groups and row gather
 * (utility.cpp:1058, :758, :1079). */
int gptoss_moe_permute(gptoss_moe_t *h, const void *t, int n_tokens, void *stream);
/* grouped gate_up GEMM + bias + SwiGLU, grouped down GEMM + bias, times the
 * routing weight (matmul.cpp:1023-1431, :1470-1874). */
int gptoss_moe_experts(gptoss_moe_t *h, int layer, void *stream);
/* sum of the K expert outputs per token plus residual (utility.cpp:701-726,
 * :158-173). */
int gptoss_moe_combine(gptoss_moe_t *h, void *x, int n_tokens, void *stream);

/* ffn RMSNorm that feeds the block (rmsnorm_batch_kernel, utility.cpp:194-271):
 * out = w * x * rsqrt(mean(x^2) + 1e-5), bf16 in/out, fp32 scale w [H]. */
int gptoss_moe_rmsnorm(gptoss_moe_t *h, void *out, const void *x, const float *w_dev,
                       const int *pos, int n_tokens, void *stream);

/*
 * Debug taps of the last forward (host destination buffers, any may be NULL;
 * synchronises the device).  topk_i / topk_v [n_tokens,K] (inactive rows: -1 /
 * 0), expert_offsets [E_local+1], sorted_token [n_assignments] (row of t, in
 * per-expert order; under expert parallelism the owner's order holds rows of every
 * rank's batch: room for max_tokens * ep_size * K entries), logits [n_tokens,E] only when enabled with
 * gptoss_moe_set_option("keep_logits", 1).
 */
int gptoss_moe_get_routing(gptoss_moe_t *h, int n_tokens, int *topk_i, float *topk_v,
                           int *expert_offsets, int *sorted_token, float *logits);
/* bf16 [n_assignments, IM] activations after SwiGLU, in per-expert order. */
int gptoss_moe_get_activations(gptoss_moe_t *h, void *act_host, size_t bytes);

/* Options: "gemm_impl" (GPTOSS_GEMM_*), "keep_logits" (0/1),
 * "exact_ties" (0/1, default 1: re-evaluate near-tied router logits in fp64),
 * "router_impl" (0 = tcgen05 router, the default; 1 = the mma.sync router),
 * "ep_transport" (0/1, see gptoss_moe_ep_transport), "ep_overlap" (0/1, default 0;
 * peer-memory transport only: the owner pulls the rows of the second half of its
 * experts on a second stream while the gate_up GEMM of the first half runs;
 * "ep_gather_ctas", default 64, is the size of that second gather's grid),
 * "ep_dedup" (0/1, default 1; peer-memory transport only: a remote token that
 * has several of its experts on this rank crosses the link once and is copied
 * locally for the others),
 * "ep_push" (0/1, default 1; peer-memory transport only: the owner's down GEMM
 * stores each expert output row straight into the memory of the rank its token
 * came from, under its own tiles; 0: the rows stay at the owner and that rank's
 * combine kernel fetches them),
 * "time_stages" (0/1, see gptoss_moe_stage_ms), "dependent_launch" (0/1, default 1:
 * the layer's kernels are launched with programmatic stream serialization, so a
 * kernel's set-up overlaps its predecessor's tail), "l2_hints" (0/1, default 1:
 * the CTA-pair GEMM marks its token loads evict-last in L2 and the weight loads of
 * experts whose rows fit one token tile evict-first), "mx_tmem" (0/1, default 1;
 * MXFP4 weights, decode-sized batches: a pipeline stage carries three K blocks and the
 * expanded weights are stored into tensor memory, where the MMA reads them; 0: one K
 * block per stage, expanded into the shared-memory operand ring),
 * "wait_limit_ms" (1..60000, default 2000: how long a
 * kernel of the peer-memory transport waits for another rank's flag before it
 * gives up with status 106).  Every option leaves the results unchanged. */
int gptoss_moe_set_option(gptoss_moe_t *h, const char *name, int value);
/* Kernels launched by this handle since creation. */
long long gptoss_moe_launch_count(const gptoss_moe_t *h);
/* Reads (and clears) the device status word; 0 = no kernel reported a problem.
 * Synchronises the device.  Codes: 101-103 a bounded wait inside a kernel's
 * pipeline ran out, 104 an index was out of range, 105 tensor-memory allocation,
 * 106 another rank's flag did not arrive within "wait_limit_ms".  The calls that
 * synchronise by themselves (gptoss_moe_forward_host, gptoss_moe_forward_host_wait,
 * gptoss_decode_step) check the word and return GPTOSS_E_DEVICE when it is set. */
int gptoss_moe_device_status(gptoss_moe_t *h);
/* Average duration in milliseconds of one stage, measured with CUDA events
 * recorded on the launching stream around the stage's kernels in every call
 * made since gptoss_moe_set_option("time_stages", 1).  stage: 0 route,
 * 1 permute, 2 gate_up GEMM, 3 down GEMM, 4 combine, 5 dispatch, 6 return.
 * Waits for the last recorded event. */
int gptoss_moe_stage_ms(gptoss_moe_t *h, int stage, float *ms);

/*
 * Expert parallelism over NCCL (replaces warm_up_ep's peer setup,
 * expert.cpp:1176-1231, and the host rendezvous, expert.cpp:67-173).
 * Rank 0 fills a 128-byte id with gptoss_moe_ep_unique_id and hands it to the
 * other ranks by any means; every rank then calls gptoss_moe_ep_init.
 */
int gptoss_moe_ep_unique_id(void *id128);
int gptoss_moe_ep_init(gptoss_moe_t *h, const void *id128);
/*
 * The same for a host that drives all GPUs from one process with a thread per GPU,
 * as the reference does (getp_run.cpp:1038-1063, warm_up_ep expert.cpp:1176-1231):
 * engines[r] was created with ep_rank r and ep_size n_engines, each on its own
 * device.  Called once, from one thread, before any forward: enables peer access
 * between the devices and hands every engine the others' buffers as plain
 * pointers - no NCCL, no IPC.  Only the peer-memory transport exists then.  The
 * engines must be destroyed together, after all of their streams are idle.
 * Fails (on every engine alike) when the engines differ in max_tokens, hidden
 * size, expert count or top-k; gptoss_moe_ep_init makes the same check across
 * processes.
 */
int gptoss_moe_ep_init_local(gptoss_moe_t *const *engines, int n_engines);
/*
 * gptoss_moe_forward under expert parallelism over peer memory, one part at a time:
 * part 0 = router + publish (needs t, pos), 1 = owner stage (waits for every
 * rank's part 0), 2 = combine into x (waits for every rank's part 1).  For a host
 * that runs several ranks through ONE stream - every rank's part 0, then every
 * rank's part 1, then every rank's part 2 - so that no kernel is ever launched
 * before the kernels whose flags it polls; that is also the only way ranks may
 * share a GPU.  (The reference's counterpart is the three phases of
 * gpu_forward_device_batch_ep, expert.cpp:1432-1478, :1480-1552, :1554-1605.)
 */
int gptoss_moe_forward_part(gptoss_moe_t *h, int layer, int part, const void *t, void *x,
                            const int *pos, int n_tokens, void *stream);
/* How rows travel between ranks: 0 = NCCL send / recv (dispatch, owner experts,
 * return, combine as separate steps, one host synchronisation per layer for the
 * row counts), 1 = peer memory (each owner's gather kernel reads the rows it
 * needs out of the home ranks' HBM over NVLink and each home's combine kernel
 * reads the owners' per-row sums the same way; routing results are written into
 * the peers' memory and the two rendezvous of a layer are flags in peer memory
 * with bounded polls - no NCCL call and no host synchronisation in the layer; a
 * flag that does not arrive within "wait_limit_ms" (2 s) leaves status 106 in
 * gptoss_moe_device_status; the reference's counterpart is the peer copies of
 * expert.cpp:1520-1535 and :1577).  gptoss_moe_ep_init selects 1 when every rank could map
 * every peer's buffers through CUDA IPC (one process per rank, one node), else 0;
 * gptoss_moe_set_option(h, "ep_transport", v) changes it (all ranks alike).
 * Both give the same bits.  Returns -1 before gptoss_moe_ep_init. */
int gptoss_moe_ep_transport(const gptoss_moe_t *h);

/*
 * The permutation stage for callers that cannot allocate device memory.  (No
 * counterpart in the reference: its count / scan / build kernels work on buffers
 * the engine allocated at start-up.)
 *
 * Who needs it: a host engine that has already given every free byte of HBM to
 * its own pool (the reference grows its KV cache until allocation fails), or a
 * serving loop that cannot afford the device-wide synchronisation a cudaMalloc
 * or cudaFree implies.  This call takes no engine handle and allocates nothing,
 * neither with cudaMalloc nor through any library: its scratch (per-block expert
 * histograms and the tile schedule) is a fixed 78 KB array inside the library
 * image, present on every GPU that loads the library until the process exits.
 *
 * Same result as gptoss_moe_permute without the row gather: for n_rows rows with
 * top_k slots each (slot_expert: expert id or -1 to skip the slot; ids >=
 * n_experts are skipped too, silently: this call has no status word to report
 * them in), a stable counting sort by expert.  All pointers
 * are device pointers owned by the caller:
 *   expert_offsets [n_experts+1], sorted_row / sorted_weight [n_rows*top_k]
 *   (first expert_offsets[n_experts] entries valid), row_of [n_rows*top_k]
 *   (position of each slot in sorted order, -1 for skipped slots).
 * Limits: n_rows <= 8192, n_experts <= 256, top_k <= 8; anything larger is
 * rejected with GPTOSS_E_CAPACITY (text via gptoss_moe_last_error(NULL)).
 *
 * The first call on each device looks up the array's device address (several host
 * threads may make it at once); make that first call before starting any stream
 * capture.  All calls on one GPU share
 * the one array, which keeps the previous call's contents (the call clears the
 * words that must start at zero): two calls whose kernels overlap on the GPU,
 * from different streams or threads, race - serialise them.
 */
int gptoss_moe_permute_static(const int *slot_expert, const float *slot_weight, int n_rows,
                              int top_k, int n_experts, int *expert_offsets, int *sorted_row,
                              float *sorted_weight, int *row_of, void *stream);

/* Library / build information. */
const char *gptoss_moe_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GPTOSS_MOE_B200_H */
