// extern "C" layer of the MoE engine: handle life cycle, weight residency, the
// per-layer forward and its stages, debug taps.  See include/gptoss_moe_b200.h
// for the contract of every entry point.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

#include "common.cuh"
#include "engine.h"
#include "ep.h"

using namespace gptoss;

static thread_local std::string g_create_err;

static int fail(const gptoss_moe *h, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (h)
    h->err = buf;
  else
    g_create_err = buf;
  return code;
}

namespace gptoss {
int set_global_error(int code, const char *text) {
  g_create_err = text ? text : "";
  return code;
}
}  // namespace gptoss

#define CK(h, call)                                                                      \
  do {                                                                                    \
    cudaError_t e__ = (call);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return fail((h), GPTOSS_E_CUDA, "%s failed: %s (%s:%d)", #call,                     \
                  cudaGetErrorString(e__), __FILE__, __LINE__);                           \
  } while (0)

template <typename T>
static cudaError_t dev_alloc(T **p, size_t n) {
  return cudaMalloc(reinterpret_cast<void **>(p), std::max<size_t>(n, 1) * sizeof(T));
}

extern "C" {

const char *gptoss_moe_version(void) { return "gptoss-moe-b200 0.1 (sm_100a)"; }

const char *gptoss_moe_last_error(const gptoss_moe_t *h) {
  return h ? h->err.c_str() : g_create_err.c_str();
}

int gptoss_moe_create(const gptoss_moe_config_t *cfg, gptoss_moe_t **out) {
  if (!cfg || !out) return fail(nullptr, GPTOSS_E_INVALID, "null argument");
  *out = nullptr;
  const int H = cfg->hidden_dim, IM = cfg->intermediate_dim, E = cfg->n_experts;
  const int K = cfg->experts_per_token;
  if (H <= 0 || IM <= 0 || E <= 0 || K <= 0 || cfg->n_layers <= 0 || cfg->max_tokens <= 0)
    return fail(nullptr, GPTOSS_E_INVALID, "non-positive dimension");
  if (H % 8 || IM % 8)
    return fail(nullptr, GPTOSS_E_INVALID,
                "hidden_dim and intermediate_dim must be multiples of 8 (16-byte rows)");
  if (K > GPTOSS_MAX_TOPK || K > E)
    return fail(nullptr, GPTOSS_E_INVALID, "experts_per_token must be <= %d and <= n_experts",
                GPTOSS_MAX_TOPK);
  if (E > 256) return fail(nullptr, GPTOSS_E_INVALID, "n_experts > 256 not supported");
  const int ep_size = cfg->ep_size > 1 ? cfg->ep_size : 1;
  const int ep_rank = ep_size > 1 ? cfg->ep_rank : 0;
  if (ep_rank < 0 || ep_rank >= ep_size || E % ep_size)
    return fail(nullptr, GPTOSS_E_INVALID, "ep_rank/ep_size do not partition n_experts");
  if (cfg->weight_format != GPTOSS_WEIGHTS_BF16 && cfg->weight_format != GPTOSS_WEIGHTS_MXFP4)
    return fail(nullptr, GPTOSS_E_INVALID, "unknown weight_format");
  if (cfg->weight_format == GPTOSS_WEIGHTS_MXFP4 && (H % 32 || IM % 32))
    return fail(nullptr, GPTOSS_E_INVALID, "MXFP4 needs dimensions that are multiples of 32");

  int ndev = 0;
  cudaError_t ce = cudaGetDeviceCount(&ndev);
  if (ce != cudaSuccess || ndev <= 0)
    return fail(nullptr, GPTOSS_E_CUDA, "no CUDA device: %s", cudaGetErrorString(ce));
  if (cfg->device < 0 || cfg->device >= ndev)
    return fail(nullptr, GPTOSS_E_INVALID, "device %d out of range (%d devices)", cfg->device,
                ndev);
  CK(nullptr, cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  CK(nullptr, cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10)
    return fail(nullptr, GPTOSS_E_CUDA,
                "device %d is sm_%d%d; this library holds sm_100a code only", cfg->device,
                prop.major, prop.minor);

  gptoss_moe *h = new gptoss_moe();
  h->cfg = *cfg;
  h->H = H; h->IM = IM; h->E = E; h->K = K; h->L = cfg->n_layers;
  h->ep_rank = ep_rank; h->ep_size = ep_size;
  h->El = E / ep_size;
  h->max_tokens = cfg->max_tokens;
  h->rows_cap = cfg->max_tokens * ep_size;
  h->assign_cap = h->rows_cap * K;
  h->mtiles_cap = h->assign_cap / 64 + h->El + 1;  // the narrowest row tile is 64
  h->perm_blocks_cap = (h->rows_cap + kPermTokens - 1) / kPermTokens;
  h->num_sms = prop.multiProcessorCount;
  h->layers.resize(h->L);

  const size_t T = h->max_tokens;
#define CKH(call)                                                                         \
  do {                                                                                    \
    cudaError_t e__ = (call);                                                             \
    if (e__ != cudaSuccess) {                                                             \
      int rc__ = fail(nullptr, GPTOSS_E_CUDA, "%s failed: %s", #call,                     \
                      cudaGetErrorString(e__));                                           \
      gptoss_moe_destroy(h);                                                              \
      return rc__;                                                                        \
    }                                                                                     \
  } while (0)
  CKH(dev_alloc(&h->topk_i, T * K));
  CKH(dev_alloc(&h->topk_v, T * K));
  CKH(dev_alloc(&h->block_counts, (size_t)h->perm_blocks_cap * h->El));
  CKH(dev_alloc(&h->expert_offsets, (size_t)h->El + 1));
  CKH(dev_alloc(&h->sorted_row, (size_t)h->assign_cap));
  CKH(dev_alloc(&h->sorted_weight, (size_t)h->assign_cap));
  CKH(dev_alloc(&h->row_of, (size_t)h->rows_cap * K));
  CKH(dev_alloc(&h->mtile_expert, (size_t)h->mtiles_cap));
  CKH(dev_alloc(&h->mtile_row0, (size_t)h->mtiles_cap));
  CKH(dev_alloc(&h->mtile_rows, (size_t)h->mtiles_cap));
  CKH(dev_alloc(&h->num_mtiles, 1));
  CKH(dev_alloc(&h->mtile_split, 1));
  CKH(dev_alloc(&h->status, 1));
  CKH(dev_alloc(&h->xs, (size_t)h->assign_cap * H));
  CKH(dev_alloc(&h->hact, (size_t)h->assign_cap * IM));
  CKH(dev_alloc(&h->ys, (size_t)h->assign_cap * H));
  CKH(cudaMemset(h->xs, 0, (size_t)h->assign_cap * H * sizeof(bf16)));
  CKH(cudaMemset(h->hact, 0, (size_t)h->assign_cap * IM * sizeof(bf16)));
  CKH(cudaMemset(h->status, 0, sizeof(int)));
  CKH(cudaMemset(h->num_mtiles, 0, sizeof(int)));
  CKH(cudaMemset(h->mtile_split, 0, sizeof(int)));
  CKH(cudaMemset(h->expert_offsets, 0, sizeof(int) * (h->El + 1)));
#undef CKH
  std::string terr;
  if (make_tmap_2d_bf16(&h->tmap_xs, h->xs, H, h->assign_cap, kTileK, kTileM, &terr) ||
      make_tmap_2d_bf16(&h->tmap_h, h->hact, IM, h->assign_cap, kTileK, kTileM, &terr) ||
      make_tmap_2d_bf16(&h->tmap_xs32, h->xs, H, h->assign_cap, kTileK, 32, &terr) ||
      make_tmap_2d_bf16(&h->tmap_h32, h->hact, IM, h->assign_cap, kTileK, 32, &terr) ||
      make_tmap_2d_bf16(&h->tmap_xs8, h->xs, H, h->assign_cap, kTileK, 8, &terr) ||
      make_tmap_2d_bf16(&h->tmap_h8, h->hact, IM, h->assign_cap, kTileK, 8, &terr)) {
    int rc = fail(nullptr, GPTOSS_E_CUDA, "%s", terr.c_str());
    gptoss_moe_destroy(h);
    return rc;
  }
  *out = h;
  return GPTOSS_OK;
}

int gptoss_moe_destroy(gptoss_moe_t *h) {
  if (!h) return GPTOSS_OK;
  cudaSetDevice(h->cfg.device);
  cudaDeviceSynchronize();
  ep_destroy(h);
  for (auto &lw : h->layers) {
    cudaFree(lw.w_router); cudaFree(lw.b_router); cudaFree(lw.w1); cudaFree(lw.b1);
    cudaFree(lw.w2); cudaFree(lw.b2); cudaFree(lw.w1_blocks); cudaFree(lw.w2_blocks);
    cudaFree(lw.router_tiled);
    cudaFree(lw.rms_ffn);
  }
  cudaFree(h->topk_i); cudaFree(h->topk_v); cudaFree(h->logits); cudaFree(h->block_counts);
  cudaFree(h->expert_offsets); cudaFree(h->sorted_row); cudaFree(h->sorted_weight);
  cudaFree(h->row_of); cudaFree(h->mtile_expert); cudaFree(h->mtile_row0);
  cudaFree(h->mtile_rows); cudaFree(h->num_mtiles); cudaFree(h->mtile_split); cudaFree(h->status); cudaFree(h->xs);
  cudaFree(h->hact); cudaFree(h->ys); cudaFree(h->row_dst); cudaFree(h->t_dev); cudaFree(h->x_dev);
  cudaFree(h->pos_dev);
  for (auto &sl : h->host_slots) {
    if (sl.busy) cudaEventSynchronize(sl.d2h);
    cudaFree(sl.t); cudaFree(sl.x); cudaFree(sl.pos);
    if (sl.h2d) cudaEventDestroy(sl.h2d);
    if (sl.done) cudaEventDestroy(sl.done);
    if (sl.d2h) cudaEventDestroy(sl.d2h);
  }
  if (h->s_h2d) cudaStreamDestroy(h->s_h2d);
  if (h->s_comp) cudaStreamDestroy(h->s_comp);
  if (h->s_d2h) cudaStreamDestroy(h->s_d2h);
  gptoss_moe_release_upload_staging(h);
  for (auto &t : h->timers) {
    for (auto e : t.beg) cudaEventDestroy(e);
    for (auto e : t.end) cudaEventDestroy(e);
  }
  delete h;
  return GPTOSS_OK;
}

// Reads the device status word after the caller has synchronised the stream the kernels ran
// on; a non-zero word is cleared and reported as GPTOSS_E_DEVICE.
int gptoss_moe_take_status(gptoss_moe *h) {
  int s = 0;
  CK(h, cudaMemcpy(&s, h->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (!s) return GPTOSS_OK;
  CK(h, cudaMemset(h->status, 0, sizeof(int)));
  return fail(h, GPTOSS_E_DEVICE,
              "a kernel reported status %d (101-103: a pipeline wait ran out, 104: index out of "
              "range, 105: tensor memory, 106: another rank's flag did not arrive in time)", s);
}

// ------------------------------------------------------------------ weights
static int alloc_layer(gptoss_moe *h, LayerWeights &lw) {
  const size_t H = h->H, IM = h->IM, E = h->E, El = h->El;
  if (!lw.w_router) CK(h, dev_alloc(&lw.w_router, E * H));
  if (!lw.b_router) CK(h, dev_alloc(&lw.b_router, E));
  if (!lw.w1) CK(h, dev_alloc(&lw.w1, El * 2 * IM * H));
  if (!lw.b1) CK(h, dev_alloc(&lw.b1, El * 2 * IM));
  if (!lw.w2) CK(h, dev_alloc(&lw.w2, El * H * IM));
  if (!lw.b2) CK(h, dev_alloc(&lw.b2, El * H));
  return GPTOSS_OK;
}

static int finish_layer(gptoss_moe *h, LayerWeights &lw) {
  std::string terr;
  const int bn = gemm_tile_n(0);
  if (make_tmap_2d_bf16(&lw.tmap_w1, lw.w1, h->H, (uint64_t)h->El * 2 * h->IM, kTileK, bn,
                        &terr) ||
      make_tmap_2d_bf16(&lw.tmap_w2, lw.w2, h->IM, (uint64_t)h->El * h->H, kTileK, bn, &terr) ||
      make_tmap_2d_bf16(&lw.tmap_w1_rows, lw.w1, h->H, (uint64_t)h->El * 2 * h->IM, kTileK, 128,
                        &terr) ||
      make_tmap_2d_bf16(&lw.tmap_w2_rows, lw.w2, h->IM, (uint64_t)h->El * h->H, kTileK, 128,
                        &terr))
    return fail(h, GPTOSS_E_CUDA, "%s", terr.c_str());
  if (int rc = build_router_tiles(h, lw)) return rc;
  lw.loaded = true;
  return GPTOSS_OK;
}

// fp32 host -> bf16 device through a pinned double buffer (not part of the public
// header; the decode engine's loader uses it too).  The stream, the two pinned and the
// two device staging buffers and their events belong to the engine: made on the first
// upload, reused by every later one, released by gptoss_moe_release_upload_staging (the
// loaders call it when a model is in place) or with the engine.
static int upload_staging(gptoss_moe *h) {
  if (h->up_stream) return GPTOSS_OK;
  CK(h, cudaStreamCreateWithFlags(&h->up_stream, cudaStreamNonBlocking));
  for (int i = 0; i < 2; i++) {
    CK(h, cudaMallocHost(reinterpret_cast<void **>(&h->up_pinned[i]), gptoss_moe::kUploadChunk * 4));
    CK(h, dev_alloc(&h->up_dev[i], gptoss_moe::kUploadChunk));
    CK(h, cudaEventCreateWithFlags(&h->up_done[i], cudaEventDisableTiming));
  }
  return GPTOSS_OK;
}

void gptoss_moe_release_upload_staging(gptoss_moe *h) {
  if (!h) return;
  if (h->up_stream) cudaStreamSynchronize(h->up_stream);
  for (int i = 0; i < 2; i++) {
    if (h->up_pinned[i]) cudaFreeHost(h->up_pinned[i]);
    if (h->up_dev[i]) cudaFree(h->up_dev[i]);
    if (h->up_done[i]) cudaEventDestroy(h->up_done[i]);
    h->up_pinned[i] = nullptr;
    h->up_dev[i] = nullptr;
    h->up_done[i] = nullptr;
  }
  if (h->up_stream) cudaStreamDestroy(h->up_stream);
  h->up_stream = nullptr;
  h->up_next = 0;
}

int upload_f32_as_bf16(gptoss_moe *h, bf16 *dst, const float *src, size_t n) {
  int rc = upload_staging(h);
  if (rc) {
    gptoss_moe_release_upload_staging(h);
    return rc;
  }
  const size_t chunk = gptoss_moe::kUploadChunk;
  for (size_t off = 0; off < n; off += chunk) {
    const int b = h->up_next;
    h->up_next ^= 1;
    const size_t m = std::min(chunk, n - off);
    CK(h, cudaEventSynchronize(h->up_done[b]));  // buffer free again (no-op the first time)
    memcpy(h->up_pinned[b], src + off, m * 4);
    CK(h, cudaMemcpyAsync(h->up_dev[b], h->up_pinned[b], m * 4, cudaMemcpyHostToDevice, h->up_stream));
    CK(h, launch_f32_to_bf16(dst + off, h->up_dev[b], m, h->up_stream, &h->launches));
    CK(h, cudaEventRecord(h->up_done[b], h->up_stream));
  }
  return GPTOSS_OK;
}

// Everything queued by upload_f32_as_bf16 has landed.
int upload_finish(gptoss_moe *h) {
  if (h->up_stream) CK(h, cudaStreamSynchronize(h->up_stream));
  return GPTOSS_OK;
}

int gptoss_moe_load_layer_f32(gptoss_moe_t *h, int layer, const float *w_router,
                              const float *b_router, const float *w_mlp1, const float *b_mlp1,
                              const float *w_mlp2, const float *b_mlp2) {
  if (!h) return GPTOSS_E_INVALID;
  if (layer < 0 || layer >= h->L) return fail(h, GPTOSS_E_INVALID, "layer out of range");
  if (!w_router || !b_router || !w_mlp1 || !b_mlp1 || !w_mlp2 || !b_mlp2)
    return fail(h, GPTOSS_E_INVALID, "null weight pointer");
  if (h->cfg.weight_format != GPTOSS_WEIGHTS_BF16)
    return fail(h, GPTOSS_E_STATE, "engine was created for another weight format");
  CK(h, cudaSetDevice(h->cfg.device));
  LayerWeights &lw = h->layers[layer];
  int rc = alloc_layer(h, lw);
  if (rc) return rc;
  const size_t H = h->H, IM = h->IM, E = h->E;
  if ((rc = upload_f32_as_bf16(h, lw.w_router, w_router, E * H))) return rc;
  CK(h, cudaMemcpy(lw.b_router, b_router, E * 4, cudaMemcpyHostToDevice));
  for (int j = 0; j < h->El; j++) {
    const size_t e = (size_t)j * h->ep_size + h->ep_rank;  // global expert of local id j
    if ((rc = upload_f32_as_bf16(h, lw.w1 + j * 2 * IM * H, w_mlp1 + e * 2 * IM * H, 2 * IM * H)))
      return rc;
    if ((rc = upload_f32_as_bf16(h, lw.w2 + j * H * IM, w_mlp2 + e * H * IM, H * IM))) return rc;
    CK(h, cudaMemcpy(lw.b1 + j * 2 * IM, b_mlp1 + e * 2 * IM, 2 * IM * 4, cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(lw.b2 + j * H, b_mlp2 + e * H, H * 4, cudaMemcpyHostToDevice));
  }
  if ((rc = upload_finish(h))) return rc;
  return finish_layer(h, lw);
}

int gptoss_moe_load_layer_bf16(gptoss_moe_t *h, int layer, const void *w_router,
                               const float *b_router, const void *w_mlp1, const float *b_mlp1,
                               const void *w_mlp2, const float *b_mlp2, int on_device) {
  if (!h) return GPTOSS_E_INVALID;
  if (layer < 0 || layer >= h->L) return fail(h, GPTOSS_E_INVALID, "layer out of range");
  if (!w_router || !b_router || !w_mlp1 || !b_mlp1 || !w_mlp2 || !b_mlp2)
    return fail(h, GPTOSS_E_INVALID, "null weight pointer");
  if (h->cfg.weight_format != GPTOSS_WEIGHTS_BF16)
    return fail(h, GPTOSS_E_STATE, "engine was created for another weight format");
  CK(h, cudaSetDevice(h->cfg.device));
  LayerWeights &lw = h->layers[layer];
  int rc = alloc_layer(h, lw);
  if (rc) return rc;
  const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  const size_t H = h->H, IM = h->IM, E = h->E;
  const bf16 *w1 = static_cast<const bf16 *>(w_mlp1), *w2 = static_cast<const bf16 *>(w_mlp2);
  CK(h, cudaMemcpy(lw.w_router, w_router, E * H * 2, kind));
  CK(h, cudaMemcpy(lw.b_router, b_router, E * 4, kind));
  for (int j = 0; j < h->El; j++) {
    const size_t e = (size_t)j * h->ep_size + h->ep_rank;
    CK(h, cudaMemcpy(lw.w1 + j * 2 * IM * H, w1 + e * 2 * IM * H, 2 * IM * H * 2, kind));
    CK(h, cudaMemcpy(lw.w2 + j * H * IM, w2 + e * H * IM, H * IM * 2, kind));
    CK(h, cudaMemcpy(lw.b1 + j * 2 * IM, b_mlp1 + e * 2 * IM, 2 * IM * 4, kind));
    CK(h, cudaMemcpy(lw.b2 + j * H, b_mlp2 + e * H, H * 4, kind));
  }
  return finish_layer(h, lw);
}

// gptoss_moe_load_layer_mxfp4 lives in mxfp4.cu

// ------------------------------------------------------------------ stages
static int check_layer(gptoss_moe *h, int layer, int n_tokens) {
  if (layer < 0 || layer >= h->L) return fail(h, GPTOSS_E_INVALID, "layer out of range");
  if (!h->layers[layer].loaded)
    return fail(h, GPTOSS_E_STATE, "weights of layer %d not loaded", layer);
  if (n_tokens < 0) return fail(h, GPTOSS_E_INVALID, "negative n_tokens");
  if (n_tokens > h->max_tokens)
    return fail(h, GPTOSS_E_CAPACITY, "n_tokens %d exceeds max_tokens %d", n_tokens,
                h->max_tokens);
  return GPTOSS_OK;
}

struct StageScope {
  gptoss_moe *h;
  int id;
  cudaStream_t st;
  StageScope(gptoss_moe *h_, int id_, cudaStream_t st_) : h(h_), id(id_), st(st_) {
    if (!h->opt_time_stages) return;
    StageTimer &t = h->timers[id];
    if (t.used == t.beg.size()) {
      cudaEvent_t b, e;
      cudaEventCreate(&b);
      cudaEventCreate(&e);
      t.beg.push_back(b);
      t.end.push_back(e);
    }
    cudaEventRecord(t.beg[t.used], st);
  }
  ~StageScope() {
    if (!h->opt_time_stages) return;
    StageTimer &t = h->timers[id];
    cudaEventRecord(t.end[t.used], st);
    t.used++;
  }
};

int gptoss_moe_route(gptoss_moe_t *h, int layer, const void *t, const int *pos, int n_tokens,
                     void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  if (!t && n_tokens > 0) return fail(h, GPTOSS_E_INVALID, "null input");
  int rc = check_layer(h, layer, n_tokens);
  if (rc) return rc;
  CK(h, cudaSetDevice(h->cfg.device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (h->opt_keep_logits && !h->logits)
    CK(h, dev_alloc(&h->logits, (size_t)h->max_tokens * h->E));
  StageScope sc(h, 0, st);
  CK(h, launch_router_topk(h, layer, static_cast<const bf16 *>(t), pos, n_tokens,
                           h->opt_keep_logits ? h->logits : nullptr, st));
  return GPTOSS_OK;
}

int gptoss_moe_permute(gptoss_moe_t *h, const void *t, int n_tokens, void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  if (!t && n_tokens > 0) return fail(h, GPTOSS_E_INVALID, "null input");
  if (n_tokens < 0 || n_tokens > h->max_tokens)
    return fail(h, GPTOSS_E_CAPACITY, "n_tokens out of range");
  if (h->ep_size > 1)
    return fail(h, GPTOSS_E_STATE, "stage calls are single-GPU; use gptoss_moe_forward");
  CK(h, cudaSetDevice(h->cfg.device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  h->stage_rows = static_cast<const bf16 *>(t);
  h->stage_expert = h->topk_i;
  h->stage_weight = h->topk_v;
  h->stage_R = n_tokens;
  StageScope sc(h, 1, st);
  CK(h, launch_permute(h, st));
  return GPTOSS_OK;
}

int gptoss_moe_experts(gptoss_moe_t *h, int layer, void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  int rc = check_layer(h, layer, 0);
  if (rc) return rc;
  CK(h, cudaSetDevice(h->cfg.device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    StageScope sc(h, 2, st);
    CK(h, launch_gate_up(h, layer, st));
  }
  {
    StageScope sc(h, 3, st);
    CK(h, launch_down(h, layer, st));
  }
  return GPTOSS_OK;
}

int gptoss_moe_combine(gptoss_moe_t *h, void *x, int n_tokens, void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  if (!x && n_tokens > 0) return fail(h, GPTOSS_E_INVALID, "null output");
  if (n_tokens < 0 || n_tokens > h->max_tokens)
    return fail(h, GPTOSS_E_CAPACITY, "n_tokens out of range");
  if (h->ep_size > 1)
    return fail(h, GPTOSS_E_STATE, "stage calls are single-GPU; use gptoss_moe_forward");
  CK(h, cudaSetDevice(h->cfg.device));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  StageScope sc(h, 4, st);
  CK(h, launch_combine(h, static_cast<bf16 *>(x), h->topk_i, n_tokens, st));
  return GPTOSS_OK;
}

int gptoss_moe_forward(gptoss_moe_t *h, int layer, const void *t, void *x, const int *pos,
                       int n_tokens, void *stream) {
  if (!h) return GPTOSS_E_INVALID;
  if ((!t || !x) && n_tokens > 0) return fail(h, GPTOSS_E_INVALID, "null activation pointer");
  int rc = check_layer(h, layer, n_tokens);
  if (rc) return rc;
  if (n_tokens == 0 && h->ep_size <= 1) return GPTOSS_OK;
  if ((rc = gptoss_moe_route(h, layer, t, pos, n_tokens, stream))) return rc;
  if (h->ep_size > 1) return ep_forward(h, layer, t, x, n_tokens, stream);
  if ((rc = gptoss_moe_permute(h, t, n_tokens, stream))) return rc;
  if ((rc = gptoss_moe_experts(h, layer, stream))) return rc;
  return gptoss_moe_combine(h, x, n_tokens, stream);
}

// Submissions still in flight use the engine's workspaces: let them finish first.
static int drain_host_slots(gptoss_moe *h) {
  for (auto &sl : h->host_slots) {
    if (sl.busy) {
      CK(h, cudaEventSynchronize(sl.d2h));
      sl.busy = false;
    }
  }
  return GPTOSS_OK;
}

int gptoss_moe_forward_host(gptoss_moe_t *h, int layer, const void *t_host, void *x_host,
                            const int *pos_host, int n_tokens) {
  if (!h) return GPTOSS_E_INVALID;
  if (int drc = drain_host_slots(h)) return drc;
  if ((!t_host || !x_host) && n_tokens > 0)
    return fail(h, GPTOSS_E_INVALID, "null activation pointer");
  int rc = check_layer(h, layer, n_tokens);
  if (rc) return rc;
  if (n_tokens == 0 && h->ep_size <= 1) return GPTOSS_OK;
  if (rc) return rc;
  CK(h, cudaSetDevice(h->cfg.device));
  const size_t cap = (size_t)h->max_tokens * h->H;
  if (!h->t_dev) CK(h, dev_alloc(&h->t_dev, cap));
  if (!h->x_dev) CK(h, dev_alloc(&h->x_dev, cap));
  if (!h->pos_dev) CK(h, dev_alloc(&h->pos_dev, (size_t)h->max_tokens));
  const size_t bytes = (size_t)n_tokens * h->H * sizeof(bf16);
  cudaStream_t st = nullptr;
  CK(h, cudaMemcpyAsync(h->t_dev, t_host, bytes, cudaMemcpyHostToDevice, st));
  CK(h, cudaMemcpyAsync(h->x_dev, x_host, bytes, cudaMemcpyHostToDevice, st));
  if (pos_host)
    CK(h, cudaMemcpyAsync(h->pos_dev, pos_host, (size_t)n_tokens * 4, cudaMemcpyHostToDevice, st));
  rc = gptoss_moe_forward(h, layer, h->t_dev, h->x_dev, pos_host ? h->pos_dev : nullptr,
                          n_tokens, st);
  if (rc) return rc;
  CK(h, cudaMemcpyAsync(x_host, h->x_dev, bytes, cudaMemcpyDeviceToHost, st));
  CK(h, cudaStreamSynchronize(st));
  return gptoss_moe_take_status(h);
}

int gptoss_moe_load_ffn_norm(gptoss_moe_t *h, int layer, const float *scale_host) {
  if (!h || !scale_host) return GPTOSS_E_INVALID;
  if (layer < 0 || layer >= h->L) return fail(h, GPTOSS_E_INVALID, "layer out of range");
  CK(h, cudaSetDevice(h->cfg.device));
  LayerWeights &lw = h->layers[layer];
  if (!lw.rms_ffn) CK(h, dev_alloc(&lw.rms_ffn, (size_t)h->H));
  CK(h, cudaMemcpy(lw.rms_ffn, scale_host, sizeof(float) * h->H, cudaMemcpyHostToDevice));
  return GPTOSS_OK;
}

int gptoss_moe_forward_host_submit(gptoss_moe_t *h, int layer, const void *t_host, void *x_host,
                                   const int *pos_host, int n_tokens, int *ticket) {
  if (!h || !ticket) return GPTOSS_E_INVALID;
  if (!x_host && n_tokens > 0) return fail(h, GPTOSS_E_INVALID, "null activation pointer");
  int rc = check_layer(h, layer, n_tokens);
  if (rc) return rc;
  if (!t_host && !h->layers[layer].rms_ffn)
    return fail(h, GPTOSS_E_STATE,
                "t_host is NULL but the layer has no RMSNorm scale (gptoss_moe_load_ffn_norm)");
  if (h->ep_size > 1 && ep_get_transport(h) != 1)
    return fail(h, GPTOSS_E_STATE,
                "under expert parallelism the pipelined host path needs the peer-memory transport "
                "(the NCCL transport synchronises with the host inside every layer)");
  CK(h, cudaSetDevice(h->cfg.device));
  if (!h->s_comp) {
    CK(h, cudaStreamCreateWithFlags(&h->s_h2d, cudaStreamNonBlocking));
    CK(h, cudaStreamCreateWithFlags(&h->s_comp, cudaStreamNonBlocking));
    CK(h, cudaStreamCreateWithFlags(&h->s_d2h, cudaStreamNonBlocking));
  }
  const int si = static_cast<int>(h->host_submitted % gptoss_moe::kHostSlots);
  gptoss_moe::HostSlot &sl = h->host_slots[si];
  if (!sl.t) {
    const size_t cap = (size_t)h->max_tokens * h->H;
    CK(h, dev_alloc(&sl.t, cap));
    CK(h, dev_alloc(&sl.x, cap));
    CK(h, dev_alloc(&sl.pos, (size_t)h->max_tokens));
    CK(h, cudaEventCreateWithFlags(&sl.h2d, cudaEventDisableTiming));
    CK(h, cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming));
    CK(h, cudaEventCreateWithFlags(&sl.d2h, cudaEventDisableTiming));
  }
  if (sl.busy) {  // the submission that used this slot three calls ago
    CK(h, cudaEventSynchronize(sl.d2h));
    sl.busy = false;
  }
  const size_t bytes = (size_t)n_tokens * h->H * sizeof(bf16);
  if (n_tokens > 0) {
    if (t_host) CK(h, cudaMemcpyAsync(sl.t, t_host, bytes, cudaMemcpyHostToDevice, h->s_h2d));
    CK(h, cudaMemcpyAsync(sl.x, x_host, bytes, cudaMemcpyHostToDevice, h->s_h2d));
    if (pos_host)
      CK(h, cudaMemcpyAsync(sl.pos, pos_host, (size_t)n_tokens * 4, cudaMemcpyHostToDevice, h->s_h2d));
  }
  CK(h, cudaEventRecord(sl.h2d, h->s_h2d));
  CK(h, cudaStreamWaitEvent(h->s_comp, sl.h2d, 0));
  if (n_tokens > 0) {
    if (!t_host)  // the block's own RMSNorm: t = scale * x / rms(x)
      CK(h, launch_rmsnorm(sl.t, sl.x, h->layers[layer].rms_ffn, pos_host ? sl.pos : nullptr,
                           n_tokens, h->H, h->s_comp, &h->launches));
    rc = gptoss_moe_forward(h, layer, sl.t, sl.x, pos_host ? sl.pos : nullptr, n_tokens, h->s_comp);
    if (rc) return rc;
  }
  CK(h, cudaEventRecord(sl.done, h->s_comp));
  CK(h, cudaStreamWaitEvent(h->s_d2h, sl.done, 0));
  if (n_tokens > 0)
    CK(h, cudaMemcpyAsync(x_host, sl.x, bytes, cudaMemcpyDeviceToHost, h->s_d2h));
  CK(h, cudaEventRecord(sl.d2h, h->s_d2h));
  sl.busy = true;
  *ticket = static_cast<int>(h->host_submitted & 0x7fffffff);
  h->host_submitted++;
  return GPTOSS_OK;
}

int gptoss_moe_forward_host_wait(gptoss_moe_t *h, int ticket) {
  if (!h) return GPTOSS_E_INVALID;
  const long long newest = h->host_submitted - 1;
  const long long t = (newest & ~0x7fffffffll) | ticket;
  if (ticket < 0 || t > newest) return fail(h, GPTOSS_E_INVALID, "unknown ticket");
  if (newest - t >= gptoss_moe::kHostSlots) return GPTOSS_OK;  // its slot was reused: long done
  gptoss_moe::HostSlot &sl = h->host_slots[t % gptoss_moe::kHostSlots];
  if (sl.busy) {
    CK(h, cudaSetDevice(h->cfg.device));
    CK(h, cudaEventSynchronize(sl.d2h));
    sl.busy = false;
    // the status word is the engine's, not the ticket's: a problem in a later submission
    // that has already run shows up here too
    return gptoss_moe_take_status(h);
  }
  return GPTOSS_OK;
}

int gptoss_moe_rmsnorm(gptoss_moe_t *h, void *out, const void *x, const float *w_dev,
                       const int *pos, int n_tokens, void *stream) {
  if (!h || !out || !x || !w_dev) return GPTOSS_E_INVALID;
  if (n_tokens < 0) return fail(h, GPTOSS_E_INVALID, "negative n_tokens");
  CK(h, cudaSetDevice(h->cfg.device));
  CK(h, launch_rmsnorm(static_cast<bf16 *>(out), static_cast<const bf16 *>(x), w_dev, pos,
                       n_tokens, h->H, static_cast<cudaStream_t>(stream), &h->launches));
  return GPTOSS_OK;
}

// ------------------------------------------------------------------ taps
int gptoss_moe_get_routing(gptoss_moe_t *h, int n_tokens, int *topk_i, float *topk_v,
                           int *expert_offsets, int *sorted_token, float *logits) {
  if (!h) return GPTOSS_E_INVALID;
  if (n_tokens < 0 || n_tokens > h->max_tokens) return fail(h, GPTOSS_E_CAPACITY, "n_tokens");
  CK(h, cudaSetDevice(h->cfg.device));
  CK(h, cudaDeviceSynchronize());
  const size_t nk = (size_t)n_tokens * h->K;
  if (topk_i) CK(h, cudaMemcpy(topk_i, h->topk_i, nk * 4, cudaMemcpyDeviceToHost));
  if (topk_v) CK(h, cudaMemcpy(topk_v, h->topk_v, nk * 4, cudaMemcpyDeviceToHost));
  std::vector<int> off(h->El + 1);
  CK(h, cudaMemcpy(off.data(), h->expert_offsets, off.size() * 4, cudaMemcpyDeviceToHost));
  if (expert_offsets) memcpy(expert_offsets, off.data(), off.size() * 4);
  if (sorted_token && off[h->El] > 0) {
    if (off[h->El] > h->assign_cap) return fail(h, GPTOSS_E_DEVICE, "corrupt offsets");
    CK(h, cudaMemcpy(sorted_token, h->sorted_row, (size_t)off[h->El] * 4,
                     cudaMemcpyDeviceToHost));
  }
  if (logits) {
    if (!h->logits) return fail(h, GPTOSS_E_STATE, "keep_logits was not enabled");
    CK(h, cudaMemcpy(logits, h->logits, (size_t)n_tokens * h->E * 4, cudaMemcpyDeviceToHost));
  }
  return GPTOSS_OK;
}

int gptoss_moe_get_activations(gptoss_moe_t *h, void *act_host, size_t bytes) {
  if (!h || !act_host) return GPTOSS_E_INVALID;
  CK(h, cudaSetDevice(h->cfg.device));
  CK(h, cudaDeviceSynchronize());
  if (bytes > (size_t)h->assign_cap * h->IM * sizeof(bf16))
    return fail(h, GPTOSS_E_CAPACITY, "more bytes than the activation buffer holds");
  CK(h, cudaMemcpy(act_host, h->hact, bytes, cudaMemcpyDeviceToHost));
  return GPTOSS_OK;
}

int gptoss_moe_set_option(gptoss_moe_t *h, const char *name, int value) {
  if (!h || !name) return GPTOSS_E_INVALID;
  if (!strcmp(name, "gemm_impl")) {
    if (value != GPTOSS_GEMM_TCGEN05 && value != GPTOSS_GEMM_SIMT && value != GPTOSS_GEMM_PAIR)
      return fail(h, GPTOSS_E_INVALID, "unknown gemm_impl %d", value);
    if (h->cfg.weight_format == GPTOSS_WEIGHTS_MXFP4 && value != GPTOSS_GEMM_PAIR)
      return fail(h, GPTOSS_E_INVALID, "MXFP4 weights are only read by the CTA-pair kernel");
    h->opt_gemm_impl = value;
  } else if (!strcmp(name, "keep_logits")) {
    h->opt_keep_logits = value != 0;
  } else if (!strcmp(name, "exact_ties")) {
    h->opt_exact_ties = value != 0;
  } else if (!strcmp(name, "router_impl")) {
    if (value != 0 && value != 1) return fail(h, GPTOSS_E_INVALID, "router_impl must be 0 or 1");
    h->opt_router_impl = value;
  } else if (!strcmp(name, "l2_hints")) {
    h->opt_l2_hints = value != 0;
  } else if (!strcmp(name, "mx_tmem")) {
    h->opt_mx_tmem = value != 0;
  } else if (!strcmp(name, "ep_dedup")) {
    h->opt_ep_dedup = value != 0;
  } else if (!strcmp(name, "ep_push")) {
    h->opt_ep_push = value != 0;
  } else if (!strcmp(name, "dependent_launch")) {
    h->opt_dependent_launch = value != 0;
  } else if (!strcmp(name, "wait_limit_ms")) {
    if (value < 1 || value > 60000)
      return fail(h, GPTOSS_E_INVALID, "wait_limit_ms must be 1..60000");
    h->opt_wait_limit_ms = value;
  } else if (!strcmp(name, "ep_overlap")) {
    h->opt_ep_overlap = value != 0;
  } else if (!strcmp(name, "ep_gather_ctas")) {
    if (value < 1 || value > 4096) return fail(h, GPTOSS_E_INVALID, "ep_gather_ctas must be 1..4096");
    h->opt_ep_gather_ctas = value;
  } else if (!strcmp(name, "ep_transport")) {
    return ep_set_transport(h, value);
  } else if (!strcmp(name, "time_stages")) {
    // value 1 starts a fresh series of measurements (event pairs are reused)
    h->opt_time_stages = value != 0;
    if (value) for (auto &t : h->timers) t.used = 0;
  } else {
    return fail(h, GPTOSS_E_INVALID, "unknown option '%s'", name);
  }
  return GPTOSS_OK;
}

long long gptoss_moe_launch_count(const gptoss_moe_t *h) { return h ? h->launches : 0; }

int gptoss_moe_device_status(gptoss_moe_t *h) {
  if (!h) return GPTOSS_E_INVALID;
  CK(h, cudaSetDevice(h->cfg.device));
  CK(h, cudaDeviceSynchronize());
  int s = 0;
  CK(h, cudaMemcpy(&s, h->status, 4, cudaMemcpyDeviceToHost));
  if (s) CK(h, cudaMemset(h->status, 0, 4));
  return s;
}

int gptoss_moe_stage_ms(gptoss_moe_t *h, int stage, float *ms) {
  if (!h || !ms || stage < 0 || stage >= 8) return GPTOSS_E_INVALID;
  StageTimer &t = h->timers[stage];
  if (!t.used) return fail(h, GPTOSS_E_STATE, "stage %d was not timed", stage);
  CK(h, cudaEventSynchronize(t.end[t.used - 1]));
  double sum = 0.0;
  for (size_t i = 0; i < t.used; i++) {
    float one = 0.f;
    CK(h, cudaEventElapsedTime(&one, t.beg[i], t.end[i]));
    sum += one;
  }
  *ms = static_cast<float>(sum / static_cast<double>(t.used));
  return GPTOSS_OK;
}

}  // extern "C"
