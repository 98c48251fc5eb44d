// Internal declarations shared by the translation units of the MoE library:
// the engine object behind the opaque C handle and the kernel launchers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/gptoss_moe_b200.h"

namespace gptoss {

typedef __nv_bfloat16 bf16;

// Rows of one M tile of the grouped GEMMs (UMMA M) and the K extent of one
// pipeline stage (one 128-byte swizzle row of bf16).
constexpr int kTileM = 128;
constexpr int kTileK = 64;
// Tokens handled by one CTA of the permutation kernels.
constexpr int kPermTokens = 128;

struct LayerWeights {
  bf16 *w_router = nullptr;   // [E, H]
  float *b_router = nullptr;  // [E]
  bf16 *w1 = nullptr;         // [E_local, 2*IM, H]
  float *b1 = nullptr;        // [E_local, 2*IM]
  bf16 *w2 = nullptr;         // [E_local, H, IM]
  float *b2 = nullptr;        // [E_local, H]
  // MXFP4 storage, tiled: [expert][128-row block][64-k block][4096 B codes + 256 B scales]
  uint8_t *w1_blocks = nullptr, *w2_blocks = nullptr;
  CUtensorMap tmap_w1, tmap_w2;            // boxes of 240 weight rows (N operand)
  CUtensorMap tmap_w1_rows, tmap_w2_rows;  // boxes of 128 weight rows (M operand, CTA pairs)
  // router rows tile by tile (128 rows x 64 k, zero padded; weights.cu's layout): the
  // tcgen05 router's M operand, one box per K chunk
  bf16 *router_tiled = nullptr;
  CUtensorMap tmap_router_tiled;
  float *rms_ffn = nullptr;   // [H] scale of the RMSNorm in front of the block (optional)
  bool loaded = false;
};

// CUDA-event pairs recorded around one stage on the launching stream; one pair
// per call while stage timing is on, averaged by gptoss_moe_stage_ms.
struct StageTimer {
  std::vector<cudaEvent_t> beg, end;
  size_t used = 0;
};

}  // namespace gptoss

struct gptoss_moe {
  gptoss_moe_config_t cfg;
  int H, IM, E, K, L, El;  // El = experts owned by this rank
  int ep_rank, ep_size;
  int max_tokens;
  int rows_cap;     // rows that can enter the expert stage (T, or ep_size*T)
  int assign_cap;   // (row, slot) pairs that can enter the expert stage
  int mtiles_cap;   // M tiles of the grouped GEMMs
  int perm_blocks_cap;
  int num_sms;

  std::vector<gptoss::LayerWeights> layers;

  // home-side routing results for the rank's own tokens
  int *topk_i = nullptr;      // [T, K] global expert ids, -1 on inactive rows
  float *topk_v = nullptr;    // [T, K]
  float *logits = nullptr;    // [T, E], only with keep_logits

  // expert-stage inputs (single GPU: t / topk_i / topk_v of the caller's batch;
  // expert parallel: the rows received from all homes)
  const gptoss::bf16 *stage_rows = nullptr;  // [R, H]
  const int *stage_expert = nullptr;         // [R, K] local expert id or -1
  const float *stage_weight = nullptr;       // [R, K]
  int stage_R = 0;
  int cur_tile_rows = 128;  // row tile of the schedule the last permutation built

  // permutation outputs
  int *block_counts = nullptr;   // [perm_blocks_cap, El]
  int *expert_offsets = nullptr; // [El + 1]
  int *sorted_row = nullptr;     // [assign_cap] source row
  float *sorted_weight = nullptr;// [assign_cap]
  int *row_of = nullptr;         // [rows_cap * K] position in sorted order or -1
  int *mtile_expert = nullptr;   // [mtiles_cap]
  int *mtile_row0 = nullptr;     // [mtiles_cap] first sorted row of the tile
  int *mtile_rows = nullptr;     // [mtiles_cap] valid rows in the tile
  int *num_mtiles = nullptr;     // [1]
  int *mtile_split = nullptr;    // [1] first token tile of expert >= the split expert

  gptoss::bf16 *xs = nullptr;    // [assign_cap + pad, H]  gathered inputs
  gptoss::bf16 *hact = nullptr;  // [assign_cap + pad, IM] SwiGLU activations
  gptoss::bf16 *ys = nullptr;    // [assign_cap, H]        weighted expert outputs
  CUtensorMap tmap_xs, tmap_h;            // boxes of 128 rows
  CUtensorMap tmap_xs32, tmap_h32;        // boxes of 32 rows (narrow token tiles)
  CUtensorMap tmap_xs8, tmap_h8;          // boxes of 8 rows

  // host-call staging
  gptoss::bf16 *t_dev = nullptr, *x_dev = nullptr;
  int *pos_dev = nullptr;
  // pipelined host-buffer path: staging slots, one stream per direction and one for the
  // kernels, events that order them
  struct HostSlot {
    gptoss::bf16 *t = nullptr, *x = nullptr;
    int *pos = nullptr;
    cudaEvent_t h2d = nullptr, done = nullptr, d2h = nullptr;
    bool busy = false;
  };
  static constexpr int kHostSlots = 3;
  HostSlot host_slots[kHostSlots];
  cudaStream_t s_h2d = nullptr, s_comp = nullptr, s_d2h = nullptr;
  long long host_submitted = 0;

  // router: tensor map of the caller's activations, kept while the same buffer comes back
  CUtensorMap tmap_router_t;
  const void *router_t_ptr = nullptr;
  int router_t_rows = 0, router_t_box = 0;

  // weight upload: fp32 host tensors through pinned and device staging, converted on the device
  static constexpr size_t kUploadChunk = (size_t)8 << 20;  // elements per chunk (32 MB of fp32)
  cudaStream_t up_stream = nullptr;
  float *up_pinned[2] = {nullptr, nullptr}, *up_dev[2] = {nullptr, nullptr};
  cudaEvent_t up_done[2] = {nullptr, nullptr};
  int up_next = 0;

  int *status = nullptr;  // device status word
  int opt_gemm_impl = GPTOSS_GEMM_PAIR;
  int opt_keep_logits = 0;
  int opt_exact_ties = 1;
  int opt_time_stages = 0;
  int opt_ep_overlap = 0;  // peer transport: second half of the experts gathered under the first half's GEMM
  int opt_ep_gather_ctas = 64;  // CTAs of that overlapped gather
  int opt_router_impl = 0;  // 0 = tcgen05 router, 1 = mma.sync router
  int opt_dependent_launch = 1;  // programmatic dependent launch between the layer's kernels
  int opt_l2_hints = 1;
  int opt_mx_tmem = 1;  // MXFP4, decode-sized tiles: three K blocks per stage, expanded weights in TMEM
  // peer transport: the down GEMM stores every expert output row straight into the memory of
  // the rank whose token it belongs to (1), or leaves it here for that rank to fetch (0)
  int opt_ep_push = 1;
  int opt_ep_dedup = 1;  // peer transport: a remote token with several experts here is fetched once
  unsigned long long *row_dst = nullptr;  // [assign_cap] destinations of the sorted rows (set per pass)
  bool push_rows = false;                 // this pass: the down GEMM uses row_dst     // CTA-pair GEMM: weights evict-first, token tiles evict-last
  int opt_wait_limit_ms = 2000;  // longest wait for another rank's flag (peer-memory transport)
  gptoss::StageTimer timers[8];
  long long launches = 0;
  mutable std::string err;

  // expert parallelism (ep.cu)
  void *ep = nullptr;
};

namespace gptoss {

// router.cu
cudaError_t launch_router_topk(gptoss_moe *h, int layer, const bf16 *t, const int *pos, int T,
                               float *logits_opt, cudaStream_t stream);
// the router rows re-tiled for the tcgen05 router (after w_router is in place)
int build_router_tiles(gptoss_moe *h, LayerWeights &lw);
cudaError_t launch_rmsnorm(bf16 *out, const bf16 *x, const float *w, const int *pos, int T, int H,
                           cudaStream_t stream, long long *launches);

// permute.cu
cudaError_t launch_permute(gptoss_moe *h, cudaStream_t stream);
cudaError_t launch_permute_plan_only(gptoss_moe *h, cudaStream_t stream);
// h->mtile_split = index of the first token tile whose expert is >= e_split
cudaError_t launch_mtile_split(gptoss_moe *h, int e_split, cudaStream_t stream);
cudaError_t launch_combine(gptoss_moe *h, bf16 *x, const int *topk_i_rows, int T,
                           cudaStream_t stream);
cudaError_t launch_reduce_rows(gptoss_moe *h, bf16 *out_rows, int R, cudaStream_t stream,
                               bool skip_empty = false);

// A counting sort of (row, slot) pairs by key on caller-named buffers.
struct PermPlan {
  const int *slot_expert;    // [R, K] key (0 .. El-1) or -1
  const float *slot_weight;  // [R, K]
  int R, K, El;
  int *block_counts;         // [blocks_cap, El]
  int blocks_cap;
  int *expert_offsets;       // [El + 1]
  int *sorted_row;           // [assign_cap]
  float *sorted_weight;      // [assign_cap]
  int *row_of;               // [R * K]
  int *mtile_expert, *mtile_row0, *mtile_rows, *num_mtiles;
  int mtiles_cap, assign_cap;
};
cudaError_t launch_perm_plan(const PermPlan &p, int *status, cudaStream_t stream,
                             long long *launches);
cudaError_t launch_combine_rows(bool residual, bf16 *out, const bf16 *ys, const int *row_of, int R,
                                int K, int H, int assign_cap, int *status, cudaStream_t stream,
                                long long *launches);

// grouped_gemm.cu
// part: 0 = all token tiles; 1 / 2 = the tiles of the experts before / from the split
// written by launch_mtile_split (CTA-pair kernel; the others do everything in part 1)
cudaError_t launch_gate_up(gptoss_moe *h, int layer, cudaStream_t stream, int part = 0);
cudaError_t launch_down(gptoss_moe *h, int layer, cudaStream_t stream);
int make_tmap_2d_bf16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                      uint32_t box_inner, uint32_t box_outer, std::string *err);
int gemm_tile_n(int which);  // N extent of one tile: 0 = gate_up, 1 = down
// grouped_gemm_pair.cu
cudaError_t launch_gate_up_pair(gptoss_moe *h, int layer, cudaStream_t stream, int part = 0);
cudaError_t launch_down_pair(gptoss_moe *h, int layer, cudaStream_t stream);
struct GemmArgs;
cudaError_t launch_linear_pair(int num_sms, const CUtensorMap &tw, const CUtensorMap *tx,
                               const GemmArgs &g, cudaStream_t stream, long long *launches,
                               bool f32_out = false);

// moe_api.cu: error text for entry points that take no handle (read back with
// gptoss_moe_last_error(NULL)); returns `code`
int set_global_error(int code, const char *text);

// weights.cu
cudaError_t launch_f32_to_bf16(bf16 *dst, const float *src, size_t n, cudaStream_t stream,
                               long long *launches);
size_t tiled_weight_elems(int rows, int k, int n_experts);
cudaError_t launch_retile_weights(bf16 *dst, const bf16 *src, int rows, int k, int n_experts,
                                  cudaStream_t stream, long long *launches);
// a tensor of 16 KB tiles as rows of 512 bytes, one tile per box of 32 rows, no swizzle
int make_tmap_tiles_bf16(CUtensorMap *map, const void *base, uint64_t n_tiles, std::string *err);

}  // namespace gptoss

// moe_api.cu: after a stream synchronisation, GPTOSS_E_DEVICE (and the word cleared) when a
// kernel of this engine reported a problem
extern "C" int gptoss_moe_take_status(gptoss_moe *h);
// moe_api.cu: fp32 host tensor -> bf16 device tensor (round to nearest even) through a
// pinned double buffer; errors go to the handle's error text
extern "C" int upload_f32_as_bf16(gptoss_moe *h, gptoss::bf16 *dst, const float *src, size_t n);
// waits for the uploads queued so far / gives the staging buffers back
extern "C" int upload_finish(gptoss_moe *h);
extern "C" void gptoss_moe_release_upload_staging(gptoss_moe *h);
