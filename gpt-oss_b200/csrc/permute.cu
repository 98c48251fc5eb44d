// Token permutation into per-expert groups, and the inverse (combine).
//
// Replaces count_expert_assignments_kernel / exclusive_scan_small_kernel /
// build_expert_assignments_kernel (getp-csrc/utility/utility.cpp:1058, :758,
// :1079) and reduce_mlp2_slots_kernel + residual_add_batch_kernel
// (utility.cpp:701-726, :158-173) of the reference.
//
// Input of the expert stage: R rows, each with K slots (local expert id or -1,
// routing weight).  Output: the (row, slot) pairs sorted by expert, in flat
// (row, slot) order inside an expert - a stable counting sort, so the result
// is the same on every run (the reference's atomic scatter is not).
//   count:        per-CTA histogram of 128 rows           -> block_counts
//   scan_scatter: every CTA re-derives its own base offsets from block_counts,
//                 ranks its items with warp match + per-warp histograms and
//                 scatters; CTA 0 also writes expert_offsets and the M-tile
//                 schedule of the grouped GEMMs
//   gather:       copies the source rows into sorted order (16-byte accesses)
// All kernels are bound by latency (<= 200k items) or HBM (gather, combine).
#include <atomic>

#include "common.cuh"
#include "engine.h"

namespace gptoss {

constexpr int kScanThreads = 512;

// <<<grid, block, smem, stream>>> with the stream-serialization attribute when the engine
// runs its layer with programmatic dependent launches (every kernel launched this way
// starts with grid_dependency_wait()).
template <typename... KArgs, typename... Args>
static cudaError_t launch_kernel(void (*kernel)(KArgs...), unsigned grid, unsigned block,
                                 size_t smem, cudaStream_t stream, bool dependent, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__global__ void __launch_bounds__(256)
perm_count_kernel(const int *__restrict__ slot_expert, int R, int K, int El,
                  int *__restrict__ block_counts, int *status) {
  extern __shared__ int hist[];
  grid_dependency_wait();
  grid_launch_dependents();
  for (int e = threadIdx.x; e < El; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int r0 = blockIdx.x * kPermTokens;
  const int items = kPermTokens * K;
  for (int i = threadIdx.x; i < items; i += blockDim.x) {
    const int row = r0 + i / K;
    if (row < R) {
      const int e = slot_expert[static_cast<size_t>(r0) * K + i];
      if (e >= El) {
        set_status(status, kStatusBadIndex);
      } else if (e >= 0) {
        atomicAdd(&hist[e], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < El; e += blockDim.x)
    block_counts[static_cast<size_t>(blockIdx.x) * El + e] = hist[e];
}

__global__ void __launch_bounds__(kScanThreads)
perm_scan_scatter_kernel(const int *__restrict__ slot_expert,
                         const float *__restrict__ slot_weight, int R, int K, int El,
                         const int *__restrict__ block_counts, int nblocks,
                         int *__restrict__ expert_offsets, int *__restrict__ sorted_row,
                         float *__restrict__ sorted_weight, int *__restrict__ row_of,
                         int *__restrict__ mtile_expert, int *__restrict__ mtile_row0,
                         int *__restrict__ mtile_rows, int *__restrict__ num_mtiles,
                         int mtiles_cap, int assign_cap, int *status, int tile_rows) {
  extern __shared__ int sm[];
  int *s_tot = sm;                 // [El] rows of each expert over all CTAs
  int *s_base = sm + El;           // [El] next free position for this CTA
  int *s_off = sm + 2 * El;        // [El + 1] exclusive scan of s_tot
  int *s_whist = sm + 3 * El + 1;  // [warps][El]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kScanThreads / 32;
  grid_dependency_wait();
  grid_launch_dependents();

  // totals and this CTA's base per expert: the CTAs' counts are split over
  // kScanThreads / El thread groups (adjacent threads = adjacent experts) and summed
  // through shared atomics, so a long list of CTAs does not serialise on El threads
  for (int e = tid; e < El; e += kScanThreads) {
    s_tot[e] = 0;
    s_base[e] = 0;
  }
  __syncthreads();
  {
    const int groups = El < kScanThreads ? kScanThreads / El : 1;
    const int grp = tid / El;  // 0 for every thread when El >= kScanThreads
    if (grp < groups) {
      for (int e = tid - grp * El; e < El; e += kScanThreads) {
        int tot = 0, before = 0;
        for (int b = grp; b < nblocks; b += groups) {
          const int c = block_counts[static_cast<size_t>(b) * El + e];
          tot += c;
          if (b < static_cast<int>(blockIdx.x)) before += c;
        }
        if (tot) atomicAdd(&s_tot[e], tot);
        if (before) atomicAdd(&s_base[e], before);
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive scan over experts: each lane owns a run of consecutive experts
    const int per = (El + 31) / 32;
    int local = 0;
    for (int j = 0; j < per; j++) {
      const int e = lane * per + j;
      if (e < El) local += s_tot[e];
    }
    int incl = local;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    int run = incl - local;
    for (int j = 0; j < per; j++) {
      const int e = lane * per + j;
      if (e < El) {
        s_off[e] = run;
        run += s_tot[e];
      }
    }
    if (lane == 31) s_off[El] = incl;
  }
  __syncthreads();
  for (int e = tid; e < El; e += kScanThreads) s_base[e] += s_off[e];

  if (blockIdx.x == 0) {
    for (int e = tid; e <= El; e += kScanThreads) expert_offsets[e] = s_off[e];
    // M-tile schedule: expert e gets ceil(rows / kTileM) tiles, experts in order
    if (warp == 0) {
      const int per = (El + 31) / 32;
      int local = 0;
      for (int j = 0; j < per; j++) {
        const int e = lane * per + j;
        if (e < El) local += (s_tot[e] + tile_rows - 1) / tile_rows;
      }
      int incl = local;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
      }
      int mt = incl - local;
      for (int j = 0; j < per; j++) {
        const int e = lane * per + j;
        if (e < El) {
          const int rows = s_tot[e];
          // tiles of 128 rows are the MMA's fixed M; wider tiles are its N, which may be
          // any multiple of 16: spread the expert's rows evenly over its tiles
          const int cnt = (rows + tile_rows - 1) / tile_rows;
          const int step =
              (tile_rows == kTileM || cnt == 0) ? tile_rows : (((rows + cnt - 1) / cnt + 15) & ~15);
          for (int i = 0; i * step < rows; i++, mt++) {
            if (mt < mtiles_cap) {
              mtile_expert[mt] = e;
              mtile_row0[mt] = s_off[e] + i * step;
              mtile_rows[mt] = min(step, rows - i * step);
            } else {
              set_status(status, kStatusBadIndex);
            }
          }
        }
      }
      if (lane == 31) *num_mtiles = min(incl, mtiles_cap);
    }
  }

  const int r0 = blockIdx.x * kPermTokens;
  const int items = kPermTokens * K;
  for (int c0 = 0; c0 < items; c0 += kScanThreads) {
    __syncthreads();
    for (int i = tid; i < kWarps * El; i += kScanThreads) s_whist[i] = 0;
    __syncthreads();
    const int i = c0 + tid;
    const int row = r0 + i / K;
    int e = -1;
    float wgt = 0.f;
    if (i < items && row < R) {
      e = slot_expert[static_cast<size_t>(r0) * K + i];
      wgt = slot_weight[static_cast<size_t>(r0) * K + i];
      if (e >= El) e = -1;
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) s_whist[warp * El + e] = __popc(peers);
    __syncthreads();
    if (e >= 0) {
      int before = 0;
      for (int w = 0; w < warp; w++) before += s_whist[w * El + e];
      const int dst = s_base[e] + before + rank;
      if (dst < assign_cap) {
        sorted_row[dst] = row;
        sorted_weight[dst] = wgt;
        row_of[static_cast<size_t>(r0) * K + i] = dst;
      } else {
        set_status(status, kStatusBadIndex);
        row_of[static_cast<size_t>(r0) * K + i] = -1;
      }
    } else if (i < items && row < R) {
      row_of[static_cast<size_t>(r0) * K + i] = -1;
    }
    __syncthreads();
    for (int ee = tid; ee < El; ee += kScanThreads) {
      int add = 0;
      for (int w = 0; w < kWarps; w++) add += s_whist[w * El + ee];
      s_base[ee] += add;
    }
  }
}

// xs[r, :] = rows[sorted_row[r], :] for r < expert_offsets[El]; one warp per row.
__global__ void __launch_bounds__(256)
gather_rows_kernel(bf16 *__restrict__ xs, const bf16 *__restrict__ rows,
                   const int *__restrict__ sorted_row, const int *__restrict__ expert_offsets,
                   int El, int H, int R, int *status) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int total = expert_offsets[El];
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  const int n4 = H >> 3;
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += nwarps) {
    const int src = sorted_row[r];
    if (src < 0 || src >= R) {
      set_status(status, kStatusBadIndex);
      continue;
    }
    const uint4 *s4 = reinterpret_cast<const uint4 *>(rows + static_cast<size_t>(src) * H);
    uint4 *d4 = reinterpret_cast<uint4 *>(xs + static_cast<size_t>(r) * H);
    // eight loads in flight per lane before the first store; the copy is written once and
    // read once by the next kernel: streaming stores
    for (int p0 = lane; p0 < n4; p0 += 256) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++)
        if (p0 + u * 32 < n4) v[u] = __ldg(s4 + p0 + u * 32);
#pragma unroll
      for (int u = 0; u < 8; u++)
        if (p0 + u * 32 < n4) __stcs(d4 + p0 + u * 32, v[u]);
    }
  }
}

// RESIDUAL: x[row] = bf16(float(x[row]) + sum_k ys[row_of[row,k]]), rows without
//           any valid slot untouched (inactive rows keep their x).
// otherwise: out[row] = bf16(sum_k ys[row_of[row,k]]) for every row (zero when
//           the row has no valid slot) - the owner-side pre-reduction under
//           expert parallelism (getp-csrc/expert.cpp:394-410).
// SKIP_EMPTY: rows without a valid slot are not written at all (nobody reads them).
template <bool RESIDUAL, bool SKIP_EMPTY = false>
__global__ void __launch_bounds__(256)
combine_rows_kernel(bf16 *__restrict__ out, const bf16 *__restrict__ ys,
                    const int *__restrict__ row_of, int R, int K, int H, int assign_cap,
                    int *status) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= R) return;
  int src[GPTOSS_MAX_TOPK];
  int nvalid = 0;
#pragma unroll
  for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
    src[k] = -1;
    if (k < K) {
      const int s = row_of[static_cast<size_t>(row) * K + k];
      if (s >= assign_cap) {
        set_status(status, kStatusBadIndex);
      } else if (s >= 0) {
        src[k] = s;
        nvalid++;
      }
    }
  }
  if ((RESIDUAL || SKIP_EMPTY) && nvalid == 0) return;
  uint4 *o4 = reinterpret_cast<uint4 *>(out + static_cast<size_t>(row) * H);
  const int n4 = H >> 3;
  // two 16-byte columns per lane and trip: up to 2 * (K + 1) loads in flight per lane
  for (int p0 = lane; p0 < n4; p0 += 64) {
    const int p1 = p0 + 32;
    const bool two = p1 < n4;
    uint4 xv[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint4 yv[2][GPTOSS_MAX_TOPK];
    if (RESIDUAL) {
      xv[0] = o4[p0];
      if (two) xv[1] = o4[p1];
    }
#pragma unroll
    for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
      if (k < K && src[k] >= 0) {
        const uint4 *y4 = reinterpret_cast<const uint4 *>(ys + static_cast<size_t>(src[k]) * H);
        yv[0][k] = __ldcs(y4 + p0);
        if (two) yv[1][k] = __ldcs(y4 + p1);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
      if (u == 1 && !two) break;
      float s[8];
#pragma unroll
      for (int i = 0; i < 8; i++) s[i] = 0.f;
#pragma unroll
      for (int k = 0; k < GPTOSS_MAX_TOPK; k++) {
        if (k < K && src[k] >= 0) {
          const uint4 v = yv[u][k];
          s[0] += bf16_lo(v.x); s[1] += bf16_hi(v.x); s[2] += bf16_lo(v.y); s[3] += bf16_hi(v.y);
          s[4] += bf16_lo(v.z); s[5] += bf16_hi(v.z); s[6] += bf16_lo(v.w); s[7] += bf16_hi(v.w);
        }
      }
      const uint4 v = xv[u];  // zeros without a residual
      uint4 o;
      o.x = pack_bf16(bf16_lo(v.x) + s[0], bf16_hi(v.x) + s[1]);
      o.y = pack_bf16(bf16_lo(v.y) + s[2], bf16_hi(v.y) + s[3]);
      o.z = pack_bf16(bf16_lo(v.z) + s[4], bf16_hi(v.z) + s[5]);
      o.w = pack_bf16(bf16_lo(v.w) + s[6], bf16_hi(v.w) + s[7]);
      o4[u == 0 ? p0 : p1] = o;
    }
  }
}

cudaError_t launch_permute(gptoss_moe *h, cudaStream_t stream) {
  cudaError_t e = launch_permute_plan_only(h, stream);
  if (e != cudaSuccess || h->stage_R <= 0) return e;
  h->launches++;
  return launch_kernel(gather_rows_kernel, h->num_sms * 4, 256, 0, stream,
                       h->opt_dependent_launch != 0, h->xs, h->stage_rows, h->sorted_row,
                       h->expert_offsets, h->El, h->H, h->stage_R, h->status);
}

// The tile schedule is ordered by expert: first tile of an expert >= e_split (the tile
// count when there is none).
__global__ void mtile_split_kernel(const int *__restrict__ mtile_expert,
                                   const int *__restrict__ num_mtiles, int e_split,
                                   int *__restrict__ out) {
  __shared__ int best;
  const int n = *num_mtiles;
  if (threadIdx.x == 0) best = n;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    if (mtile_expert[i] >= e_split) {
      atomicMin(&best, i);
      break;  // later tiles of this thread are larger
    }
  __syncthreads();
  if (threadIdx.x == 0) *out = best;
}

cudaError_t launch_mtile_split(gptoss_moe *h, int e_split, cudaStream_t stream) {
  mtile_split_kernel<<<1, 256, 0, stream>>>(h->mtile_expert, h->num_mtiles, e_split,
                                            h->mtile_split);
  h->launches++;
  return cudaGetLastError();
}

// Sorted order and tile schedule only; the caller gathers the rows.
cudaError_t launch_permute_plan_only(gptoss_moe *h, cudaStream_t stream) {
  const int R = h->stage_R, K = h->K, El = h->El;
  // row tile of the GEMM schedule: 128 = the single-CTA kernel's fixed M; the
  // CTA-pair kernel takes token tiles of up to 256, or up to 64 when MXFP4 weights
  // meet a decode-sized batch (on average at most 128 rows per expert)
  h->cur_tile_rows = kTileM;
  if (h->opt_gemm_impl == GPTOSS_GEMM_PAIR) {
    const bool decode = h->cfg.weight_format == GPTOSS_WEIGHTS_MXFP4 &&
                        static_cast<long long>(R) * K <= 128ll * El;
    h->cur_tile_rows = decode ? 64 : 256;
  }
  const int nblocks = (R + kPermTokens - 1) / kPermTokens;
  if (R <= 0) {
    // nothing routed here: empty schedule
    cudaError_t e = cudaMemsetAsync(h->expert_offsets, 0, sizeof(int) * (El + 1), stream);
    if (e != cudaSuccess) return e;
    return cudaMemsetAsync(h->num_mtiles, 0, sizeof(int), stream);
  }
  if (nblocks > h->perm_blocks_cap) return cudaErrorInvalidValue;
  const bool dep = h->opt_dependent_launch != 0;
  h->launches++;
  cudaError_t e = launch_kernel(perm_count_kernel, nblocks, 256, El * sizeof(int), stream, dep,
                                h->stage_expert, R, K, El, h->block_counts, h->status);
  if (e != cudaSuccess) return e;
  const size_t smem = (static_cast<size_t>(3 + kScanThreads / 32) * El + 1) * sizeof(int);
  h->launches++;
  return launch_kernel(perm_scan_scatter_kernel, nblocks, kScanThreads, smem, stream, dep,
                       h->stage_expert, h->stage_weight, R, K, El, h->block_counts, nblocks,
                       h->expert_offsets, h->sorted_row, h->sorted_weight, h->row_of,
                       h->mtile_expert, h->mtile_row0, h->mtile_rows, h->num_mtiles, h->mtiles_cap,
                       h->assign_cap, h->status, h->cur_tile_rows);
}

cudaError_t launch_combine(gptoss_moe *h, bf16 *x, const int *, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  const int warps = 8;
  h->launches++;
  return launch_kernel(combine_rows_kernel<true, false>, (T + warps - 1) / warps, warps * 32, 0,
                       stream, h->opt_dependent_launch != 0, x, h->ys, h->row_of, T, h->K, h->H,
                       h->assign_cap, h->status);
}

cudaError_t launch_reduce_rows(gptoss_moe *h, bf16 *out_rows, int R, cudaStream_t stream,
                               bool skip_empty) {
  if (R <= 0) return cudaSuccess;
  const int warps = 8;
  if (skip_empty)
    combine_rows_kernel<false, true><<<(R + warps - 1) / warps, warps * 32, 0, stream>>>(
        out_rows, h->ys, h->row_of, R, h->K, h->H, h->assign_cap, h->status);
  else
    combine_rows_kernel<false><<<(R + warps - 1) / warps, warps * 32, 0, stream>>>(
        out_rows, h->ys, h->row_of, R, h->K, h->H, h->assign_cap, h->status);
  h->launches++;
  return cudaGetLastError();
}

// The same kernels on caller-named buffers: expert parallelism sorts a rank's
// tokens by OWNER with them (one "expert" per peer rank) before dispatch.
cudaError_t launch_perm_plan(const PermPlan &p, int *status, cudaStream_t stream,
                             long long *launches) {
  if (p.R <= 0) {
    cudaError_t e = cudaMemsetAsync(p.expert_offsets, 0, sizeof(int) * (p.El + 1), stream);
    if (e != cudaSuccess) return e;
    return cudaMemsetAsync(p.num_mtiles, 0, sizeof(int), stream);
  }
  const int nblocks = (p.R + kPermTokens - 1) / kPermTokens;
  if (nblocks > p.blocks_cap) return cudaErrorInvalidValue;
  perm_count_kernel<<<nblocks, 256, p.El * sizeof(int), stream>>>(p.slot_expert, p.R, p.K, p.El,
                                                                   p.block_counts, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const size_t smem = (static_cast<size_t>(3 + kScanThreads / 32) * p.El + 1) * sizeof(int);
  perm_scan_scatter_kernel<<<nblocks, kScanThreads, smem, stream>>>(
      p.slot_expert, p.slot_weight, p.R, p.K, p.El, p.block_counts, nblocks, p.expert_offsets,
      p.sorted_row, p.sorted_weight, p.row_of, p.mtile_expert, p.mtile_row0, p.mtile_rows,
      p.num_mtiles, p.mtiles_cap, p.assign_cap, status, kTileM);
  if (launches) *launches += 2;
  return cudaGetLastError();
}

cudaError_t launch_combine_rows(bool residual, bf16 *out, const bf16 *ys, const int *row_of, int R,
                                int K, int H, int assign_cap, int *status, cudaStream_t stream,
                                long long *launches) {
  if (R <= 0) return cudaSuccess;
  const int warps = 8;
  const int grid = (R + warps - 1) / warps;
  if (residual)
    combine_rows_kernel<true><<<grid, warps * 32, 0, stream>>>(out, ys, row_of, R, K, H,
                                                               assign_cap, status);
  else
    combine_rows_kernel<false><<<grid, warps * 32, 0, stream>>>(out, ys, row_of, R, K, H,
                                                                assign_cap, status);
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace gptoss

// ---------------------------------------------------------------------------
// Permutation without any allocation: gptoss_moe_permute_static.
//
// Same two kernels as launch_permute (count, scan + scatter), but the scratch
// they need - the per-CTA expert histograms and the M-tile schedule - lives in a
// fixed array in device memory that is part of the library image, so the call
// needs neither an engine handle nor cudaMalloc.  Every GPU that loads the
// library holds the array (kStaticInts * 4 bytes = 78 KB) until the process
// exits.  Limits: kStaticMaxRows rows, kStaticMaxExperts experts, top-k <= 8.
namespace gptoss {

constexpr int kStaticMaxRows = 8192;
constexpr int kStaticMaxExperts = 256;
constexpr int kStaticBlocks = kStaticMaxRows / kPermTokens;  // 64 CTAs at most
constexpr int kStaticMtilesPad = 1024;  // >= 8192 * 8 / 128 + 256 + 1 M tiles
// ints: [block counts: 64 x 256][mtile_expert | mtile_row0 | mtile_rows: 3 x 1024][num_mtiles, pad]
constexpr int kStaticCountsInts = kStaticBlocks * kStaticMaxExperts;
constexpr int kStaticInts = kStaticCountsInts + 3 * kStaticMtilesPad + 64;

static __device__ __align__(256) int g_perm_scratch[kStaticInts];

// In host code `g_perm_scratch` is only a handle for the runtime, not an address
// a kernel can use; the device address is looked up once per device.  Several host
// threads may make the first call on a device at the same time: each looks the address
// up and stores the same value.
static std::atomic<int *> g_perm_scratch_dev[64];

static cudaError_t static_scratch(int **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  int *p = g_perm_scratch_dev[dev].load(std::memory_order_acquire);
  if (!p) {
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_perm_scratch);
    if (e != cudaSuccess) return e;
    g_perm_scratch_dev[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return cudaSuccess;
}

}  // namespace gptoss

extern "C" int gptoss_moe_permute_static(const int *slot_expert, const float *slot_weight,
                                         int n_rows, int top_k, int n_experts,
                                         int *expert_offsets, int *sorted_row,
                                         float *sorted_weight, int *row_of, void *stream) {
  using namespace gptoss;
  if (n_rows < 0 || top_k <= 0 || n_experts <= 0 || !expert_offsets)
    return set_global_error(GPTOSS_E_INVALID, "gptoss_moe_permute_static: bad argument");
  if (n_rows > kStaticMaxRows || n_experts > kStaticMaxExperts || top_k > GPTOSS_MAX_TOPK)
    return set_global_error(
        GPTOSS_E_CAPACITY,
        "gptoss_moe_permute_static: at most 8192 rows, 256 experts and top-8 fit the fixed scratch");
  if (n_rows > 0 && (!slot_expert || !slot_weight || !sorted_row || !sorted_weight || !row_of))
    return set_global_error(GPTOSS_E_INVALID, "gptoss_moe_permute_static: null buffer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int *scratch = nullptr;
  cudaError_t e = static_scratch(&scratch);
  if (e != cudaSuccess) return set_global_error(GPTOSS_E_CUDA, cudaGetErrorString(e));
  if (n_rows == 0) {
    e = cudaMemsetAsync(expert_offsets, 0, sizeof(int) * (n_experts + 1), st);
    return e == cudaSuccess ? GPTOSS_OK : set_global_error(GPTOSS_E_CUDA, cudaGetErrorString(e));
  }
  int *block_counts = scratch;
  int *mtile_expert = scratch + kStaticCountsInts;
  int *mtile_row0 = mtile_expert + kStaticMtilesPad;
  int *mtile_rows = mtile_row0 + kStaticMtilesPad;
  int *num_mtiles = mtile_rows + kStaticMtilesPad;
  // No status word: slots whose expert id is out of range are skipped, as documented, and
  // the sizes were checked above, so the kernels have nothing to report.
  int *status = nullptr;
  // the array keeps what the previous call left: the tile count starts from zero again;
  // everything else the kernels read is fully rewritten first
  e = cudaMemsetAsync(num_mtiles, 0, sizeof(int), st);
  if (e != cudaSuccess) return set_global_error(GPTOSS_E_CUDA, cudaGetErrorString(e));
  const int nblocks = (n_rows + kPermTokens - 1) / kPermTokens;
  perm_count_kernel<<<nblocks, 256, n_experts * sizeof(int), st>>>(slot_expert, n_rows, top_k,
                                                                   n_experts, block_counts, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_global_error(GPTOSS_E_CUDA, cudaGetErrorString(e));
  const size_t smem = (static_cast<size_t>(3 + kScanThreads / 32) * n_experts + 1) * sizeof(int);
  perm_scan_scatter_kernel<<<nblocks, kScanThreads, smem, st>>>(
      slot_expert, slot_weight, n_rows, top_k, n_experts, block_counts, nblocks, expert_offsets,
      sorted_row, sorted_weight, row_of, mtile_expert, mtile_row0, mtile_rows, num_mtiles,
      kStaticMtilesPad, n_rows * top_k, status, kTileM);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_global_error(GPTOSS_E_CUDA, cudaGetErrorString(e));
  return GPTOSS_OK;
}
