// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM),
// fed by TMA, with the layer's element-wise work fused into the epilogue.
//
//   gate_up:  hact[r, j] = swiglu(xs[r,:] . W1[e][2j,:] + b1[e][2j],
//                                 xs[r,:] . W1[e][2j+1,:] + b1[e][2j+1])
//   down:     ys[r, n]   = (hact[r,:] . W2[e][n,:] + b2[e][n]) * weight[r]
//
// r runs over the (row, slot) pairs in per-expert order, e is the expert that
// owns r.  Replaces mlp1_kernel / mlp1_120b_kernel and mlp2_kernel_noatomic /
// mlp2_120b_kernel of the reference (getp-csrc/matmul/matmul.cpp:1023-1465,
// :1470-1914) including their fused epilogues (:1384-1430, :1842-1873).
//
// One persistent CTA per SM, 10 warps (the epilogue needs 8 of them: with 4 it,
// not the main loop, set the time per tile):
//   warp 0      TMA producer: A tile [128 rows, 64 k] and B tile [BN rows, 64 k]
//               per stage, 128-byte swizzle, 4-stage mbarrier ring
//   warp 1      allocates TMEM and issues tcgen05.mma (M=128, N=BN, K=16, bf16 ->
//               fp32) from one thread; two accumulators of 256 TMEM columns so the
//               epilogue of a tile overlaps the main loop of the next one
//   warps 2-9   epilogue, two warps per TMEM lane quarter, each taking half of the
//               tile's columns: tcgen05.ld of the warp's 32 TMEM lanes (= 32 rows),
//               bias + SwiGLU (gate and up are adjacent accumulator columns, held
//               by one thread) or bias * routing weight, bf16, 16-byte stores
// Tile order: tile id = m_tile * n_tiles + n_tile, so the CTAs of one wave share
// the m tiles of one or two experts and stream that expert's weight tiles once
// from HBM (the others hit L2).
//
// Weights stay in the checkpoint's own [rows, k] row-major order (K-major for the
// MMA); TMA applies the shared-memory swizzle, so there is no re-tiling pass.
#include <cuda.h>

#include "common.cuh"
#include "engine.h"
#include "gemm_epilogue.cuh"

namespace gptoss {

constexpr int kGemmThreads = 320;  // producer warp, MMA warp, 8 epilogue warps
constexpr int kStages = 4;
constexpr int kAccCols = 256;         // TMEM columns reserved per accumulator
constexpr int kTmemCols = 512;
constexpr int kABytes = kTileM * kTileK * 2;  // 16 KB

// N extent of one tile.  240 divides both 2*IM = 5760 and H = 2880 of the
// gpt-oss shapes (24 and 12 tiles) and keeps the MMA's shared-memory reads
// (A 4 KB + B 7.5 KB per 120 cycles) under the 128 B/clk of one SM.
constexpr int kBN = 240;

int gemm_tile_n(int) { return kBN; }

template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g) {
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N for M=128");
  constexpr int kBBytes = BN * kTileK * 2;
  constexpr int kStageBytes = kABytes + kBBytes;
  static_assert(kBBytes % 1024 == 0, "stage bases must stay 1024-byte aligned");

  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
  uint64_t *empty_bar = full_bar + kStages;
  uint64_t *tfull_bar = empty_bar + kStages;   // [2]
  uint64_t *tempty_bar = tfull_bar + 2;        // [2]
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tempty_bar + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
  // per-epilogue-warp staging tiles behind the barriers (256 bytes reserved)
  unsigned char *epi_stage = smem + kStages * kStageBytes + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], kGemmThreads / 32 - 2);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int n_tiles = (g.n_cols + BN - 1) / BN;
  const int total_tiles = *g.num_mtiles * n_tiles;
  const int kb_count = (g.k_dim + kTileK - 1) / kTileK;

  // the producer and the MMA warp walk the ring whole and one elected lane issues (a loop
  // that only one lane runs makes every load and MMA several times dearer to issue)
  if (warp == 0) {
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // the schedule entry of the next tile is fetched while this tile's loads are
      // issued, so the ring does not drain at a tile boundary
      int e_next = 0, row0_next = 0;
      if (static_cast<int>(blockIdx.x) < total_tiles) {
        e_next = g.mtile_expert[blockIdx.x / n_tiles];
        row0_next = g.mtile_row0[blockIdx.x / n_tiles];
      }
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
        const int e = e_next;
        const int row0 = row0_next;
        const int tile2 = tile + gridDim.x;
        if (tile2 < total_tiles) {
          e_next = g.mtile_expert[tile2 / n_tiles];
          row0_next = g.mtile_row0[tile2 / n_tiles];
        }
        (void)mt;
        const int brow = e * g.n_cols + nt * BN;
        for (int kb = 0; kb < kb_count; kb++) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            set_status(g.status, kStatusWaitTimeoutProducer);
            *abort_flag = 1;
            ok = false;
            break;
          }
          unsigned char *sa = smem + stage * kStageBytes;
          if (elect_one()) {
            mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
            tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kTileK, row0);
            tma_load_2d(sa + kABytes, &tmap_b, &full_bar[stage], kb * kTileK, brow);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    {
      constexpr uint32_t idesc = umma_idesc_bf16(kTileM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          set_status(g.status, kStatusWaitTimeoutMma);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < kb_count; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
            set_status(g.status, kStatusWaitTimeoutMma);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint64_t da = umma_smem_desc_sw128(sa);
          const uint64_t db = umma_smem_desc_sw128(sa + kABytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < kTileK / 16; k++) {
              // +32 bytes along K inside the 128-byte swizzle row = +2 in the
              // descriptor's (address >> 4) field
              umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) are the ones this warp may read
    const int half = (warp - 2) >> 2;  // which half of the tile's columns
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
      const int e = g.mtile_expert[mt];
      const int row0 = g.mtile_row0[mt];
      const int rows = g.mtile_rows[mt];
      const int row = q * 32 + lane;
      float wrow = 0.f;
      if (EPI == kEpiDown && row < rows) wrow = g.row_weight[row0 + row];
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
        set_status(g.status, kStatusWaitTimeoutEpilogue);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kAccCols;
      {
        // two warps share a lane quarter and split the tile's columns
        constexpr int kSplit = ((BN / 16 + 1) / 2) * 16;
        unsigned char *stage = epi_stage + (warp - 2) * kEpiStageBytes;
        if (half == 0)
          epilogue_cols<EPI, kSplit>(taddr, nt * BN, e, row0 + q * 32, rows - q * 32, lane, wrow,
                                     g, stage);
        else
          epilogue_cols<EPI, BN - kSplit>(taddr + kSplit, nt * BN + kSplit, e, row0 + q * 32,
                                          rows - q * 32, lane, wrow, g, stage);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // a role gave up: give copies and MMAs still in flight time to land before
    // shared memory and TMEM go back to the SM
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ SIMT
// CUDA-core grouped GEMM with the same epilogues.  Slow; exists only so tests
// can cross-check the tensor-core kernel on the GPU at sizes the CPU oracle
// cannot reach.  Never selected automatically.
template <int EPI>
__global__ void __launch_bounds__(256)
grouped_gemm_simt_kernel(const bf16 *__restrict__ a, int lda, const bf16 *__restrict__ w,
                         const GemmArgs g) {
  constexpr int BM = 128, BNS = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BNS + 4];
  const int mt = blockIdx.y;
  if (mt >= *g.num_mtiles) return;
  const int e = g.mtile_expert[mt], row0 = g.mtile_row0[mt], rows = g.mtile_rows[mt];
  const int n0 = blockIdx.x * BNS;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const bf16 *wb = w + static_cast<size_t>(e) * g.n_cols * g.k_dim;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < g.k_dim; k0 += BK) {
    for (int i = tid; i < BM * BK; i += 256) {
      const int r = i / BK, k = i % BK;
      float v = 0.f;
      if (r < rows && k0 + k < g.k_dim)
        v = __bfloat162float(a[static_cast<size_t>(row0 + r) * lda + k0 + k]);
      As[k][r] = v;
    }
    for (int i = tid; i < BNS * BK; i += 256) {
      const int n = i / BK, k = i % BK;
      float v = 0.f;
      if (n0 + n < g.n_cols && k0 + k < g.k_dim)
        v = __bfloat162float(wb[static_cast<size_t>(n0 + n) * g.k_dim + k0 + k]);
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; k++) {
      float av[8], bv[4];
#pragma unroll
      for (int i = 0; i < 8; i++) av[i] = As[k][ty * 8 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const float *bias = g.bias + static_cast<size_t>(e) * g.n_cols;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int r = ty * 8 + i;
    if (r >= rows) continue;
    const int grow = row0 + r;
    const int n = n0 + tx * 4;
    if (EPI == kEpiSwiglu) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        if (n + j + 1 < g.n_cols) {
          const float gate = acc[i][j] + bias[n + j];
          const float up = acc[i][j + 1] + bias[n + j + 1];
          g.out[static_cast<size_t>(grow) * g.out_ld + ((n + j) >> 1)] =
              __float2bfloat16_rn(swiglu_act(gate, up, g.limit));
        }
      }
    } else {
      const float wrow = g.row_weight[grow];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (n + j < g.n_cols)
          g.out[static_cast<size_t>(grow) * g.out_ld + n + j] =
              __float2bfloat16_rn((acc[i][j] + bias[n + j]) * wrow);
      }
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn(std::string *err) {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void *p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p) {
    if (err) *err = std::string("cuTensorMapEncodeTiled not available: ") + cudaGetErrorString(e);
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Row-major bf16 matrix [outer, inner] -> tensor map with box [box_outer,
// box_inner] and 128-byte swizzle.  inner*2 bytes must be a multiple of 16.
int make_tmap_2d_bf16(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                      uint32_t box_inner, uint32_t box_outer, std::string *err) {
  EncodeTiledFn fn = get_encode_fn(err);
  if (!fn) return GPTOSS_E_CUDA;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
    return GPTOSS_E_CUDA;
  }
  return GPTOSS_OK;
}

int make_tmap_tiles_bf16(CUtensorMap *map, const void *base, uint64_t n_tiles, std::string *err) {
  EncodeTiledFn fn = get_encode_fn(err);
  if (!fn) return GPTOSS_E_CUDA;
  cuuint64_t dims[2] = {256, n_tiles * 32};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {256, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled (tiles) failed with CUresult " + std::to_string((int)r);
    return GPTOSS_E_CUDA;
  }
  return GPTOSS_OK;
}

template <int EPI>
static cudaError_t launch_tc(gptoss_moe *h, const CUtensorMap &ta, const CUtensorMap &tb,
                             const GemmArgs &g, cudaStream_t stream) {
  constexpr int kStageBytes = kABytes + kBN * kTileK * 2;
  // alignment slack + operand ring + barriers + one staging tile per epilogue warp
  const size_t smem =
      1024 + kStages * kStageBytes + 256 + (kGemmThreads / 32 - 2) * kEpiStageBytes;
  // per device, cheap: set on every launch so every GPU a process drives has it
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_tc_kernel<kBN, EPI>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  grouped_gemm_tc_kernel<kBN, EPI><<<h->num_sms, kGemmThreads, smem, stream>>>(ta, tb, g);
  h->launches++;
  return cudaGetLastError();
}

cudaError_t launch_gate_up(gptoss_moe *h, int layer, cudaStream_t stream, int part) {
  if (h->opt_gemm_impl == GPTOSS_GEMM_PAIR) return launch_gate_up_pair(h, layer, stream, part);
  if (part == 2) return cudaSuccess;  // the other kernels take the whole schedule in part 1
  LayerWeights &lw = h->layers[layer];
  GemmArgs g;
  g.bias = lw.b1;
  g.out = h->hact;
  g.row_weight = nullptr;
  g.mtile_expert = h->mtile_expert;
  g.mtile_row0 = h->mtile_row0;
  g.mtile_rows = h->mtile_rows;
  g.num_mtiles = h->num_mtiles;
  g.k_dim = h->H;
  g.n_cols = 2 * h->IM;
  g.out_ld = h->IM;
  g.limit = h->cfg.swiglu_limit;
  g.status = h->status;
  if (h->opt_gemm_impl == GPTOSS_GEMM_SIMT) {
    dim3 grid((g.n_cols + 63) / 64, h->mtiles_cap);
    grouped_gemm_simt_kernel<kEpiSwiglu><<<grid, 256, 0, stream>>>(h->xs, h->H, lw.w1, g);
    h->launches++;
    return cudaGetLastError();
  }
  return launch_tc<kEpiSwiglu>(h, h->tmap_xs, lw.tmap_w1, g, stream);
}

cudaError_t launch_down(gptoss_moe *h, int layer, cudaStream_t stream) {
  if (h->opt_gemm_impl == GPTOSS_GEMM_PAIR) return launch_down_pair(h, layer, stream);
  LayerWeights &lw = h->layers[layer];
  GemmArgs g;
  g.bias = lw.b2;
  g.out = h->ys;
  g.row_weight = h->sorted_weight;
  g.mtile_expert = h->mtile_expert;
  g.mtile_row0 = h->mtile_row0;
  g.mtile_rows = h->mtile_rows;
  g.num_mtiles = h->num_mtiles;
  g.k_dim = h->IM;
  g.n_cols = h->H;
  g.out_ld = h->H;
  g.limit = h->cfg.swiglu_limit;
  g.status = h->status;
  if (h->opt_gemm_impl == GPTOSS_GEMM_SIMT) {
    dim3 grid((g.n_cols + 63) / 64, h->mtiles_cap);
    grouped_gemm_simt_kernel<kEpiDown><<<grid, 256, 0, stream>>>(h->hact, h->IM, lw.w2, g);
    h->launches++;
    return cudaGetLastError();
  }
  return launch_tc<kEpiDown>(h, h->tmap_h, lw.tmap_w2, g, stream);
}

}  // namespace gptoss
