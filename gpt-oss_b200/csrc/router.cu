// Router stage: logits = t . Wr^T + b, top-K by value (lowest index first on
// equal values), softmax over the K selected logits.  One kernel; the logits
// never go to HBM unless the debug tap asks for them.
//
// Replaces matmul_router_kernel (getp-csrc/matmul/matmul.cpp:945-1019) and
// fused_topk_softmax_batch_kernel (getp-csrc/utility/utility.cpp:274-365) of the
// reference.  Bound by HBM: the only large stream is t [T,H] bf16, read once.
//
// Two kernels: router_tx_kernel (tcgen05, further down; the default) and
// router_topk_kernel (mma.sync, "router_impl" 1), described first.
//
// Layout of router_topk_kernel: a CTA owns 32 consecutive tokens.  8 warps = 2 token groups of 16 x 4
// expert slices; bf16 tensor-core MMAs (m16n8k16, fp32 accumulate) over K chunks
// of 64.  A ninth warp is the producer: an elected lane issues two TMA tile loads per
// chunk (32 token rows, all expert rows; 128-byte swizzle, rows past T or E read
// as zeros) into a ring of 3 to 8 stages guarded by full / empty mbarriers, so the
// compute warps spend their instructions on ldmatrix and MMAs only.  The fp32 logits
// of the 32 tokens then sit in shared memory and one warp per token does the
// selection in registers.
//
// Exact selection: fp32 tensor-core accumulation differs from the reference's
// double-precision dot product by up to ~1e-5, enough to flip two near-tied
// experts.  A token whose top-(K+1) logits contain two neighbours closer than
// kTieGuard gets the logits of every contender (anything within 2*kTieGuard of
// the K-th value) recomputed in fp64 by the same warp, and is re-selected.
#include "common.cuh"
#include "engine.h"

namespace gptoss {

constexpr int kRtTokens = 32;      // tokens per CTA
constexpr int kRtKC = 64;          // K elements per pipeline stage
// ring depth per expert-tile count: enough bytes in flight per SM to cover HBM
// latency while two CTAs still fit one SM where possible
template <int NT> struct RtStages { static constexpr int value = NT == 1 ? 8 : (NT == 2 ? 6 : (NT == 4 ? 4 : 3)); };
constexpr int kRtRowBytes = 128;   // one 64-element K chunk of a row; 128-byte swizzle
constexpr int kRtComputeWarps = 8;
constexpr int kRtThreads = (kRtComputeWarps + 1) * 32;
constexpr float kTieGuard = 2.5e-4f;

// byte offset of 16-byte chunk c of row r inside a 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128(int r, int c) {
  return static_cast<uint32_t>(r) * kRtRowBytes + (static_cast<uint32_t>(c ^ (r & 7)) << 4);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                            uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t &r0, uint32_t &r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4],
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, "
      "{%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Dot product of two bf16 rows the way the reference's CPU matmul does it
// (run.cpp:356-369): exact float products summed in double, rounded to float
// once at the end.  Whole warp cooperates; every lane returns the result.
__device__ __forceinline__ float warp_exact_dot(const bf16 *a, const bf16 *b, int H, int lane) {
  // Loads of up to 12 pieces per lane and operand (one round trip for H <= 3072) are
  // issued together and four independent accumulators keep the fp64 add chains short.  The order
  // of the fp64 additions differs from the reference's left-to-right sum by
  // rounding errors ~1e-16 relative, which the final rounding to float hides.
  double acc0 = 0.0, acc1 = 0.0, acc2 = 0.0, acc3 = 0.0;
  const uint4 *a4 = reinterpret_cast<const uint4 *>(a);
  const uint4 *b4 = reinterpret_cast<const uint4 *>(b);
  const int n4 = H >> 3;
  constexpr int kU = 12;
  for (int p0 = lane; p0 < n4; p0 += 32 * kU) {
    uint4 av[kU], bv[kU];
#pragma unroll
    for (int u = 0; u < kU; u++) {
      const int p = p0 + u * 32;
      av[u] = p < n4 ? __ldg(a4 + p) : make_uint4(0, 0, 0, 0);
      bv[u] = p < n4 ? __ldg(b4 + p) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kU; u++) {
      acc0 += static_cast<double>(__fmul_rn(bf16_lo(av[u].x), bf16_lo(bv[u].x)));
      acc1 += static_cast<double>(__fmul_rn(bf16_hi(av[u].x), bf16_hi(bv[u].x)));
      acc2 += static_cast<double>(__fmul_rn(bf16_lo(av[u].y), bf16_lo(bv[u].y)));
      acc3 += static_cast<double>(__fmul_rn(bf16_hi(av[u].y), bf16_hi(bv[u].y)));
      acc0 += static_cast<double>(__fmul_rn(bf16_lo(av[u].z), bf16_lo(bv[u].z)));
      acc1 += static_cast<double>(__fmul_rn(bf16_hi(av[u].z), bf16_hi(bv[u].z)));
      acc2 += static_cast<double>(__fmul_rn(bf16_lo(av[u].w), bf16_lo(bv[u].w)));
      acc3 += static_cast<double>(__fmul_rn(bf16_hi(av[u].w), bf16_hi(bv[u].w)));
    }
  }
  double acc = (acc0 + acc1) + (acc2 + acc3);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  return __double2float_rn(acc);
}

// NT = 8-expert MMA tiles per warp; the CTA covers EPAD = 32*NT experts.
// SPLIT = CTAs of a cluster that share one group of 32 tokens, each taking 1/SPLIT of the
// K chunks (small batches: the K loop is a latency chain and there are SMs to spare); the
// partial logits meet in the first CTA through distributed shared memory, added in rank
// order, and the first CTA selects.
template <int NT, int SPLIT>
__global__ void __launch_bounds__(kRtThreads)
router_topk_kernel(const __grid_constant__ CUtensorMap tmap_t,
                   const __grid_constant__ CUtensorMap tmap_w, const bf16 *__restrict__ t,
                   const bf16 *__restrict__ w_router, const float *__restrict__ b_router,
                   const int *__restrict__ pos, int T, int H, int E, int K,
                   int *__restrict__ topk_i, float *__restrict__ topk_v,
                   float *__restrict__ logits_out, int exact_ties, int *status) {
  constexpr int EPAD = 32 * NT;
  constexpr int kRtStages = RtStages<NT>::value;
  constexpr int kTokBytes = kRtTokens * kRtRowBytes;           // 4 KB
  constexpr int kStageBytes = kTokBytes + EPAD * kRtRowBytes;  // both tiles 1024-byte aligned
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + kRtStages * kStageBytes);
  uint64_t *empty_bar = full_bar + kRtStages;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(empty_bar + kRtStages);
  float *lg = reinterpret_cast<float *>(smem + kRtStages * kStageBytes + 256);  // [32][EPAD]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int crank = SPLIT > 1 ? static_cast<int>(blockIdx.x % SPLIT) : 0;  // rank in the cluster
  const int tok0 = static_cast<int>(blockIdx.x / SPLIT) * kRtTokens;
  const int nk_all = (H + kRtKC - 1) / kRtKC;
  const int kc_lo = crank * nk_all / SPLIT, kc_hi = (crank + 1) * nk_all / SPLIT;

  if (tid == 0) {
    for (int s = 0; s < kRtStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kRtComputeWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_t);
    tma_prefetch_desc(&tmap_w);
  }
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  const int tg = warp & 1;   // token group: rows tg*16 .. +15
  const int sl = warp >> 1;  // expert slice: experts sl*NT*8 .. +NT*8-1

  if (warp == kRtComputeWarps) {
    {
      int stage = 0;
      uint32_t phase = 0;
      for (int kc = kc_lo; kc < kc_hi; kc++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
          set_status(status, kStatusWaitTimeoutProducer);
          *abort_flag = 1;
          break;
        }
        unsigned char *dst = smem + stage * kStageBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(dst, &tmap_t, &full_bar[stage], kc * kRtKC, tok0);
          tma_load_2d(dst + kTokBytes, &tmap_w, &full_bar[stage], kc * kRtKC, 0);
        }
        if (++stage == kRtStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    int stage = 0;
    uint32_t phase = 0;
    for (int kc = kc_lo; kc < kc_hi; kc++) {
      if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
        set_status(status, kStatusWaitTimeoutMma);
        *abort_flag = 1;
        break;
      }
      const uint32_t sbase = smem_u32(smem + stage * kStageBytes);
      const uint32_t w_base = sbase + kTokBytes;
      const int a_row = tg * 16 + (lane & 15);
#pragma unroll
      for (int kk = 0; kk < kRtKC / 16; kk++) {
        uint32_t a[4];
        ldmatrix_x4(sbase + sw128(a_row, kk * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
        if constexpr (NT == 1) {
          uint32_t b0, b1;
          const int row = sl * 8 + (lane & 7);
          ldmatrix_x2(w_base + sw128(row, kk * 2 + ((lane >> 3) & 1)), b0, b1);
          mma_bf16_16816(acc[0], a, b0, b1);
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b0, b1, b2, b3;
            const int mat = lane >> 3;
            const int row = (sl * NT + nt + (mat >> 1)) * 8 + (lane & 7);
            ldmatrix_x4(w_base + sw128(row, kk * 2 + (mat & 1)), b0, b1, b2, b3);
            mma_bf16_16816(acc[nt], a, b0, b1);
            mma_bf16_16816(acc[nt + 1], a, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == kRtStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  }
  // accumulators -> shared logits [32][EPAD]
  if (warp < kRtComputeWarps) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int col = (sl * NT + nt) * 8 + (lane & 3) * 2;
      const int r0 = tg * 16 + (lane >> 2);
      lg[r0 * EPAD + col] = acc[nt][0];
      lg[r0 * EPAD + col + 1] = acc[nt][1];
      lg[(r0 + 8) * EPAD + col] = acc[nt][2];
      lg[(r0 + 8) * EPAD + col + 1] = acc[nt][3];
    }
  }
  if constexpr (SPLIT > 1) {
    // every CTA's partial logits are in its shared memory; the first CTA adds the others'
    // in rank order, then everybody may leave
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (crank == 0) {
      const uint32_t lg_s = smem_u32(lg);
      for (int i = tid; i < kRtTokens * EPAD; i += kRtThreads) {
        float v = lg[i];
#pragma unroll
        for (int r = 1; r < SPLIT; r++) {
          uint32_t remote;
          float pv;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(lg_s + 4 * i), "r"(r));
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv) : "r"(remote) : "memory");
          v += pv;
        }
        lg[i] = v;
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (crank != 0) return;
  }
  __syncthreads();
  if (warp == kRtComputeWarps) return;  // the producer warp takes no part in the selection

  // selection: warp w owns tokens w*4 .. w*4+3 of the CTA
  const int rounds_sel = K;
  const int rounds_chk = (K + 1 <= E) ? K + 1 : E;
  for (int i = 0; i < kRtTokens / 8; i++) {
    const int row = warp * (kRtTokens / 8) + i;
    const int tok = tok0 + row;
    if (tok >= T) break;
    if (pos && pos[tok] < 0) {
      if (lane < K) {
        topk_i[static_cast<size_t>(tok) * K + lane] = -1;
        topk_v[static_cast<size_t>(tok) * K + lane] = 0.f;
      }
      continue;
    }
    float v[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
      const int e = lane + 32 * j;
      v[j] = (e < E) ? lg[row * EPAD + e] + __ldg(b_router + e) : -INFINITY;
    }
    float selv[GPTOSS_MAX_TOPK + 1];
    int seli[GPTOSS_MAX_TOPK + 1];

    auto select = [&](int rounds) {
      uint32_t taken = 0;
#pragma unroll
      for (int r = 0; r < GPTOSS_MAX_TOPK + 1; r++) {
        if (r < rounds) {
          float bv = -INFINITY;
          int bi = 0x7fffffff;
#pragma unroll
          for (int j = 0; j < NT; j++) {
            const int e = lane + 32 * j;
            if (!((taken >> j) & 1u) && e < E && (v[j] > bv || bi == 0x7fffffff)) {
              bv = v[j];
              bi = e;
            }
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
              bv = ov;
              bi = oi;
            }
          }
          selv[r] = bv;
          seli[r] = bi;
          if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
        }
      }
    };

    select(rounds_chk);
    if (exact_ties) {
      bool near = false;
#pragma unroll
      for (int r = 0; r < GPTOSS_MAX_TOPK; r++)
        if (r + 1 < rounds_chk && selv[r] - selv[r + 1] < kTieGuard) near = true;
      if (near) {
        float kth = selv[0];
#pragma unroll
        for (int r = 1; r < GPTOSS_MAX_TOPK; r++)
          if (r < K) kth = selv[r];
        const float thr = kth - 2.f * kTieGuard;
        const bf16 *trow = t + static_cast<size_t>(tok) * H;
#pragma unroll
        for (int j = 0; j < NT; j++) {
          uint32_t mask = __ballot_sync(0xffffffffu, (lane + 32 * j) < E && v[j] >= thr);
          while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const int e = src + 32 * j;
            const float ex = warp_exact_dot(trow, w_router + static_cast<size_t>(e) * H, H, lane);
            if (lane == src) v[j] = ex + __ldg(b_router + e);
          }
        }
        select(rounds_sel);
      }
    }
    if (logits_out) {
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int e = lane + 32 * j;
        if (e < E) logits_out[static_cast<size_t>(tok) * E + e] = v[j];
      }
    }
    // softmax over the K selected values (run.cpp:336-354: double max/sum)
    float ev[GPTOSS_MAX_TOPK];
    double sum = 0.0;
    const double mx = static_cast<double>(selv[0]);
#pragma unroll
    for (int r = 0; r < GPTOSS_MAX_TOPK; r++) {
      if (r < K) {
        ev[r] = expf(static_cast<float>(static_cast<double>(selv[r]) - mx));
        sum += static_cast<double>(ev[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < GPTOSS_MAX_TOPK; r++) {
      if (r < K && lane == r) {
        topk_i[static_cast<size_t>(tok) * K + r] = seli[r];
        topk_v[static_cast<size_t>(tok) * K + r] =
            static_cast<float>(static_cast<double>(ev[r]) / sum);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The router on the 5th-generation tensor cores, computed transposed.
//
//   logits^T[e, j] = sum_k Wr[e, k] * t[tok0 + j, k]
// The router rows are the MMA's M (128 per instruction, padded with zero rows; two
// instructions for more than 128 experts) and a CTA's tokens its N: any multiple of 16 up
// to 64, chosen by the launcher so that the token tiles fill the GPU in one wave - no
// split of the hidden dimension, no cluster, no reduction between CTAs.  The router rows
// come as one pre-tiled 16 KB piece per K chunk (weights.cu's layout, made once at load
// time) and stay in L2; the CTA's token rows are the only stream from HBM.
//
// Warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue (tcgen05.mma M=128, N=tokens,
// K=16, bf16 -> fp32 in TMEM).  Then warps 2-5 read the accumulator (a TMEM lane is an
// expert, a column a token), add the bias and transpose it into shared memory, and FOUR
// LANES PER TOKEN select: each keeps the best K+1 of its quarter of the row sorted in
// registers by a branch-free insertion, and the four lists meet in two shuffle steps (a
// warp per token with shuffles, as the mma.sync kernel does it, costs about a thousand
// dependent instructions per token and was 30 of that kernel's 45 microseconds).  Measured
// on one CTA of the 120b shape: K loop 11 us (the CTA's ingest of the router matrix from
// L2), readout 0.9, selection 1.4.
//
// Exact selection: a token whose best K+1 logits contain two neighbours closer than the
// guard lists every expert within twice the guard of its K-th value; the CTA's warps then
// recompute the listed logits the way the reference's CPU matmul does (float products
// summed in double), one (token, expert) pair per warp at a time, and the token's lanes
// select again from the corrected row.  The guard is tighter than the mma.sync kernel's:
// the tensor core's fp32 accumulation was measured within 3e-6 of the reference's double
// sums at H = 2880.
constexpr int kRxThreads = 192;
constexpr int kRxMaxTok = 64;
constexpr int kRxTileBytes = 128 * kRtRowBytes;  // one 128-row x 64-k router tile: 16 KB
constexpr int kRxPairs = 1024;                   // (token, expert) pairs a CTA recomputes
constexpr float kTieGuardTc = 3e-5f;
constexpr int kRxAccs = 2;  // accumulators the K chunks alternate between

// NT = 32-expert groups (EPAD = 32 * NT); NS = length of the sorted list a lane keeps
template <int NT, int NS>
__global__ void __launch_bounds__(kRxThreads, 1)
router_tx_kernel(const __grid_constant__ CUtensorMap tmap_t,
                 const __grid_constant__ CUtensorMap tmap_wr, const bf16 *__restrict__ t,
                 const bf16 *__restrict__ w_router, const float *__restrict__ b_router,
                 const int *__restrict__ pos, int T, int H, int E, int K, int ntok,
                 int *__restrict__ topk_i, float *__restrict__ topk_v,
                 float *__restrict__ logits_out, int exact_ties, int *status) {
  constexpr int EPAD = 32 * NT;
  constexpr int EM = EPAD > 128 ? 2 : 1;           // 128-row MMA tiles of router rows
  // logits row pitch, = 4 (mod 32): the four lanes of a row and the eight rows of a warp read
  // 32 different banks; the accumulator readout writes consecutive experts of one row
  constexpr int kPitch = EPAD + 4;
  constexpr int kTokBytes = kRxMaxTok * kRtRowBytes;            // 8 KB slot for up to 64 tokens
  constexpr int kStageBytes = EM * kRxTileBytes + kTokBytes;
  constexpr int kStages = EM == 1 ? 8 : 4;
  constexpr int kAccCols = 64;                                   // TMEM columns per router tile
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  unsigned char *after = smem + kStages * kStageBytes;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(after);
  uint64_t *empty_bar = full_bar + kStages;
  uint64_t *tfull_bar = empty_bar + kStages;
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tfull_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
  int *n_pairs = const_cast<int *>(abort_flag) + 1;
  int *n_whole = n_pairs + 1;
  int *pairs = reinterpret_cast<int *>(after + 256);  // [kRxPairs] row << 16 | expert
  int *whole = pairs + kRxPairs;                      // [kRxMaxTok] rows recomputed entirely
  // the logits of the CTA's tokens, [token][expert], over the ring once the MMAs are done
  float *lg = reinterpret_cast<float *>(smem);
  static_assert(kRxMaxTok * kPitch * 4 <= kStages * kStageBytes, "logits must fit the ring");

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = static_cast<int>(blockIdx.x) * ntok;
  const int nk = (H + kRtKC - 1) / kRtKC;

  if (tid == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    *n_pairs = 0;
    *n_whole = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_t);
    tma_prefetch_desc(&tmap_wr);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kRxAccs * EM * kAccCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  grid_dependency_wait();
  grid_launch_dependents();

  // the producer and the MMA warp walk the ring whole (every lane polls the barriers) and
  // one elected lane issues: a loop that only one lane runs makes every load and MMA several
  // times dearer to issue
  if (warp == 0) {
    {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t bytes = EM * kRxTileBytes + ntok * kRtRowBytes;
      for (int kc = 0; kc < nk; kc++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
          set_status(status, kStatusWaitTimeoutProducer);
          *abort_flag = 1;
          break;
        }
        unsigned char *dst = smem + stage * kStageBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(&full_bar[stage], bytes);
          tma_load_2d(dst + EM * kRxTileBytes, &tmap_t, &full_bar[stage], kc * kRtKC, tok0);
#pragma unroll
          for (int m = 0; m < EM; m++)
            tma_load_2d(dst + m * kRxTileBytes, &tmap_wr, &full_bar[stage], 0, (m * nk + kc) * 32);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    {
      const uint32_t idesc = umma_idesc_bf16(128, ntok);
      int stage = 0;
      uint32_t phase = 0;
      for (int kc = 0; kc < nk; kc++) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
          set_status(status, kStatusWaitTimeoutMma);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * kStageBytes);
        const uint64_t db = umma_smem_desc_sw128(sa + EM * kRxTileBytes);
        // consecutive MMAs into one accumulator wait for each other; with so few columns
        // that wait, not the tensor pipe, sets the pace: the chunks alternate between
        // kRxAccs accumulators, added up when the logits are read
        const int a = kc % kRxAccs;
        if (elect_one()) {
#pragma unroll
          for (int m = 0; m < EM; m++) {
            const uint64_t da = umma_smem_desc_sw128(sa + m * kRxTileBytes);
#pragma unroll
            for (int k = 0; k < kRtKC / 16; k++)
              umma_bf16(tmem_base + (a * EM + m) * kAccCols, da + 2 * k, db + 2 * k, idesc,
                        (kc >= kRxAccs || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (elect_one()) umma_commit(tfull_bar);
    }
  } else {
    // accumulator -> logits [token][expert] in shared memory, bias added
    if (!mbar_wait(tfull_bar, 0, abort_flag)) {
      set_status(status, kStatusWaitTimeoutEpilogue);
      *abort_flag = 1;
    }
    __syncwarp();
    tc_fence_after();
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) are this warp's
#pragma unroll
    for (int m = 0; m < EM; m++) {
      const int e = m * 128 + q * 32 + lane;
      const float bias = e < E ? __ldg(b_router + e) : 0.f;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + m * kAccCols;
      const int accs = nk < kRxAccs ? nk : kRxAccs;  // accumulators that were written at all
      for (int c0 = 0; c0 < ntok; c0 += 16) {
        uint32_t r[16];
        float sum[16];
#pragma unroll
        for (int j = 0; j < 16; j++) sum[j] = bias;
        for (int a = 0; a < accs; a++) {
          tmem_ld16(taddr + a * EM * kAccCols + c0, r);
          tmem_ld_wait16(r);
#pragma unroll
          for (int j = 0; j < 16; j++) sum[j] += __uint_as_float(r[j]);
        }
        if (e < EPAD) {
#pragma unroll
          for (int j = 0; j < 16; j++) lg[(c0 + j) * kPitch + e] = sum[j];
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();

  // ---- selection: four lanes per token row, kRowsPerPass rows at a time.  Lane s of a row
  // keeps the best NS of the logits e = s, s + 4, ... (sorted: value descending, lower index
  // first on equal values) by branch-free insertion, then the four lists meet in two
  // exchange steps, after which every lane of the row holds the row's best NS.
  constexpr int kG = 4;
  constexpr int kRowsPerPass = kRxThreads / kG;
  constexpr int kPasses = (kRxMaxTok + kRowsPerPass - 1) / kRowsPerPass;
  const int sub = tid & (kG - 1);
  const int rounds_chk = (K + 1 <= E) ? K + 1 : E;
  float bv[NS];
  int bi[NS];
  // v enters the sorted list where it belongs; all the comparisons are independent of each
  // other and every slot is rewritten from the old list, so an insertion is three
  // instructions deep (the list is sorted: once v beats a slot it beats the ones after it).
  // The comparisons are combined with | and &, not || and &&: the short-circuit forms compile
  // to a branch per slot, and the selection then takes 7 us instead of 1.4.
  auto insert = [&](float v, int i) {
    bool up[NS];
#pragma unroll
    for (int p = 0; p < NS; p++) up[p] = (v > bv[p]) | ((v == bv[p]) & (i < bi[p]));
#pragma unroll
    for (int p = NS - 1; p > 0; p--) {
      bv[p] = up[p] ? (up[p - 1] ? bv[p - 1] : v) : bv[p];
      bi[p] = up[p] ? (up[p - 1] ? bi[p - 1] : i) : bi[p];
    }
    bv[0] = up[0] ? v : bv[0];
    bi[0] = up[0] ? i : bi[0];
  };
  auto scan_row = [&](const float *my) {
#pragma unroll
    for (int p = 0; p < NS; p++) {
      bv[p] = -INFINITY;
      bi[p] = 0x7fffffff;
    }
    // eight loads in flight before the first compare
    for (int j0 = 0; j0 * kG < E; j0 += 8) {
      float v8[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int e = sub + kG * (j0 + u);
        v8[u] = e < E ? my[e] : -INFINITY;
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int e = sub + kG * (j0 + u);
        insert(v8[u], e < E ? e : 0x7fffffff);  // (-inf, 0x7fffffff) never enters the list
      }
    }
#pragma unroll
    for (int m = 1; m < kG; m <<= 1) {
      float ov[NS];
      int oi[NS];
#pragma unroll
      for (int p = 0; p < NS; p++) {
        ov[p] = __shfl_xor_sync(0xffffffffu, bv[p], m);
        oi[p] = __shfl_xor_sync(0xffffffffu, bi[p], m);
      }
#pragma unroll
      for (int p = 0; p < NS; p++) insert(ov[p], oi[p]);
    }
  };
  // softmax over the K selected values (run.cpp:336-354) and the token's outputs
  auto write_out = [&](int tok, const float *my) {
    if (sub == 0) {
      float ev[NS];
      float sum = 0.f;
#pragma unroll
      for (int r = 0; r < NS; r++) {
        if (r < K) {
          ev[r] = expf(bv[r] - bv[0]);
          sum += ev[r];
        }
      }
#pragma unroll
      for (int r = 0; r < NS; r++) {
        if (r < K) {
          topk_i[static_cast<size_t>(tok) * K + r] = bi[r];
          topk_v[static_cast<size_t>(tok) * K + r] = ev[r] / sum;
        }
      }
    }
    if (logits_out)
      for (int e = sub; e < E; e += kG) logits_out[static_cast<size_t>(tok) * E + e] = my[e];
  };

  bool flagged[kPasses];
#pragma unroll
  for (int pass = 0; pass < kPasses; pass++) {
    flagged[pass] = false;
    if (pass * kRowsPerPass >= ntok) continue;  // (the same for the whole CTA)
    const int row = pass * kRowsPerPass + (tid >> 2);
    const int tok = tok0 + row;
    const bool mine = row < ntok && tok < T;
    const bool live = mine && !(pos && pos[tok] < 0);
    // rows past the tile are scanned like the others (the lanes stay together for the
    // exchanges) but from a row that exists, and nothing of theirs is kept
    const float *my = lg + (row < kRxMaxTok ? row : kRxMaxTok - 1) * kPitch;
    scan_row(my);
    bool flag = false;
    if (live && exact_ties) {
#pragma unroll
      for (int r = 0; r + 1 < NS; r++)
        if (r + 1 < rounds_chk && bv[r] - bv[r + 1] < kTieGuardTc) flag = true;
    }
    // list the contenders of a flagged row: everything within twice the guard of the K-th
    // value
    float kth = bv[0];
#pragma unroll
    for (int r = 1; r < NS; r++)
      if (r < K) kth = bv[r];
    const float thr = kth - 2.f * kTieGuardTc;
    bool full = false;
    if (flag && bv[NS - 1] < thr) {
      // the usual case: the band ends inside the kept list, which then names every contender
      // (walking the row again for them cost a CTA with a near tie 4.5 us)
      if (sub == 0) {
#pragma unroll
        for (int p = 0; p < NS; p++) {
          if (bv[p] >= thr) {
            const int at = atomicAdd(n_pairs, 1);
            if (at < kRxPairs)
              pairs[at] = (row << 16) | bi[p];
            else
              full = true;
          }
        }
      }
    } else if (flag) {
      // even the last kept value is inside the band: there may be more beyond the list
      for (int e = sub; e < E && !full; e += kG) {
        if (my[e] >= thr) {
          const int at = atomicAdd(n_pairs, 1);
          if (at < kRxPairs)
            pairs[at] = (row << 16) | e;
          else
            full = true;
        }
      }
    }
    // the list is full (hundreds of near ties in one tile): the row is recomputed whole
#pragma unroll
    for (int m = 1; m < kG; m <<= 1) full |= __shfl_xor_sync(0xffffffffu, full ? 1 : 0, m) != 0;
    if (full && sub == 0) whole[atomicAdd(n_whole, 1)] = row;
    flagged[pass] = flag;
    if (live && !flag) {
      write_out(tok, my);
    } else if (mine && !live && sub == 0) {
      for (int r = 0; r < K; r++) {
        topk_i[static_cast<size_t>(tok) * K + r] = -1;
        topk_v[static_cast<size_t>(tok) * K + r] = 0.f;
      }
    }
  }
  __syncthreads();

  // ---- near ties: the exact logits, one (token, expert) pair per warp at a time
  const int np = *n_pairs < kRxPairs ? *n_pairs : kRxPairs;
  const int nw = *n_whole;
  if (np + nw > 0) {
    for (int p = warp; p < np; p += kRxThreads / 32) {
      const int row = pairs[p] >> 16, e = pairs[p] & 0xffff;
      const float ex = warp_exact_dot(t + static_cast<size_t>(tok0 + row) * H,
                                      w_router + static_cast<size_t>(e) * H, H, lane);
      if (lane == 0) lg[row * kPitch + e] = ex + __ldg(b_router + e);
    }
    for (int i = 0; i < nw; i++) {
      const int row = whole[i];
      for (int e = warp; e < E; e += kRxThreads / 32) {
        const float ex = warp_exact_dot(t + static_cast<size_t>(tok0 + row) * H,
                                        w_router + static_cast<size_t>(e) * H, H, lane);
        if (lane == 0) lg[row * kPitch + e] = ex + __ldg(b_router + e);
      }
    }
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < kPasses; pass++) {
      if (pass * kRowsPerPass >= ntok) continue;
      const int row = pass * kRowsPerPass + (tid >> 2);
      const float *my = lg + (row < kRxMaxTok ? row : kRxMaxTok - 1) * kPitch;
      // a warp rescans when one of its eight rows was flagged
      if (__any_sync(0xffffffffu, flagged[pass])) {
        scan_row(my);
        if (flagged[pass]) write_out(tok0 + row, my);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 2000000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kRxAccs * EM * kAccCols);
  }
}

template <int NT, int SPLIT>
static cudaError_t launch_router_split(const CUtensorMap &tmap_t, const CUtensorMap &tmap_w,
                                       const bf16 *t, const bf16 *w_router, const float *b_router,
                                       const int *pos, int T, int H, int E, int K, int *topk_i,
                                       float *topk_v, float *logits_opt, int exact_ties,
                                       int *status, cudaStream_t stream) {
  constexpr int EPAD = 32 * NT;
  constexpr int kRtStages = RtStages<NT>::value;
  // alignment slack + ring + barriers + logits
  const size_t smem = 1024 + static_cast<size_t>(kRtStages) * (kRtTokens + EPAD) * kRtRowBytes +
                      256 + kRtTokens * EPAD * 4;
  static_assert(2 * RtStages<NT>::value * 8 + 4 <= 256, "barrier area");
  cudaError_t e = cudaFuncSetAttribute(router_topk_kernel<NT, SPLIT>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int groups = (T + kRtTokens - 1) / kRtTokens;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(groups * SPLIT));
  cfg.blockDim = dim3(kRtThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SPLIT;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = SPLIT > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, router_topk_kernel<NT, SPLIT>, tmap_t, tmap_w, t, w_router,
                            b_router, pos, T, H, E, K, topk_i, topk_v, logits_opt, exact_ties,
                            status);
}

// The CUDA-core-MMA router (router_impl 1): kept selectable beside the tcgen05 one.
template <int NT>
static cudaError_t launch_router_nt(gptoss_moe *h, const bf16 *t, const bf16 *w_router,
                                    const float *b_router, const int *pos, int T, int *topk_i,
                                    float *topk_v, float *logits_opt, cudaStream_t stream) {
  constexpr int EPAD = 32 * NT;
  const int H = h->H, E = h->E, K = h->K;
  // tiles of one 64-element K chunk: 32 token rows, EPAD expert rows (rows that do not
  // exist read as zeros)
  CUtensorMap tmap_t, tmap_w;
  std::string err;
  if (make_tmap_2d_bf16(&tmap_t, t, H, T, kRtKC, kRtTokens, &err) ||
      make_tmap_2d_bf16(&tmap_w, w_router, H, E, kRtKC, EPAD, &err))
    return cudaErrorInvalidValue;
  // few token groups (decode batches): four CTAs per group split the K loop
  const int groups = (T + kRtTokens - 1) / kRtTokens;
  if (groups * 4 <= h->num_sms && H >= 16 * kRtKC)
    return launch_router_split<NT, 4>(tmap_t, tmap_w, t, w_router, b_router, pos, T, H, E, K,
                                      topk_i, topk_v, logits_opt, h->opt_exact_ties, h->status,
                                      stream);
  return launch_router_split<NT, 1>(tmap_t, tmap_w, t, w_router, b_router, pos, T, H, E, K,
                                    topk_i, topk_v, logits_opt, h->opt_exact_ties, h->status, stream);
}

template <int NT, int NS>
static cudaError_t launch_router_tx(gptoss_moe *h, LayerWeights &lw, const bf16 *t, const int *pos,
                                    int T, int *topk_i, float *topk_v, float *logits_opt,
                                    cudaStream_t stream) {
  constexpr int EPAD = 32 * NT;
  constexpr int EM = EPAD > 128 ? 2 : 1;
  constexpr int kStages = EM == 1 ? 8 : 4;
  const int H = h->H, E = h->E, K = h->K;
  auto kernel = router_tx_kernel<NT, NS>;
  const size_t smem = 1024 + static_cast<size_t>(kStages) * (EM * kRxTileBytes + kRxMaxTok * kRtRowBytes) +
                      256 + (kRxPairs + kRxMaxTok) * sizeof(int);
  static_assert((2 * kStages + 1) * 8 + 16 <= 256, "barrier area");
  // tokens per CTA: the token tiles fill the GPU in one wave
  int ntok = (((T + h->num_sms - 1) / h->num_sms) + 15) & ~15;
  if (ntok < 16) ntok = 16;
  if (ntok > kRxMaxTok) ntok = kRxMaxTok;
  std::string err;
  // the token map is kept while the caller hands the same buffer and batch size
  if (h->router_t_ptr != t || h->router_t_rows != T || h->router_t_box != ntok) {
    if (make_tmap_2d_bf16(&h->tmap_router_t, t, H, T, kRtKC, ntok, &err))
      return cudaErrorInvalidValue;
    h->router_t_ptr = t;
    h->router_t_rows = T;
    h->router_t_box = ntok;
  }
  // per device, cheap: set on every launch so every GPU a process drives has it
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>((T + ntok - 1) / ntok));
  cfg.blockDim = dim3(kRxThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = h->opt_dependent_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, h->tmap_router_t, lw.tmap_router_tiled, t,
                            static_cast<const bf16 *>(lw.w_router),
                            static_cast<const float *>(lw.b_router), pos, T, H, E, K, ntok, topk_i,
                            topk_v, logits_opt, h->opt_exact_ties, h->status);
}

int build_router_tiles(gptoss_moe *h, LayerWeights &lw) {
  const size_t n = tiled_weight_elems(h->E, h->H, 1);
  auto fail = [&](const std::string &what) {
    h->err = what;
    return GPTOSS_E_CUDA;
  };
  cudaError_t e;
  if (!lw.router_tiled &&
      (e = cudaMalloc(reinterpret_cast<void **>(&lw.router_tiled), n * sizeof(bf16))) != cudaSuccess)
    return fail(std::string("cudaMalloc(router tiles): ") + cudaGetErrorString(e));
  if ((e = launch_retile_weights(lw.router_tiled, lw.w_router, h->E, h->H, 1, nullptr,
                                 &h->launches)) != cudaSuccess ||
      (e = cudaStreamSynchronize(nullptr)) != cudaSuccess)
    return fail(std::string("router tiles: ") + cudaGetErrorString(e));
  std::string err;
  if (make_tmap_tiles_bf16(&lw.tmap_router_tiled, lw.router_tiled, n / (128 * kTileK), &err))
    return fail(err);
  return GPTOSS_OK;
}

cudaError_t launch_router_topk(gptoss_moe *h, int layer, const bf16 *t, const int *pos, int T,
                               float *logits_opt, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  h->launches++;
  LayerWeights &lw = h->layers[layer];
  const int E = h->E;
  if (E > 256) return cudaErrorInvalidValue;
  if (h->opt_router_impl == 1) {
    const bf16 *w = lw.w_router;
    const float *b = lw.b_router;
    if (E <= 32) return launch_router_nt<1>(h, t, w, b, pos, T, h->topk_i, h->topk_v, logits_opt, stream);
    if (E <= 64) return launch_router_nt<2>(h, t, w, b, pos, T, h->topk_i, h->topk_v, logits_opt, stream);
    if (E <= 128) return launch_router_nt<4>(h, t, w, b, pos, T, h->topk_i, h->topk_v, logits_opt, stream);
    return launch_router_nt<8>(h, t, w, b, pos, T, h->topk_i, h->topk_v, logits_opt, stream);
  }
#define GPTOSS_ROUTER_CASE(NTV)                                                                  \
  if (E <= 32 * NTV)                                                                             \
    return h->K <= 4 ? launch_router_tx<NTV, 5>(h, lw, t, pos, T, h->topk_i, h->topk_v,          \
                                                logits_opt, stream)                              \
                     : launch_router_tx<NTV, 9>(h, lw, t, pos, T, h->topk_i, h->topk_v,          \
                                                logits_opt, stream);
  GPTOSS_ROUTER_CASE(1)
  GPTOSS_ROUTER_CASE(2)
  GPTOSS_ROUTER_CASE(4)
  GPTOSS_ROUTER_CASE(8)
#undef GPTOSS_ROUTER_CASE
  return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------ RMSNorm
// out = w * x * rsqrt(mean(x^2) + 1e-5); one warp per token, 16-byte accesses.
// Replaces rmsnorm_batch_kernel (getp-csrc/utility/utility.cpp:194-271).
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(bf16 *__restrict__ out, const bf16 *__restrict__ x,
                    const float *__restrict__ w, const int *__restrict__ pos, int T, int H) {
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= T) return;
  if (pos && pos[tok] < 0) return;
  const uint4 *x4 = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(tok) * H);
  uint4 *o4 = reinterpret_cast<uint4 *>(out + static_cast<size_t>(tok) * H);
  const int n4 = H >> 3;
  float ss = 0.f;
  for (int p = lane; p < n4; p += 32) {
    const uint4 v = x4[p];
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float a = bf16_lo(u[i]), b = bf16_hi(u[i]);
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + 1e-5f);
  for (int p = lane; p < n4; p += 32) {
    const uint4 v = x4[p];
    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * p);
    const float4 w1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * p + 1);
    uint4 o;
    o.x = pack_bf16(w0.x * (inv * bf16_lo(v.x)), w0.y * (inv * bf16_hi(v.x)));
    o.y = pack_bf16(w0.z * (inv * bf16_lo(v.y)), w0.w * (inv * bf16_hi(v.y)));
    o.z = pack_bf16(w1.x * (inv * bf16_lo(v.z)), w1.y * (inv * bf16_hi(v.z)));
    o.w = pack_bf16(w1.z * (inv * bf16_lo(v.w)), w1.w * (inv * bf16_hi(v.w)));
    o4[p] = o;
  }
}

cudaError_t launch_rmsnorm(bf16 *out, const bf16 *x, const float *w, const int *pos, int T, int H,
                           cudaStream_t stream, long long *launches) {
  if (T <= 0) return cudaSuccess;
  if (launches) ++*launches;
  const int warps = 8;
  rmsnorm_rows_kernel<<<(T + warps - 1) / warps, warps * 32, 0, stream>>>(out, x, w, pos, T, H);
  return cudaGetLastError();
}

}  // namespace gptoss
