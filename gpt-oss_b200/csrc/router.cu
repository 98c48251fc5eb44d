// Router stage: logits = t . Wr^T + b, top-K by value (lowest index first on
// equal values), softmax over the K selected logits.  One kernel; the logits
// never go to HBM unless the debug tap asks for them.
//
// Replaces matmul_router_kernel (getp-csrc/matmul/matmul.cpp:945-1019) and
// fused_topk_softmax_batch_kernel (getp-csrc/utility/utility.cpp:274-365) of the
// reference.  Bound by HBM: the only large stream is t [T,H] bf16, read once.
//
// Layout: a CTA owns 32 consecutive tokens.  8 warps = 2 token groups of 16 x 4
// expert slices; bf16 tensor-core MMAs (m16n8k16, fp32 accumulate) over K chunks
// of 64.  A ninth warp is the producer: one thread issues two TMA tile loads per
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
  // Loads of up to 4 pieces per lane are issued together (their latency overlaps)
  // and four independent accumulators keep the fp64 add chains short.  The order
  // of the fp64 additions differs from the reference's left-to-right sum by
  // rounding errors ~1e-16 relative, which the final rounding to float hides.
  double acc0 = 0.0, acc1 = 0.0, acc2 = 0.0, acc3 = 0.0;
  const uint4 *a4 = reinterpret_cast<const uint4 *>(a);
  const uint4 *b4 = reinterpret_cast<const uint4 *>(b);
  const int n4 = H >> 3;
  for (int p0 = lane; p0 < n4; p0 += 128) {
    uint4 av[4], bv[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int p = p0 + u * 32;
      av[u] = p < n4 ? __ldg(a4 + p) : make_uint4(0, 0, 0, 0);
      bv[u] = p < n4 ? __ldg(b4 + p) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kc = kc_lo; kc < kc_hi; kc++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
          set_status(status, kStatusWaitTimeoutProducer);
          *abort_flag = 1;
          break;
        }
        unsigned char *dst = smem + stage * kStageBytes;
        mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
        tma_load_2d(dst, &tmap_t, &full_bar[stage], kc * kRtKC, tok0);
        tma_load_2d(dst + kTokBytes, &tmap_w, &full_bar[stage], kc * kRtKC, 0);
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

template <int NT>
static cudaError_t launch_router_nt(const bf16 *t, const bf16 *w_router, const float *b_router,
                                    const int *pos, int T, int H, int E, int K, int *topk_i,
                                    float *topk_v, float *logits_opt, int exact_ties, int *status,
                                    cudaStream_t stream) {
  constexpr int EPAD = 32 * NT;
  // tiles of one 64-element K chunk: 32 token rows, EPAD expert rows (rows that do not
  // exist read as zeros)
  CUtensorMap tmap_t, tmap_w;
  std::string err;
  if (make_tmap_2d_bf16(&tmap_t, t, H, T, kRtKC, kRtTokens, &err) ||
      make_tmap_2d_bf16(&tmap_w, w_router, H, E, kRtKC, EPAD, &err))
    return cudaErrorInvalidValue;
  // few token groups (decode batches): four CTAs per group split the K loop
  static int num_sms = 0;
  if (!num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int groups = (T + kRtTokens - 1) / kRtTokens;
  if (groups * 4 <= num_sms && H >= 16 * kRtKC)
    return launch_router_split<NT, 4>(tmap_t, tmap_w, t, w_router, b_router, pos, T, H, E, K,
                                      topk_i, topk_v, logits_opt, exact_ties, status, stream);
  return launch_router_split<NT, 1>(tmap_t, tmap_w, t, w_router, b_router, pos, T, H, E, K,
                                    topk_i, topk_v, logits_opt, exact_ties, status, stream);
}

cudaError_t launch_router_topk(const bf16 *t, const bf16 *w_router, const float *b_router,
                               const int *pos, int T, int H, int E, int K, int *topk_i,
                               float *topk_v, float *logits_opt, int exact_ties, int *status,
                               cudaStream_t stream, long long *launches) {
  if (T <= 0) return cudaSuccess;
  if (launches) ++*launches;
  if (E <= 32)
    return launch_router_nt<1>(t, w_router, b_router, pos, T, H, E, K, topk_i, topk_v, logits_opt,
                               exact_ties, status, stream);
  if (E <= 64)
    return launch_router_nt<2>(t, w_router, b_router, pos, T, H, E, K, topk_i, topk_v, logits_opt,
                               exact_ties, status, stream);
  if (E <= 128)
    return launch_router_nt<4>(t, w_router, b_router, pos, T, H, E, K, topk_i, topk_v, logits_opt,
                               exact_ties, status, stream);
  if (E <= 256)
    return launch_router_nt<8>(t, w_router, b_router, pos, T, H, E, K, topk_i, topk_v, logits_opt,
                               exact_ties, status, stream);
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
