// Batched greedy decode step around the MoE block: see include/gptoss_decode_b200.h.
//
// What runs per step for a batch of B rows (row i = one sequence with its own
// KV-cache slot), following forward() of the reference (run.cpp:536-766) row by
// row:
//   embed_rows_kernel                    x = E[token]                      (run.cpp:550-552)
//   per layer:
//     rmsnorm_rows_kernel                t = rmsnorm(x) * w                (run.cpp:556)
//     grouped_gemm_pair_kernel<down>     qkv = t Wqkv^T + bias (one group) (run.cpp:568-574)
//     qkv_rope_cache_kernel              rotate q and k, append k,v        (run.cpp:575-596)
//     attn_decode_kernel                 softmax(qK/sqrt(D) | sink) V      (run.cpp:601-647)
//     grouped_gemm_pair_kernel<down> + bias_residual_kernel
//                                        x += o Wo^T + b_o                 (run.cpp:649-661)
//     rmsnorm_rows_kernel, gptoss_moe_forward                              (run.cpp:664-750)
//   rmsnorm_rows_kernel, grouped_gemm_pair_kernel<f32>
//                                        logits = rmsnorm(x) Wout^T        (run.cpp:752-757)
//   argmax_rows_kernel                   next = argmax (lowest index on ties)
// Rows with pos < 0 are skipped by every kernel (the GEMMs compute them and the
// results are ignored).
#include <cublas_v2.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/gptoss_decode_b200.h"
#include "common.cuh"
#include "engine.h"
#include "gemm_epilogue.cuh"

namespace gptoss {

struct CublasApi {
  void *lib = nullptr;
  cublasStatus_t (*Create)(cublasHandle_t *) = nullptr;
  cublasStatus_t (*Destroy)(cublasHandle_t) = nullptr;
  cublasStatus_t (*SetStream)(cublasHandle_t, cudaStream_t) = nullptr;
  cublasStatus_t (*GemmEx)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int,
                           const void *, const void *, cudaDataType, int, const void *,
                           cudaDataType, int, const void *, void *, cudaDataType, int,
                           cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
};
static CublasApi g_blas;

static bool load_cublas(std::string *err) {
  if (g_blas.lib) return true;
  void *lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libcublas.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("/usr/local/cuda/lib64/libcublas.so.12", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) {
    *err = std::string("cannot load cuBLAS: ") + dlerror();
    return false;
  }
#define SYM(field, name)                                                \
  *reinterpret_cast<void **>(&g_blas.field) = dlsym(lib, name);         \
  if (!g_blas.field) {                                                  \
    *err = std::string("cuBLAS symbol missing: ") + name;               \
    return false;                                                       \
  }
  SYM(Create, "cublasCreate_v2")
  SYM(Destroy, "cublasDestroy_v2")
  SYM(SetStream, "cublasSetStream_v2")
  SYM(GemmEx, "cublasGemmEx")
#undef SYM
  g_blas.lib = lib;
  return true;
}

// x[i, :] = table[token[i], :]
__global__ void __launch_bounds__(256)
embed_rows_kernel(bf16 *__restrict__ x, const bf16 *__restrict__ table,
                  const int *__restrict__ tokens, const int *__restrict__ pos, int B, int H,
                  int V, int *status) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= B || pos[row] < 0) return;
  const int tok = tokens[row];
  if (tok < 0 || tok >= V) {
    set_status(status, kStatusBadIndex);
    return;
  }
  const uint4 *s4 = reinterpret_cast<const uint4 *>(table + static_cast<size_t>(tok) * H);
  uint4 *d4 = reinterpret_cast<uint4 *>(x + static_cast<size_t>(row) * H);
  for (int p = lane; p < (H >> 3); p += 32) d4[p] = __ldg(s4 + p);
}

// qkv [B, (Hq + 2 Hkv) D] fp32 (rows q | k | v) + bias; q and k rotated
// (apply_rotary_emb, run.cpp:511-533: pairs (i, i + D/2), cos/sin of pos * inv_freq[i]
// times the YaRN concentration); q stays fp32, k and v go to the row's cache slot at
// position pos as bf16.  One CTA per row.
// QKV_BF: the projection comes from this library's GEMM as bf16 with the bias already
// added; otherwise fp32 from cuBLAS and the bias is added here.
template <bool QKV_BF>
__global__ void __launch_bounds__(256)
qkv_rope_cache_kernel(const void *__restrict__ qkv_any, const float *__restrict__ bias,
                      const int *__restrict__ pos, const float *__restrict__ inv_freq,
                      float concentration, float *__restrict__ q_out, bf16 *__restrict__ k_cache,
                      bf16 *__restrict__ v_cache, int B, int Hq, int Hkv, int D, int S) {
  const int row = blockIdx.x;
  const int p = pos[row];
  if (p < 0) return;
  const int half = D >> 1;
  const int dq = Hq * D, dkv = Hkv * D, ld = dq + 2 * dkv;
  auto val = [&](int i) -> float {
    if (QKV_BF)
      return __bfloat162float(static_cast<const bf16 *>(qkv_any)[static_cast<size_t>(row) * ld + i]);
    return static_cast<const float *>(qkv_any)[static_cast<size_t>(row) * ld + i] + bias[i];
  };
  // rotated pairs of q and k
  for (int i = threadIdx.x; i < (Hq + Hkv) * half; i += blockDim.x) {
    const int head = i / half, j = i - head * half;
    const int base = head * D;  // q heads first, then k heads: contiguous in qkv
    const float x1 = val(base + j);
    const float x2 = val(base + half + j);
    const float ang = static_cast<float>(p) * inv_freq[j];
    const float c = cosf(ang) * concentration, s = sinf(ang) * concentration;
    const float o1 = x1 * c - x2 * s, o2 = x2 * c + x1 * s;
    if (head < Hq) {
      q_out[static_cast<size_t>(row) * dq + base + j] = o1;
      q_out[static_cast<size_t>(row) * dq + base + half + j] = o2;
    } else {
      const int kb = base - dq;
      bf16 *dst = k_cache + (static_cast<size_t>(row) * S + p) * dkv;
      dst[kb + j] = __float2bfloat16_rn(o1);
      dst[kb + half + j] = __float2bfloat16_rn(o2);
    }
  }
  for (int i = threadIdx.x; i < dkv; i += blockDim.x) {
    bf16 *dst = v_cache + (static_cast<size_t>(row) * S + p) * dkv;
    dst[i] = __float2bfloat16_rn(val(dq + dkv + i));
  }
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, "
      "{%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Attention of one decode step over the KV cache, on tensor cores.
//
// One CTA per (row, KV head): the up to 8 query heads that share the KV head are the rows
// of an m16n8k16 tile (rows 8-15 stay zero), so K and V are read once for all of them.
// The CTA's 4 warps take every fourth block of 16 cache positions; per block a warp
// computes S = Q K^T (positions as the MMA's N), keeps a running maximum and sum per head
// (online softmax, fp32), and accumulates O += P V with P rounded to bf16 (as V is); the
// four partial results and the head's sink logit - which takes probability mass but has
// no value row - are merged through shared memory (run.cpp:601-647; the sliding-window
// mask of even layers, run.cpp:176-183, 619-621, is the lower bound t0 = pos - window + 1).
// Cache rows past pos are read as zeros.  Output bf16 [B, Hq D].
constexpr int kAttnWarps = 4;

template <int D>
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_decode_kernel(const float *__restrict__ q, const bf16 *__restrict__ k_cache,
                   const bf16 *__restrict__ v_cache, const float *__restrict__ sinks,
                   const int *__restrict__ pos, bf16 *__restrict__ out, int B, int Hq, int Hkv,
                   int S, int window) {
  constexpr int RS = D * 2 + 16;        // padded row pitch of a staged tile (bytes)
  constexpr int kChunks = 16 * (D / 8);  // 16-byte chunks of one 16-position tile
  constexpr int kPerLane = kChunks / 32;
  __shared__ __align__(16) unsigned char tiles[kAttnWarps][2][16 * RS];  // [warp][K | V]
  __shared__ float sm_m[kAttnWarps][8], sm_l[kAttnWarps][8];
  static_assert(8 * D * 4 <= 2 * 16 * RS, "a warp's partial output reuses its own tiles");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x / Hkv, kvh = blockIdx.x - row * Hkv;
  const int p = pos[row];
  if (p < 0) return;  // the whole CTA leaves
  const int group = Hq / Hkv;
  const int dkv = Hkv * D;
  const int t0 = window > 0 ? max(0, p - window + 1) : 0;
  const int n_blocks = (p - t0 + 16) / 16;
  const int hr = lane >> 2, qd = lane & 3;  // head row of this thread's fragment, quad lane

  // Q fragments (A operand): rows = heads of the group, pre-scaled by 1/sqrt(D)
  uint32_t qa[D / 16][4];
  {
    const float scale = 1.0f / sqrtf(static_cast<float>(D));
    const float *qrow = q + (static_cast<size_t>(row) * Hq + kvh * group + hr) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
      float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
      if (hr < group) {
        lo = *reinterpret_cast<const float2 *>(qrow + kk * 16 + 2 * qd);
        hi = *reinterpret_cast<const float2 *>(qrow + kk * 16 + 8 + 2 * qd);
      }
      qa[kk][0] = pack_bf16(lo.x * scale, lo.y * scale);
      qa[kk][1] = 0u;  // rows 8-15
      qa[kk][2] = pack_bf16(hi.x * scale, hi.y * scale);
      qa[kk][3] = 0u;
    }
  }
  float m = -INFINITY, l = 0.f;
  float o[D / 8][2];
#pragma unroll
  for (int n = 0; n < D / 8; n++) o[n][0] = o[n][1] = 0.f;

  const size_t base = static_cast<size_t>(row) * S * dkv + kvh * D;
  unsigned char *tk = tiles[warp][0], *tv = tiles[warp][1];
  const uint32_t tk_s = smem_u32(tk), tv_s = smem_u32(tv);
  uint4 rk[kPerLane], rv[kPerLane];
  auto fetch = [&](int blk) {
    const int tb = t0 + blk * 16;
#pragma unroll
    for (int u = 0; u < kPerLane; u++) {
      const int c = lane + 32 * u, r = c / (D / 8), ch = c - r * (D / 8);
      rk[u] = rv[u] = make_uint4(0, 0, 0, 0);
      if (tb + r <= p) {
        const size_t off = base + static_cast<size_t>(tb + r) * dkv + 8 * ch;
        rk[u] = __ldg(reinterpret_cast<const uint4 *>(k_cache + off));
        rv[u] = __ldg(reinterpret_cast<const uint4 *>(v_cache + off));
      }
    }
  };
  if (warp < n_blocks) fetch(warp);
  for (int blk = warp; blk < n_blocks; blk += kAttnWarps) {
    __syncwarp();  // the previous block's ldmatrix reads are done
#pragma unroll
    for (int u = 0; u < kPerLane; u++) {
      const int c = lane + 32 * u, r = c / (D / 8), ch = c - r * (D / 8);
      *reinterpret_cast<uint4 *>(tk + r * RS + ch * 16) = rk[u];
      *reinterpret_cast<uint4 *>(tv + r * RS + ch * 16) = rv[u];
    }
    __syncwarp();
    if (blk + kAttnWarps < n_blocks) fetch(blk + kAttnWarps);  // in flight during the math

    // S = Q K^T for 16 positions: two n-tiles of 8
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < D / 16; kk++) {
      uint32_t b[4];
      const int prow = (lane >> 4) * 8 + (lane & 7), dch = kk * 2 + ((lane >> 3) & 1);
      ldsm_x4(tk_s + prow * RS + dch * 16, b);
      mma_16816(s0, qa[kk], b[0], b[1]);
      mma_16816(s1, qa[kk], b[2], b[3]);
    }
    // this thread's four positions of head row hr: block offsets 2qd, 2qd+1, 8+2qd, 9+2qd
    const int tb = t0 + blk * 16;
    float sv[4] = {s0[0], s0[1], s1[0], s1[1]};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int t = tb + (i >> 1) * 8 + 2 * qd + (i & 1);
      if (t > p) sv[i] = -INFINITY;
    }
    float bm = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
    const float m_new = fmaxf(m, bm);  // finite: the first position of a block is <= pos
    const float corr = __expf(m - m_new);
    float pr[4];
#pragma unroll
    for (int i = 0; i < 4; i++) pr[i] = __expf(sv[i] - m_new);
    l = l * corr + (pr[0] + pr[1]) + (pr[2] + pr[3]);
    m = m_new;
#pragma unroll
    for (int n = 0; n < D / 8; n++) {
      o[n][0] *= corr;
      o[n][1] *= corr;
    }
    // O += P V: P (16 heads x 16 positions) from the score fragments, V transposed on load
    uint32_t pa[4] = {pack_bf16(pr[0], pr[1]), 0u, pack_bf16(pr[2], pr[3]), 0u};
#pragma unroll
    for (int n = 0; n < D / 8; n += 2) {
      uint32_t b[4];
      const int prow = ((lane >> 3) & 1) * 8 + (lane & 7), dch = n + (lane >> 4);
      ldsm_x4_trans(tv_s + prow * RS + dch * 16, b);
      float acc0[4] = {o[n][0], o[n][1], 0.f, 0.f}, acc1[4] = {o[n + 1][0], o[n + 1][1], 0.f, 0.f};
      mma_16816(acc0, pa, b[0], b[1]);
      mma_16816(acc1, pa, b[2], b[3]);
      o[n][0] = acc0[0]; o[n][1] = acc0[1];
      o[n + 1][0] = acc1[0]; o[n + 1][1] = acc1[1];
    }
  }
  // the quad's partial sums of l -> one per head
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (qd == 0) {
    sm_m[warp][hr] = m;
    sm_l[warp][hr] = l;
  }
  // the warp's partial output [8 heads][D] goes where its K / V tiles were
  __syncwarp();
  {
    float *my_o = reinterpret_cast<float *>(tiles[warp][0]);
#pragma unroll
    for (int n = 0; n < D / 8; n++) {
      my_o[hr * D + n * 8 + 2 * qd] = o[n][0];
      my_o[hr * D + n * 8 + 2 * qd + 1] = o[n][1];
    }
  }
  __syncthreads();
  // merge the warps and the sink; one output element per thread and trip
  for (int idx = tid; idx < group * D; idx += kAttnWarps * 32) {
    const int hl = idx / D, d = idx - hl * D;
    const int h = kvh * group + hl;
    const float sink = sinks[h];
    float m_all = sink;
#pragma unroll
    for (int w = 0; w < kAttnWarps; w++) m_all = fmaxf(m_all, sm_m[w][hl]);
    float lsum = __expf(sink - m_all), acc = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; w++) {
      const float mw = sm_m[w][hl];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - m_all);
      lsum += sm_l[w][hl] * f;
      acc += reinterpret_cast<const float *>(tiles[w][0])[hl * D + d] * f;
    }
    out[(static_cast<size_t>(row) * Hq + h) * D + d] = __float2bfloat16_rn(acc / lsum);
  }
}

// x[row] = bf16(x[row] + proj[row] + bias) for active rows (PROJ_BF: proj is bf16 with
// the bias already added).
template <bool PROJ_BF>
__global__ void __launch_bounds__(256)
bias_residual_kernel(bf16 *__restrict__ x, const void *__restrict__ proj,
                     const float *__restrict__ bias, const int *__restrict__ pos, int B, int H) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<size_t>(B) * H) return;
  const int row = static_cast<int>(i / H), c = static_cast<int>(i - static_cast<size_t>(row) * H);
  if (pos[row] < 0) return;
  const float pv = PROJ_BF ? __bfloat162float(static_cast<const bf16 *>(proj)[i])
                           : static_cast<const float *>(proj)[i] + bias[c];
  x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) + pv);
}

// next[row] = index of the largest logit, lowest index among equals; -1 on inactive rows.
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const float *__restrict__ logits, const int *__restrict__ pos,
                   int *__restrict__ next, int V) {
  const int row = blockIdx.x;
  if (pos[row] < 0) {
    if (threadIdx.x == 0) next[row] = -1;
    return;
  }
  const float *l = logits + static_cast<size_t>(row) * V;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if ((V & 3) == 0) {  // rows are 16-byte aligned: four logits per load, two loads in flight
    const float4 *l4 = reinterpret_cast<const float4 *>(l);
    const int n4 = V >> 2;
    for (int i = threadIdx.x; i < n4; i += 2 * blockDim.x) {
      const int i2 = i + blockDim.x;
      const float4 a = __ldcs(l4 + i);
      const float4 b = i2 < n4 ? __ldcs(l4 + i2) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      const float va[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int idx = (u < 4 ? 4 * i : 4 * i2) + (u & 3);
        // indices only grow inside a thread, so a strict comparison keeps the lowest one
        if (va[u] > best) {
          best = va[u];
          bi = idx;
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = l[i];
      if (v > best) {
        best = v;
        bi = i;
      }
    }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float v = sv[threadIdx.x + s];
      const int i = si[threadIdx.x + s];
      if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) {
        sv[threadIdx.x] = v;
        si[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) next[row] = si[0] == 0x7fffffff ? 0 : si[0];
}

}  // namespace gptoss

using namespace gptoss;

struct gptoss_decode {
  gptoss_model_config_t cfg;
  int max_batch = 0, device = 0;
  gptoss_moe *moe = nullptr;
  cublasHandle_t blas = nullptr;
  bool loaded = false;
  std::vector<unsigned> have;  // per layer (+1 for the model-wide tensors): bits of tensors set
  // weights
  bf16 *emb = nullptr, *unemb = nullptr, *w_qkv = nullptr, *w_o = nullptr;
  float *rms_attn = nullptr, *rms_ffn = nullptr, *rms_out = nullptr;
  float *b_qkv = nullptr, *b_o = nullptr, *sinks = nullptr, *inv_freq = nullptr;
  float concentration = 1.f;
  // state
  bf16 *x = nullptr, *t = nullptr, *attn = nullptr, *k_cache = nullptr, *v_cache = nullptr;
  float *qkv = nullptr, *q = nullptr, *proj = nullptr, *logits = nullptr;
  int *d_tokens = nullptr, *d_pos = nullptr, *d_next = nullptr, *status = nullptr;
  int *h_pinned = nullptr;  // tokens | pos | next, max_batch each
  // QKV and output projections on this library's tcgen05 kernel (one "expert" = all rows)
  bool own_gemm = true;
  int num_sms = 0, sched_B = -1, sched_cap = 0;
  int *lin_sched = nullptr;     // device: expert ids | first rows | row counts | tile count
  float *ones = nullptr;        // [max_batch] row weights of a plain linear layer
  bf16 *qkv_bf = nullptr, *proj_bf = nullptr;
  std::vector<CUtensorMap> tm_wqkv, tm_wo;  // per layer, boxes of 128 weight rows
  CUtensorMap tm_unemb;                     // the unembedding, boxes of 128 rows
  CUtensorMap tm_t[3], tm_attn[3];          // activations in boxes of 128 / 32 / 8 rows
  bool maps_ready = false;
  std::string err;
};

static thread_local std::string g_decode_create_err;

static int dfail(gptoss_decode *h, int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (h)
    h->err = buf;
  else
    g_decode_create_err = buf;
  return code;
}

#define DCK(h, call)                                                                  \
  do {                                                                                \
    cudaError_t e__ = (call);                                                         \
    if (e__ != cudaSuccess)                                                           \
      return dfail((h), GPTOSS_E_CUDA, "%s: %s", #call, cudaGetErrorString(e__));     \
  } while (0)

template <typename T>
static cudaError_t dalloc(T **p, size_t n) {
  return cudaMalloc(reinterpret_cast<void **>(p), (n ? n : 1) * sizeof(T));
}

// inv_freq and concentration exactly as the reference computes them on the host
// (compute_concentration_and_inv_freq, run.cpp:423-474; ntk_beta 32, ntk_alpha 1,
// run.cpp:583-584), in float.
static void rope_tables(const gptoss_model_config_t &c, std::vector<float> *inv_freq,
                        float *concentration) {
  const int d_half = c.head_dim / 2;
  const float base = c.rope_theta, sf = c.rope_scaling_factor;
  const float ctx = static_cast<float>(c.initial_context_length);
  const float ntk_beta = 32.0f, ntk_alpha = 1.0f;
  inv_freq->resize(d_half);
  std::vector<float> freq(d_half);
  for (int i = 0; i < d_half; i++)
    freq[i] = powf(base, static_cast<float>(2 * i) / static_cast<float>(c.head_dim));
  if (sf > 1.0f) {
    *concentration = 0.1f * logf(sf) + 1.0f;
    const float low = d_half * logf(ctx / (ntk_beta * 2.0f * M_PI)) / logf(base);
    const float high = d_half * logf(ctx / (ntk_alpha * 2.0f * M_PI)) / logf(base);
    for (int i = 0; i < d_half; i++) {
      const float interpolation = 1.0f / (sf * freq[i]);
      const float extrapolation = 1.0f / freq[i];
      float ramp = (static_cast<float>(i) - low) / (high - low);
      ramp = ramp < 0 ? 0 : (ramp > 1 ? 1 : ramp);
      const float mask = 1.0f - ramp;
      (*inv_freq)[i] = interpolation * (1.0f - mask) + extrapolation * mask;
    }
  } else {
    *concentration = 1.0f;
    for (int i = 0; i < d_half; i++) (*inv_freq)[i] = 1.0f / freq[i];
  }
}

extern "C" {

const char *gptoss_decode_last_error(const gptoss_decode_t *h) {
  return h ? h->err.c_str() : g_decode_create_err.c_str();
}

gptoss_moe_t *gptoss_decode_moe(gptoss_decode_t *h) { return h ? h->moe : nullptr; }

int gptoss_decode_device_count(void) {
  int n = 0, good = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  for (int d = 0; d < n; d++) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess &&
        major == 10)
      good++;
  }
  return good;
}

int gptoss_decode_destroy(gptoss_decode_t *h) {
  if (!h) return GPTOSS_OK;
  cudaSetDevice(h->device);
  if (h->moe) gptoss_moe_destroy(h->moe);
  if (h->blas) g_blas.Destroy(h->blas);
  cudaFree(h->emb); cudaFree(h->unemb); cudaFree(h->w_qkv); cudaFree(h->w_o);
  cudaFree(h->rms_attn); cudaFree(h->rms_ffn); cudaFree(h->rms_out); cudaFree(h->b_qkv);
  cudaFree(h->b_o); cudaFree(h->sinks); cudaFree(h->inv_freq); cudaFree(h->x); cudaFree(h->t);
  cudaFree(h->attn); cudaFree(h->k_cache); cudaFree(h->v_cache); cudaFree(h->qkv); cudaFree(h->q);
  cudaFree(h->proj); cudaFree(h->logits); cudaFree(h->d_tokens); cudaFree(h->d_pos);
  cudaFree(h->d_next); cudaFree(h->status); cudaFree(h->lin_sched); cudaFree(h->ones);
  cudaFree(h->qkv_bf); cudaFree(h->proj_bf);
  if (h->h_pinned) cudaFreeHost(h->h_pinned);
  delete h;
  return GPTOSS_OK;
}

int gptoss_decode_create(const gptoss_model_config_t *cfg, int max_batch, int device,
                         gptoss_decode_t **out) {
  return gptoss_decode_create_ep(cfg, max_batch, device, 0, 1, out);
}

int gptoss_decode_create_ep(const gptoss_model_config_t *cfg, int max_batch, int device,
                            int ep_rank, int ep_size, gptoss_decode_t **out) {
  if (!cfg || !out) return dfail(nullptr, GPTOSS_E_INVALID, "null argument");
  *out = nullptr;
  const gptoss_model_config_t &c = *cfg;
  if (c.vocab_size <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.head_dim <= 0 ||
      c.n_attn_heads <= 0 || c.n_kv_heads <= 0 || c.seq_len <= 0 || max_batch <= 0)
    return dfail(nullptr, GPTOSS_E_INVALID, "non-positive dimension");
  if (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128)
    return dfail(nullptr, GPTOSS_E_INVALID, "head_dim must be 32, 64 or 128");
  if (c.n_attn_heads % c.n_kv_heads || c.n_attn_heads / c.n_kv_heads > 8)
    return dfail(nullptr, GPTOSS_E_INVALID,
                 "n_attn_heads must be a multiple of n_kv_heads, at most 8 times it");
  if (c.hidden_dim % 8)
    return dfail(nullptr, GPTOSS_E_INVALID, "hidden_dim must be a multiple of 8");
  gptoss_moe_config_t mc = {};
  mc.hidden_dim = c.hidden_dim;
  mc.intermediate_dim = c.intermediate_dim;
  mc.n_experts = c.n_experts;
  mc.experts_per_token = c.experts_per_token;
  mc.n_layers = c.n_layers;
  mc.max_tokens = max_batch;
  mc.swiglu_limit = c.swiglu_limit;
  mc.ep_rank = ep_rank;
  mc.ep_size = ep_size < 1 ? 1 : ep_size;
  mc.weight_format = GPTOSS_WEIGHTS_BF16;
  mc.device = device;
  gptoss_moe *moe = nullptr;
  int rc = gptoss_moe_create(&mc, &moe);
  if (rc != GPTOSS_OK) return dfail(nullptr, rc, "MoE engine: %s", gptoss_moe_last_error(nullptr));
  gptoss_decode *h = new gptoss_decode();
  h->cfg = c;
  h->max_batch = max_batch;
  h->device = device;
  h->moe = moe;
  h->have.assign(c.n_layers + 1, 0u);
  auto bail = [&](int code, const std::string &msg) {
    g_decode_create_err = msg;
    gptoss_decode_destroy(h);
    return code;
  };
  std::string err;
  const size_t V = c.vocab_size, H = c.hidden_dim, L = c.n_layers, D = c.head_dim;
  const size_t dq = c.n_attn_heads * D, dkv = c.n_kv_heads * D, B = max_batch, S = c.seq_len;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
  A(dalloc(&h->emb, V * H)); A(dalloc(&h->unemb, V * H));
  A(dalloc(&h->w_qkv, L * (dq + 2 * dkv) * H)); A(dalloc(&h->w_o, L * H * dq));
  A(dalloc(&h->rms_attn, L * H)); A(dalloc(&h->rms_ffn, L * H)); A(dalloc(&h->rms_out, H));
  A(dalloc(&h->b_qkv, L * (dq + 2 * dkv))); A(dalloc(&h->b_o, L * H));
  A(dalloc(&h->sinks, L * c.n_attn_heads)); A(dalloc(&h->inv_freq, D / 2));
  A(dalloc(&h->x, B * H)); A(dalloc(&h->t, B * H)); A(dalloc(&h->attn, B * dq));
  A(dalloc(&h->k_cache, L * B * S * dkv)); A(dalloc(&h->v_cache, L * B * S * dkv));
  A(dalloc(&h->qkv, B * (dq + 2 * dkv))); A(dalloc(&h->q, B * dq)); A(dalloc(&h->proj, B * H));
  A(dalloc(&h->logits, B * V));
  A(dalloc(&h->d_tokens, B)); A(dalloc(&h->d_pos, B)); A(dalloc(&h->d_next, B));
  A(dalloc(&h->status, 1));
  h->sched_cap = (max_batch + 255) / 256 + 1;
  A(dalloc(&h->lin_sched, 3 * static_cast<size_t>(h->sched_cap) + 1));
  A(dalloc(&h->ones, B));
  A(dalloc(&h->qkv_bf, B * (dq + 2 * dkv)));
  A(dalloc(&h->proj_bf, B * H));
  A(cudaDeviceGetAttribute(&h->num_sms, cudaDevAttrMultiProcessorCount, device));
  A(cudaMallocHost(reinterpret_cast<void **>(&h->h_pinned), 3 * B * sizeof(int)));
  if (e == cudaSuccess) e = cudaMemset(h->status, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(h->x, 0, B * H * sizeof(bf16));
  if (e != cudaSuccess) return bail(GPTOSS_E_CUDA, std::string("allocation: ") + cudaGetErrorString(e));
  {
    std::vector<float> one(B, 1.0f);
    e = cudaMemcpy(h->ones, one.data(), B * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return bail(GPTOSS_E_CUDA, cudaGetErrorString(e));
  }
  std::vector<float> inv;
  rope_tables(c, &inv, &h->concentration);
  e = cudaMemcpy(h->inv_freq, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return bail(GPTOSS_E_CUDA, cudaGetErrorString(e));
  *out = h;
  return GPTOSS_OK;
}

int gptoss_decode_load_weights(gptoss_decode_t *h, const gptoss_model_weights_t *w) {
  if (!h || !w) return GPTOSS_E_INVALID;
  const gptoss_model_config_t &c = h->cfg;
  const size_t V = c.vocab_size, H = c.hidden_dim, L = c.n_layers, D = c.head_dim;
  const size_t dq = c.n_attn_heads * D, dkv = c.n_kv_heads * D;
  const size_t E = c.n_experts, IM = c.intermediate_dim;
  DCK(h, cudaSetDevice(h->device));
  int rc;
  if ((rc = upload_f32_as_bf16(h->moe, h->emb, w->token_embedding_table, V * H)) ||
      (rc = upload_f32_as_bf16(h->moe, h->unemb, w->out, V * H)) ||
      (rc = upload_f32_as_bf16(h->moe, h->w_qkv, w->w_qkv, L * (dq + 2 * dkv) * H)) ||
      (rc = upload_f32_as_bf16(h->moe, h->w_o, w->w_o, L * H * dq)))
    return dfail(h, rc, "weight upload: %s", gptoss_moe_last_error(h->moe));
  DCK(h, cudaMemcpy(h->rms_attn, w->rms_attn_w, L * H * 4, cudaMemcpyHostToDevice));
  DCK(h, cudaMemcpy(h->rms_ffn, w->rms_ffn_w, L * H * 4, cudaMemcpyHostToDevice));
  DCK(h, cudaMemcpy(h->rms_out, w->rms_out_w, H * 4, cudaMemcpyHostToDevice));
  DCK(h, cudaMemcpy(h->b_qkv, w->b_qkv, L * (dq + 2 * dkv) * 4, cudaMemcpyHostToDevice));
  DCK(h, cudaMemcpy(h->b_o, w->b_o, L * H * 4, cudaMemcpyHostToDevice));
  DCK(h, cudaMemcpy(h->sinks, w->attn_sinks, L * c.n_attn_heads * 4, cudaMemcpyHostToDevice));
  for (size_t l = 0; l < L; l++) {
    rc = gptoss_moe_load_layer_f32(h->moe, static_cast<int>(l), w->w_router + l * E * H,
                                   w->b_router + l * E, w->w_mlp1 + l * E * 2 * IM * H,
                                   w->b_mlp1 + l * E * 2 * IM, w->w_mlp2 + l * E * H * IM,
                                   w->b_mlp2 + l * E * H);
    if (rc) return dfail(h, rc, "MoE layer %d: %s", static_cast<int>(l), gptoss_moe_last_error(h->moe));
  }
  if ((rc = upload_finish(h->moe))) return dfail(h, rc, "weight upload: %s", gptoss_moe_last_error(h->moe));
  gptoss_moe_release_upload_staging(h->moe);  // the model is in place: 128 MB of staging go back
  h->loaded = true;
  return GPTOSS_OK;
}

int gptoss_decode_set_tensor(gptoss_decode_t *h, const char *name, int layer, const void *src,
                             int on_device, int is_bf16) {
  if (!h || !name || !src) return GPTOSS_E_INVALID;
  const gptoss_model_config_t &c = h->cfg;
  const size_t V = c.vocab_size, H = c.hidden_dim, D = c.head_dim;
  const size_t dq = c.n_attn_heads * D, dqkv = dq + 2 * c.n_kv_heads * D;
  struct Slot { const char *name; bool per_layer; bool bf; void *base; size_t n; int bit; };
  const Slot slots[] = {
      {"token_embedding_table", false, true, h->emb, V * H, 0},
      {"out", false, true, h->unemb, V * H, 1},
      {"rms_out_w", false, false, h->rms_out, H, 2},
      {"w_qkv", true, true, h->w_qkv, dqkv * H, 0},
      {"b_qkv", true, false, h->b_qkv, dqkv, 1},
      {"w_o", true, true, h->w_o, H * dq, 2},
      {"b_o", true, false, h->b_o, H, 3},
      {"attn_sinks", true, false, h->sinks, static_cast<size_t>(c.n_attn_heads), 4},
      {"rms_attn_w", true, false, h->rms_attn, H, 5},
      {"rms_ffn_w", true, false, h->rms_ffn, H, 6},
  };
  DCK(h, cudaSetDevice(h->device));
  for (const Slot &sl : slots) {
    if (strcmp(sl.name, name)) continue;
    if (sl.per_layer && (layer < 0 || layer >= c.n_layers)) return dfail(h, GPTOSS_E_INVALID, "layer out of range");
    const size_t l = sl.per_layer ? layer : 0;
    if (sl.bf) {
      bf16 *dst = static_cast<bf16 *>(sl.base) + l * sl.n;
      if (on_device && is_bf16) {
        DCK(h, cudaMemcpy(dst, src, sl.n * sizeof(bf16), cudaMemcpyDeviceToDevice));
      } else if (!on_device && !is_bf16) {
        int rc = upload_f32_as_bf16(h->moe, dst, static_cast<const float *>(src), sl.n);
        if (!rc) rc = upload_finish(h->moe);
        if (rc) return dfail(h, rc, "upload: %s", gptoss_moe_last_error(h->moe));
      } else {
        return dfail(h, GPTOSS_E_INVALID, "%s takes fp32 host data or bf16 device data", name);
      }
    } else {
      if (is_bf16) return dfail(h, GPTOSS_E_INVALID, "%s is an fp32 tensor", name);
      float *dst = static_cast<float *>(sl.base) + l * sl.n;
      DCK(h, cudaMemcpy(dst, src, sl.n * sizeof(float),
                        on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    }
    h->have[sl.per_layer ? layer + 1 : 0] |= 1u << sl.bit;
    bool all = h->have[0] == 0x7u;
    for (int i = 1; i <= c.n_layers; i++) all = all && h->have[i] == 0x7fu;
    h->loaded = all;  // the MoE engine checks its own layers
    return GPTOSS_OK;
  }
  return dfail(h, GPTOSS_E_INVALID, "unknown tensor '%s'", name);
}

int gptoss_decode_set_kv(gptoss_decode_t *h, int layer, int row0, int n_rows, int pos0, int n_pos,
                         const void *k_dev, const void *v_dev) {
  if (!h || !k_dev || !v_dev) return GPTOSS_E_INVALID;
  const gptoss_model_config_t &c = h->cfg;
  if (layer < 0 || layer >= c.n_layers || row0 < 0 || n_rows < 0 || row0 + n_rows > h->max_batch ||
      pos0 < 0 || n_pos < 0 || pos0 + n_pos > c.seq_len)
    return dfail(h, GPTOSS_E_INVALID, "cache region out of range");
  if (n_rows == 0 || n_pos == 0) return GPTOSS_OK;
  DCK(h, cudaSetDevice(h->device));
  const size_t dkv = static_cast<size_t>(c.n_kv_heads) * c.head_dim, S = c.seq_len;
  const size_t off = ((static_cast<size_t>(layer) * h->max_batch + row0) * S + pos0) * dkv;
  // per row: n_pos * dkv contiguous elements, rows S * dkv apart in the cache
  DCK(h, cudaMemcpy2D(h->k_cache + off, S * dkv * sizeof(bf16), k_dev, n_pos * dkv * sizeof(bf16),
                      n_pos * dkv * sizeof(bf16), n_rows, cudaMemcpyDeviceToDevice));
  DCK(h, cudaMemcpy2D(h->v_cache + off, S * dkv * sizeof(bf16), v_dev, n_pos * dkv * sizeof(bf16),
                      n_pos * dkv * sizeof(bf16), n_rows, cudaMemcpyDeviceToDevice));
  return GPTOSS_OK;
}

int gptoss_decode_get_kv(gptoss_decode_t *h, int layer, int row0, int n_rows, int pos0, int n_pos,
                         void *k_dev, void *v_dev) {
  if (!h || !k_dev || !v_dev) return GPTOSS_E_INVALID;
  const gptoss_model_config_t &c = h->cfg;
  if (layer < 0 || layer >= c.n_layers || row0 < 0 || n_rows < 0 || row0 + n_rows > h->max_batch ||
      pos0 < 0 || n_pos < 0 || pos0 + n_pos > c.seq_len)
    return dfail(h, GPTOSS_E_INVALID, "cache region out of range");
  if (n_rows == 0 || n_pos == 0) return GPTOSS_OK;
  DCK(h, cudaSetDevice(h->device));
  const size_t dkv = static_cast<size_t>(c.n_kv_heads) * c.head_dim, S = c.seq_len;
  const size_t off = ((static_cast<size_t>(layer) * h->max_batch + row0) * S + pos0) * dkv;
  DCK(h, cudaMemcpy2D(k_dev, n_pos * dkv * sizeof(bf16), h->k_cache + off, S * dkv * sizeof(bf16),
                      n_pos * dkv * sizeof(bf16), n_rows, cudaMemcpyDeviceToDevice));
  DCK(h, cudaMemcpy2D(v_dev, n_pos * dkv * sizeof(bf16), h->v_cache + off, S * dkv * sizeof(bf16),
                      n_pos * dkv * sizeof(bf16), n_rows, cudaMemcpyDeviceToDevice));
  return GPTOSS_OK;
}

int gptoss_decode_load_bin(gptoss_decode_t *h, const float *p) {
  if (!h || !p) return GPTOSS_E_INVALID;
  const gptoss_model_config_t &c = h->cfg;
  const size_t V = c.vocab_size, H = c.hidden_dim, L = c.n_layers, D = c.head_dim;
  const size_t dqkv = (c.n_attn_heads + 2 * c.n_kv_heads) * D, dq = c.n_attn_heads * D;
  const size_t E = c.n_experts, IM = c.intermediate_dim;
  gptoss_model_weights_t w;
  // the file's order (memory_map_weights, run.cpp:207-248)
  w.token_embedding_table = p; p += V * H;
  w.out = p;                   p += V * H;
  w.rms_attn_w = p;            p += L * H;
  w.rms_ffn_w = p;             p += L * H;
  w.rms_out_w = p;             p += H;
  w.w_qkv = p;                 p += L * H * dqkv;
  w.b_qkv = p;                 p += L * dqkv;
  w.w_o = p;                   p += L * dq * H;
  w.b_o = p;                   p += L * H;
  w.attn_sinks = p;            p += L * c.n_attn_heads;
  w.w_router = p;              p += L * H * E;
  w.b_router = p;              p += L * E;
  w.w_mlp1 = p;                p += L * E * 2 * IM * H;
  w.b_mlp1 = p;                p += L * E * 2 * IM;
  w.w_mlp2 = p;                p += L * E * H * IM;
  w.b_mlp2 = p;
  return gptoss_decode_load_weights(h, &w);
}

// C[B, N] (fp32) = X[B, K] (bf16) . W[N, K]^T (bf16)
static int gemm_xwt(gptoss_decode *h, const bf16 *x, const bf16 *w, float *c, int B, int N, int K,
                    cudaStream_t st) {
  if (!h->blas) {  // only shapes the library's own kernel does not take come here
    std::string err;
    if (!load_cublas(&err)) return dfail(h, GPTOSS_E_STATE, "%s", err.c_str());
    if (g_blas.Create(&h->blas) != CUBLAS_STATUS_SUCCESS) return dfail(h, GPTOSS_E_CUDA, "cublasCreate failed");
  }
  if (g_blas.SetStream(h->blas, st) != CUBLAS_STATUS_SUCCESS) return dfail(h, GPTOSS_E_CUDA, "cublasSetStream failed");
  const float one = 1.f, zero = 0.f;
  cublasStatus_t s = g_blas.GemmEx(h->blas, CUBLAS_OP_T, CUBLAS_OP_N, N, B, K, &one, w,
                                   CUDA_R_16BF, K, x, CUDA_R_16BF, K, &zero, c, CUDA_R_32F, N,
                                   CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (s != CUBLAS_STATUS_SUCCESS) return dfail(h, GPTOSS_E_CUDA, "cublasGemmEx failed (%d)", (int)s);
  return GPTOSS_OK;
}

// Tensor maps of the projections (weights per layer, the two activation buffers).
static int build_linear_maps(gptoss_decode *h) {
  const gptoss_model_config_t &c = h->cfg;
  const uint64_t H = c.hidden_dim, D = c.head_dim, dq = c.n_attn_heads * D;
  const uint64_t dqkv = dq + 2 * c.n_kv_heads * D;
  std::string err;
  h->tm_wqkv.resize(c.n_layers);
  h->tm_wo.resize(c.n_layers);
  int rc = 0;
  for (int l = 0; l < c.n_layers && !rc; l++) {
    rc = make_tmap_2d_bf16(&h->tm_wqkv[l], h->w_qkv + l * dqkv * H, H, dqkv, kTileK, 128, &err) ||
         make_tmap_2d_bf16(&h->tm_wo[l], h->w_o + l * H * dq, dq, H, kTileK, 128, &err);
  }
  if (!rc) rc = make_tmap_2d_bf16(&h->tm_unemb, h->unemb, H, c.vocab_size, kTileK, 128, &err);
  const uint32_t boxes[3] = {128, 32, 8};
  for (int i = 0; i < 3 && !rc; i++) {
    rc = make_tmap_2d_bf16(&h->tm_t[i], h->t, H, h->max_batch, kTileK, boxes[i], &err) ||
         make_tmap_2d_bf16(&h->tm_attn[i], h->attn, dq, h->max_batch, kTileK, boxes[i], &err);
  }
  if (rc) return dfail(h, GPTOSS_E_CUDA, "tensor maps of the projections: %s", err.c_str());
  h->maps_ready = true;
  return GPTOSS_OK;
}

// Tile schedule of a plain linear layer over B rows: ceil(B / 256) tiles of equal size
// (a multiple of 16), all of "expert" 0.
static int build_linear_schedule(gptoss_decode *h, int B, cudaStream_t st) {
  const int cap = h->sched_cap;
  std::vector<int> sched(3 * cap + 1, 0);
  const int cnt = (B + 255) / 256;
  const int step = (((B + cnt - 1) / cnt) + 15) & ~15;
  int n = 0;
  for (int r = 0; r < B && n < cap; r += step, n++) {
    sched[cap + n] = r;
    sched[2 * cap + n] = std::min(step, B - r);
  }
  sched[3 * cap] = n;
  DCK(h, cudaMemcpyAsync(h->lin_sched, sched.data(), sched.size() * sizeof(int),
                         cudaMemcpyHostToDevice, st));
  DCK(h, cudaStreamSynchronize(st));  // the host vector goes out of scope
  h->sched_B = B;
  return GPTOSS_OK;
}

// out[B, N] (bf16) = x[B, K] . W[N, K]^T + bias on the CTA-pair tcgen05 kernel
static int linear_own(gptoss_decode *h, const CUtensorMap &tw, const CUtensorMap *tx,
                      const float *bias, void *out, int N, int K, cudaStream_t st,
                      bool f32_out = false) {
  GemmArgs g;
  g.bias = bias;
  g.out = static_cast<bf16 *>(out);
  g.row_weight = h->ones;
  g.mtile_expert = h->lin_sched;
  g.mtile_row0 = h->lin_sched + h->sched_cap;
  g.mtile_rows = h->lin_sched + 2 * h->sched_cap;
  g.num_mtiles = h->lin_sched + 3 * h->sched_cap;
  g.k_dim = K;
  g.n_cols = N;
  g.out_ld = N;
  g.limit = 0.f;
  g.status = h->status;
  DCK(h, launch_linear_pair(h->num_sms, tw, tx, g, st, nullptr, f32_out));
  return GPTOSS_OK;
}

int gptoss_decode_step(gptoss_decode_t *h, const int *tokens, const int *pos, int B, int *next,
                       void *stream) {
  if (!h || !tokens || !pos || !next) return GPTOSS_E_INVALID;
  if (!h->loaded) return dfail(h, GPTOSS_E_STATE, "weights not loaded");
  if (B < 0 || B > h->max_batch) return dfail(h, GPTOSS_E_CAPACITY, "batch %d > max_batch %d", B, h->max_batch);
  if (B == 0) return GPTOSS_OK;
  const gptoss_model_config_t &c = h->cfg;
  for (int i = 0; i < B; i++)
    if (pos[i] >= c.seq_len) return dfail(h, GPTOSS_E_CAPACITY, "row %d: position %d >= seq_len %d", i, pos[i], c.seq_len);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DCK(h, cudaSetDevice(h->device));
  const int H = c.hidden_dim, D = c.head_dim, Hq = c.n_attn_heads, Hkv = c.n_kv_heads;
  const int dq = Hq * D, dkv = Hkv * D, S = c.seq_len, V = c.vocab_size;
  int *hp = h->h_pinned;
  memcpy(hp, tokens, B * sizeof(int));
  memcpy(hp + h->max_batch, pos, B * sizeof(int));
  DCK(h, cudaMemcpyAsync(h->d_tokens, hp, B * sizeof(int), cudaMemcpyHostToDevice, st));
  DCK(h, cudaMemcpyAsync(h->d_pos, hp + h->max_batch, B * sizeof(int), cudaMemcpyHostToDevice, st));
  const int warps = 8;
  embed_rows_kernel<<<(B + warps - 1) / warps, warps * 32, 0, st>>>(h->x, h->emb, h->d_tokens,
                                                                   h->d_pos, B, H, V, h->status);
  DCK(h, cudaGetLastError());
  int rc;
  // the tcgen05 kernel writes whole 16-byte segments: row lengths must be multiples of 8
  const bool own = h->own_gemm && ((dq + 2 * dkv) % 8 == 0) && (dq % 8 == 0);
  if (own) {
    if (!h->maps_ready && (rc = build_linear_maps(h))) return rc;
    if (h->sched_B != B && (rc = build_linear_schedule(h, B, st))) return rc;
  }
  for (int l = 0; l < c.n_layers; l++) {
    DCK(h, launch_rmsnorm(h->t, h->x, h->rms_attn + static_cast<size_t>(l) * H, h->d_pos, B, H, st, nullptr));
    if (own)
      rc = linear_own(h, h->tm_wqkv[l], h->tm_t, h->b_qkv + static_cast<size_t>(l) * (dq + 2 * dkv),
                      h->qkv_bf, dq + 2 * dkv, H, st);
    else
      rc = gemm_xwt(h, h->t, h->w_qkv + static_cast<size_t>(l) * (dq + 2 * dkv) * H, h->qkv, B,
                    dq + 2 * dkv, H, st);
    if (rc) return rc;
    bf16 *kc = h->k_cache + static_cast<size_t>(l) * h->max_batch * S * dkv;
    bf16 *vc = h->v_cache + static_cast<size_t>(l) * h->max_batch * S * dkv;
    if (own)
      qkv_rope_cache_kernel<true><<<B, 256, 0, st>>>(h->qkv_bf, nullptr, h->d_pos, h->inv_freq,
                                                     h->concentration, h->q, kc, vc, B, Hq, Hkv, D, S);
    else
      qkv_rope_cache_kernel<false><<<B, 256, 0, st>>>(
          h->qkv, h->b_qkv + static_cast<size_t>(l) * (dq + 2 * dkv), h->d_pos, h->inv_freq,
          h->concentration, h->q, kc, vc, B, Hq, Hkv, D, S);
    DCK(h, cudaGetLastError());
    // sliding window on even layers (run.cpp:619)
    const int window = (c.sliding_window > 0 && (l % 2 == 0)) ? c.sliding_window : 0;
    // one CTA per (row, KV head): the group's query heads are the rows of the MMA tiles
    const int grid = B * Hkv, threads = kAttnWarps * 32;
    const float *sinks = h->sinks + static_cast<size_t>(l) * Hq;
    if (D == 32)
      attn_decode_kernel<32><<<grid, threads, 0, st>>>(h->q, kc, vc, sinks, h->d_pos, h->attn, B, Hq, Hkv, S, window);
    else if (D == 64)
      attn_decode_kernel<64><<<grid, threads, 0, st>>>(h->q, kc, vc, sinks, h->d_pos, h->attn, B, Hq, Hkv, S, window);
    else
      attn_decode_kernel<128><<<grid, threads, 0, st>>>(h->q, kc, vc, sinks, h->d_pos, h->attn, B, Hq, Hkv, S, window);
    DCK(h, cudaGetLastError());
    const size_t n = static_cast<size_t>(B) * H;
    if (own) {
      if ((rc = linear_own(h, h->tm_wo[l], h->tm_attn, h->b_o + static_cast<size_t>(l) * H,
                           h->proj_bf, H, dq, st)))
        return rc;
      bias_residual_kernel<true><<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
          h->x, h->proj_bf, nullptr, h->d_pos, B, H);
    } else {
      if ((rc = gemm_xwt(h, h->attn, h->w_o + static_cast<size_t>(l) * H * dq, h->proj, B, H, dq, st)))
        return rc;
      bias_residual_kernel<false><<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
          h->x, h->proj, h->b_o + static_cast<size_t>(l) * H, h->d_pos, B, H);
    }
    DCK(h, cudaGetLastError());
    DCK(h, launch_rmsnorm(h->t, h->x, h->rms_ffn + static_cast<size_t>(l) * H, h->d_pos, B, H, st, nullptr));
    rc = gptoss_moe_forward(h->moe, l, h->t, h->x, h->d_pos, B, st);
    if (rc) return dfail(h, rc, "MoE layer %d: %s", l, gptoss_moe_last_error(h->moe));
  }
  DCK(h, launch_rmsnorm(h->t, h->x, h->rms_out, h->d_pos, B, H, st, nullptr));
  // fp32 logits: own kernel when the rows of the logits are 16-byte multiples, else cuBLAS
  if (own && V % 4 == 0)
    rc = linear_own(h, h->tm_unemb, h->tm_t, nullptr, h->logits, V, H, st, /*f32_out=*/true);
  else
    rc = gemm_xwt(h, h->t, h->unemb, h->logits, B, V, H, st);
  if (rc) return rc;
  argmax_rows_kernel<<<B, 256, 0, st>>>(h->logits, h->d_pos, h->d_next, V);
  DCK(h, cudaGetLastError());
  DCK(h, cudaMemcpyAsync(hp + 2 * h->max_batch, h->d_next, B * sizeof(int), cudaMemcpyDeviceToHost, st));
  DCK(h, cudaStreamSynchronize(st));
  memcpy(next, hp + 2 * h->max_batch, B * sizeof(int));
  int dev_status = 0;
  DCK(h, cudaMemcpy(&dev_status, h->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (dev_status) {
    cudaMemset(h->status, 0, sizeof(int));
    return dfail(h, GPTOSS_E_DEVICE, "a decode kernel reported status %d (token id out of range?)", dev_status);
  }
  // the MoE engine keeps its own status word: pipeline and peer-flag waits that ran out
  if (gptoss_moe_take_status(h->moe) != GPTOSS_OK)
    return dfail(h, GPTOSS_E_DEVICE, "MoE block: %s", gptoss_moe_last_error(h->moe));
  return GPTOSS_OK;
}

int gptoss_decode_get_logits(gptoss_decode_t *h, int row, float *logits_host) {
  if (!h || !logits_host) return GPTOSS_E_INVALID;
  if (row < 0 || row >= h->max_batch) return dfail(h, GPTOSS_E_INVALID, "row out of range");
  DCK(h, cudaSetDevice(h->device));
  DCK(h, cudaMemcpy(logits_host, h->logits + static_cast<size_t>(row) * h->cfg.vocab_size,
                    sizeof(float) * h->cfg.vocab_size, cudaMemcpyDeviceToHost));
  return GPTOSS_OK;
}

}  // extern "C"
