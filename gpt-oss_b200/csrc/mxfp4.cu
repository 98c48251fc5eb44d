// MXFP4 expert weights: upload and device layout.
//
// Input is the checkpoint's own form (the reference's exporter reads exactly this
// before it dequantises, export_model_bin/gpt-oss-120b/export_model_bin.py:80-137):
// blocks = packed e2m1 codes, two per byte, low nibble = even element; scales =
// e8m0 bytes (2^(s-127)), one per 32 consecutive elements of the contraction
// dimension.  The reference never keeps fp4 on the GPU; this engine does, and
// dequantises inside the GEMM's load path (grouped_gemm_pair.cu), so a layer
// streams 0.53 byte per weight from HBM instead of 2.
//
// Device layout (chosen for that kernel, one contiguous bulk copy per pipeline
// stage): weight rows are cut into blocks of 128 (one CTA's M tile; the last
// block of an expert is zero padded, and the block count per expert is even so a
// CTA pair always owns two), the contraction dimension into K blocks of 64:
//   tile[expert][block][kblock] = { codes[128 rows][32 bytes], scales[128 rows][2 bytes] }
// i.e. 4352 contiguous bytes per (block, K block): one bulk copy per stage.
// Inside every 32-bit word of codes the eight nibbles are reordered from e0 e1 ... e7
// (element k at bits 4k) to e0 e2 e4 e6 | e1 e3 e5 e7: the two elements of a bf16 pair then
// sit 16 bits apart, where one mask picks both (grouped_gemm_pair.cu expands them).
#include "common.cuh"
#include "engine.h"

namespace gptoss {

__global__ void __launch_bounds__(256)
mxfp4_tile_codes_kernel(uint8_t *__restrict__ q, const uint8_t *__restrict__ blocks, int rows,
                        int k_bytes, int nb, int kb_count, int e_local, int e_global) {
  // one thread per 16-byte piece of the tiled layout of one expert
  const size_t total = static_cast<size_t>(nb) * kb_count * 128 * 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int piece = static_cast<int>(i & 1);
    const int r = static_cast<int>((i >> 1) & 127);
    const size_t rest = i >> 8;
    const int kb = static_cast<int>(rest % kb_count);
    const int blk = static_cast<int>(rest / kb_count);
    const int row = blk * 128 + r;
    const int b0 = kb * 32 + piece * 16;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows && b0 < k_bytes) {
      const uint8_t *src = blocks + (static_cast<size_t>(e_global) * rows + row) * k_bytes + b0;
      if (b0 + 16 <= k_bytes && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        v = *reinterpret_cast<const uint4 *>(src);
      } else {
        uint8_t tmp[16];
        for (int j = 0; j < 16; j++) tmp[j] = (b0 + j < k_bytes) ? src[j] : 0;
        memcpy(&v, tmp, 16);
      }
    }
    {
      uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint32_t x = w[j];
        // even elements (nibbles 0, 2, 4, 6) to bits 0-15, odd ones to bits 16-31
        const uint32_t ev = (x & 0xFu) | ((x >> 4) & 0xF0u) | ((x >> 8) & 0xF00u) | ((x >> 12) & 0xF000u);
        const uint32_t y = x >> 4;
        const uint32_t od = (y & 0xFu) | ((y >> 4) & 0xF0u) | ((y >> 8) & 0xF00u) | ((y >> 12) & 0xF000u);
        w[j] = ev | (od << 16);
      }
      v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    // 4352-byte tiles: 4096 bytes of codes, then 256 bytes of scales
    const size_t tile = i >> 8, inside = i & 255;
    const size_t tiles_per_expert = static_cast<size_t>(nb) * kb_count;
    *reinterpret_cast<uint4 *>(q + (static_cast<size_t>(e_local) * tiles_per_expert + tile) * 4352 +
                               inside * 16) = v;
  }
}

__global__ void __launch_bounds__(256)
mxfp4_tile_scales_kernel(uint8_t *__restrict__ s, const uint8_t *__restrict__ scales, int rows,
                         int k_groups, int nb, int kb_count, int e_local, int e_global) {
  const size_t total = static_cast<size_t>(nb) * kb_count * 128 * 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i & 1);
    const int r = static_cast<int>((i >> 1) & 127);
    const size_t rest = i >> 8;
    const int kb = static_cast<int>(rest % kb_count);
    const int blk = static_cast<int>(rest / kb_count);
    const int row = blk * 128 + r;
    const int grp = kb * 2 + j;
    uint8_t v = 127;  // 2^0; the codes it scales are zero padding
    if (row < rows && grp < k_groups)
      v = scales[(static_cast<size_t>(e_global) * rows + row) * k_groups + grp];
    const size_t tile = i >> 8, inside = i & 255;
    const size_t tiles_per_expert = static_cast<size_t>(nb) * kb_count;
    s[(static_cast<size_t>(e_local) * tiles_per_expert + tile) * 4352 + 4096 + inside] = v;
  }
}

size_t mxfp4_blocks_per_expert(int rows) { return static_cast<size_t>((rows + 255) / 256) * 2; }

// Tiles one tensor ([E, rows, k] codes + scales, host or device pointers) into
// a freshly allocated device buffer *q_out for the experts this rank owns.
static int tile_tensor(gptoss_moe *h, const uint8_t *blocks, const uint8_t *scales, int rows, int k,
                       int on_device, uint8_t **q_out) {
  const int k_bytes = k / 2, k_groups = k / 32;
  const int kb_count = (k + kTileK - 1) / kTileK;
  const int nb = static_cast<int>(mxfp4_blocks_per_expert(rows));
  const size_t per_q = static_cast<size_t>(nb) * kb_count * 4352;  // codes + scales
  const size_t src_q = static_cast<size_t>(h->E) * rows * k_bytes;
  const size_t src_s = static_cast<size_t>(h->E) * rows * k_groups;
  auto fail = [&](const char *what, cudaError_t e) {
    h->err = std::string(what) + ": " + cudaGetErrorString(e);
    return GPTOSS_E_CUDA;
  };
  cudaError_t e;
  if (!*q_out && (e = cudaMalloc(reinterpret_cast<void **>(q_out), per_q * h->El)) != cudaSuccess)
    return fail("cudaMalloc(codes)", e);
  const uint8_t *dq = blocks, *ds = scales;
  uint8_t *tq = nullptr, *ts = nullptr;
  if (!on_device) {
    if ((e = cudaMalloc(reinterpret_cast<void **>(&tq), src_q)) != cudaSuccess)
      return fail("cudaMalloc(staging)", e);
    if ((e = cudaMalloc(reinterpret_cast<void **>(&ts), src_s)) != cudaSuccess) {
      cudaFree(tq);
      return fail("cudaMalloc(staging)", e);
    }
    cudaMemcpy(tq, blocks, src_q, cudaMemcpyHostToDevice);
    cudaMemcpy(ts, scales, src_s, cudaMemcpyHostToDevice);
    dq = tq;
    ds = ts;
  }
  for (int j = 0; j < h->El; j++) {
    const int eg = j * h->ep_size + h->ep_rank;
    mxfp4_tile_codes_kernel<<<592, 256>>>(*q_out, dq, rows, k_bytes, nb, kb_count, j, eg);
    mxfp4_tile_scales_kernel<<<592, 256>>>(*q_out, ds, rows, k_groups, nb, kb_count, j, eg);
    h->launches += 2;
  }
  e = cudaDeviceSynchronize();
  cudaFree(tq);
  cudaFree(ts);
  if (e != cudaSuccess) return fail("tiling kernels", e);
  return GPTOSS_OK;
}

template <typename T>
static cudaError_t put(T **dst, const T *src, size_t n, cudaMemcpyKind kind) {
  if (!*dst) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(dst), (n ? n : 1) * sizeof(T));
    if (e != cudaSuccess) return e;
  }
  return cudaMemcpy(*dst, src, n * sizeof(T), kind);
}

}  // namespace gptoss

using namespace gptoss;

extern "C" int gptoss_moe_load_layer_mxfp4(gptoss_moe_t *h, int layer, const void *w_router_bf16,
                                           const float *b_router, const uint8_t *w_mlp1_blocks,
                                           const uint8_t *w_mlp1_scales, const float *b_mlp1,
                                           const uint8_t *w_mlp2_blocks,
                                           const uint8_t *w_mlp2_scales, const float *b_mlp2,
                                           int on_device) {
  if (!h) return GPTOSS_E_INVALID;
  auto fail = [&](int code, const std::string &m) {
    h->err = m;
    return code;
  };
  if (layer < 0 || layer >= h->L) return fail(GPTOSS_E_INVALID, "layer out of range");
  if (h->cfg.weight_format != GPTOSS_WEIGHTS_MXFP4)
    return fail(GPTOSS_E_STATE, "engine was not created with GPTOSS_WEIGHTS_MXFP4");
  if (!w_router_bf16 || !b_router || !w_mlp1_blocks || !w_mlp1_scales || !b_mlp1 ||
      !w_mlp2_blocks || !w_mlp2_scales || !b_mlp2)
    return fail(GPTOSS_E_INVALID, "null weight pointer");
  if (cudaSetDevice(h->cfg.device) != cudaSuccess) return fail(GPTOSS_E_CUDA, "cudaSetDevice");
  LayerWeights &lw = h->layers[layer];
  const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  const size_t H = h->H, IM = h->IM, E = h->E;
  cudaError_t e;
  if ((e = put(&lw.w_router, static_cast<const bf16 *>(w_router_bf16), E * H, kind)) != cudaSuccess ||
      (e = put(&lw.b_router, b_router, E, kind)) != cudaSuccess)
    return fail(GPTOSS_E_CUDA, std::string("router upload: ") + cudaGetErrorString(e));
  if (!lw.b1 && (e = cudaMalloc(reinterpret_cast<void **>(&lw.b1), h->El * 2 * IM * 4)) != cudaSuccess)
    return fail(GPTOSS_E_CUDA, cudaGetErrorString(e));
  if (!lw.b2 && (e = cudaMalloc(reinterpret_cast<void **>(&lw.b2), h->El * H * 4)) != cudaSuccess)
    return fail(GPTOSS_E_CUDA, cudaGetErrorString(e));
  for (int j = 0; j < h->El; j++) {
    const size_t eg = static_cast<size_t>(j) * h->ep_size + h->ep_rank;
    if ((e = cudaMemcpy(lw.b1 + j * 2 * IM, b_mlp1 + eg * 2 * IM, 2 * IM * 4, kind)) != cudaSuccess ||
        (e = cudaMemcpy(lw.b2 + j * H, b_mlp2 + eg * H, H * 4, kind)) != cudaSuccess)
      return fail(GPTOSS_E_CUDA, std::string("bias upload: ") + cudaGetErrorString(e));
  }
  int rc = tile_tensor(h, w_mlp1_blocks, w_mlp1_scales, 2 * h->IM, h->H, on_device, &lw.w1_blocks);
  if (rc) return rc;
  rc = tile_tensor(h, w_mlp2_blocks, w_mlp2_scales, h->H, h->IM, on_device, &lw.w2_blocks);
  if (rc) return rc;
  if ((rc = build_router_tiles(h, lw))) return rc;
  lw.loaded = true;
  return GPTOSS_OK;
}
