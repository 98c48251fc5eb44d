// fp32 -> bf16 conversion on the device (round to nearest even), used while
// uploading the fp32 checkpoint tensors.  Replaces the host-side OpenMP
// conversion of the reference (getp-csrc/utility/utility.cpp:417-556), which
// dominates its 45 s warm-up.
#include "common.cuh"
#include "engine.h"

namespace gptoss {

__global__ void __launch_bounds__(256)
f32_to_bf16_kernel(bf16 *__restrict__ dst, const float *__restrict__ src, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t n4 = n >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += stride) {
    const float4 v = reinterpret_cast<const float4 *>(src)[i];
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    reinterpret_cast<uint2 *>(dst)[i] = o;
  }
  for (size_t i = (n4 << 2) + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

cudaError_t launch_f32_to_bf16(bf16 *dst, const float *src, size_t n, cudaStream_t stream,
                               long long *launches) {
  if (n == 0) return cudaSuccess;
  size_t blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks == 0) blocks = 1;
  f32_to_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(dst, src, n);
  if (launches) ++*launches;
  return cudaGetLastError();
}

// A weight matrix re-tiled into the shared-memory image of a tcgen05 operand.
//
// An MMA operand is, per pipeline step, a tile of 128 rows x 64 k in the 128-byte-swizzled
// shared-memory layout.  Read from a row-major [rows, k] matrix that is 128 row segments of
// 128 bytes; stored tile by tile in exactly the bytes the shared-memory tile holds, the
// same operand is one contiguous 16 KB piece that a box of 32 rows x 512 bytes (no swizzle)
// moves.  Used for the router rows (router.cu), which every CTA re-reads from L2 once per K
// chunk.  For the expert weights, which stream from HBM once, the tiled form measured no
// faster than the row-major one in the CTA-pair GEMM and is not kept.  (The reference
// re-tiles every weight for its MFMA kernels at upload, getp-csrc/utility/utility.cpp:558-622.)
//
// Layout: tile[(expert * blocks + row_block) * k_blocks + k_block], each 128 x 64 bf16;
// inside a tile the 16-byte chunk c of row r sits at byte r * 128 + ((c ^ (r & 7)) << 4).
// blocks = an even number of 128-row blocks per matrix; rows past the last row and k past
// the contraction length are zero.
__global__ void __launch_bounds__(256)
retile_weights_kernel(bf16 *__restrict__ dst, const bf16 *__restrict__ src, int rows, int k,
                      int blocks, int k_blocks, int n_experts) {
  // one thread per 16-byte chunk of the tiled image
  const size_t total = static_cast<size_t>(n_experts) * blocks * k_blocks * 1024;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i & 7);            // chunk of the row as stored
    const int r = static_cast<int>((i >> 3) & 127);   // row of the tile
    const size_t tile = i >> 10;
    const int kb = static_cast<int>(tile % k_blocks);
    const size_t rest = tile / k_blocks;
    const int rb = static_cast<int>(rest % blocks);
    const int e = static_cast<int>(rest / blocks);
    const int src_chunk = c ^ (r & 7);                // the chunk of the row that lives here
    const int row = rb * 128 + r;
    const int col = kb * 64 + src_chunk * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < rows && col < k)
      v = *reinterpret_cast<const uint4 *>(src + (static_cast<size_t>(e) * rows + row) * k + col);
    reinterpret_cast<uint4 *>(dst)[i] = v;
  }
}

size_t tiled_weight_elems(int rows, int k, int n_experts) {
  const size_t blocks = static_cast<size_t>((rows + 255) / 256) * 2;
  const size_t k_blocks = (k + kTileK - 1) / kTileK;
  return static_cast<size_t>(n_experts) * blocks * k_blocks * 128 * kTileK;
}

cudaError_t launch_retile_weights(bf16 *dst, const bf16 *src, int rows, int k, int n_experts,
                                  cudaStream_t stream, long long *launches) {
  const int blocks = ((rows + 255) / 256) * 2;
  const int k_blocks = (k + kTileK - 1) / kTileK;
  retile_weights_kernel<<<148 * 8, 256, 0, stream>>>(dst, src, rows, k, blocks, k_blocks, n_experts);
  if (launches) ++*launches;
  return cudaGetLastError();
}

}  // namespace gptoss
