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

}  // namespace gptoss
