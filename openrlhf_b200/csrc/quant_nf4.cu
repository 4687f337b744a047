// NF4 (4-bit NormalFloat) block quantisation of bf16 weights: blocks of 64 values share one fp32 absmax, every value
// is stored as the index of the nearest of 16 fixed levels (the quantiles of a standard normal scaled to [-1, 1],
// Dettmers et al., QLoRA), two indices per byte (first value in the high nibble).
// The reference reaches this format through bitsandbytes (openrlhf/models/actor.py:115-124).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

__constant__ float NF4_LEVELS[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f, -0.28444138169288635f,
    -0.18477343022823334f, -0.09105003625154495f, 0.0f, 0.07958029955625534f, 0.16093020141124725f,
    0.24611230194568634f, 0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f,
    1.0f};

__device__ __forceinline__ int nf4_index(float x) {
  // nearest level: the levels are sorted, compare against the 15 midpoints
  int idx = 0;
#pragma unroll
  for (int i = 0; i < 15; ++i) idx += x > 0.5f * (NF4_LEVELS[i] + NF4_LEVELS[i + 1]) ? 1 : 0;
  return idx;
}

// one warp per block of 64 values: lane l handles values 2l and 2l+1 (one output byte)
__global__ void nf4_quantize_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ codes,
                                    float* __restrict__ absmax, long long n_blocks) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long b = warp; b < n_blocks; b += warps) {
    const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(w + b * 64)[lane];
    const float a = __bfloat162float(v.x), c = __bfloat162float(v.y);
    float m = fmaxf(fabsf(a), fabsf(c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float inv = m > 0.f ? 1.f / m : 0.f;
    codes[b * 32 + lane] = (uint8_t)((nf4_index(a * inv) << 4) | nf4_index(c * inv));
    if (lane == 0) absmax[b] = m;
  }
}

__global__ void nf4_dequantize_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ absmax,
                                      __nv_bfloat16* __restrict__ w, long long n_blocks) {
  const long long total = n_blocks * 32;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const uint8_t c = codes[i];
    const float m = absmax[i >> 5];
    reinterpret_cast<__nv_bfloat162*>(w)[i] = __floats2bfloat162_rn(NF4_LEVELS[c >> 4] * m, NF4_LEVELS[c & 15] * m);
  }
}

}  // namespace b200

using namespace b200;

// n must be a multiple of 64; codes: n / 2 bytes; absmax: n / 64 floats.
extern "C" int b200_nf4_quantize(const void* w, void* codes, float* absmax, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 64) return -10;
  const long long blocks = n / 64;
  long long ctas = (blocks + 7) / 8;
  if (ctas > 148 * 16) ctas = 148 * 16;
  nf4_quantize_kernel<<<(int)ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)w, (uint8_t*)codes, absmax, blocks);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_nf4_dequantize(const void* codes, const float* absmax, void* w, long long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 64) return -10;
  const long long blocks = n / 64;
  long long ctas = (blocks * 32 + 255) / 256;
  if (ctas > 148 * 16) ctas = 148 * 16;
  nf4_dequantize_kernel<<<(int)ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)codes, absmax, (__nv_bfloat16*)w, blocks);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
