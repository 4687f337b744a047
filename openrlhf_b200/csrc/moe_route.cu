// Mixture-of-experts router: softmax over the expert logits, top-k selection, optional renormalisation of the k
// weights, per-expert token counts and per-expert probability sums (the two factors of the load-balancing loss), one
// warp per token. Replaces the softmax / topk / one-hot / mean chain of transformers' Qwen3MoeTopKRouter and
// load_balancing_loss_func, which the reference trains through (openrlhf/trainer/ray/ppo_actor.py:339-343).
#include "ptx.cuh"

namespace b200 {

constexpr int ROUTE_MAX_PER_LANE = 8;   // up to 256 experts

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int k, int norm_topk, float* __restrict__ probs,
                 float* __restrict__ weights, long long* __restrict__ experts, int* __restrict__ counts,
                 float* __restrict__ prob_sums) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float v[ROUTE_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
      const int e = lane + j * 32;
      v[j] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
      v[j] = (lane + j * 32) < E ? __expf(v[j] - mx) : 0.f;
      sum += v[j];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
      const int e = lane + j * 32;
      v[j] *= inv;
      if (e < E) {
        if (probs != nullptr) probs[(size_t)t * E + e] = v[j];
        if (prob_sums != nullptr) atomicAdd(prob_sums + e, v[j]);
      }
    }
    // k rounds of warp arg-max; ties go to the lower expert index (as torch.topk does for equal values in practice)
    float wsum = 0.f;
    float sel_w = 0.f;     // lane s (< k) keeps the s-th selection
    int sel_e = 0;
    for (int s = 0; s < k; ++s) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + j * 32;
        if (e < E && (v[j] > best || (v[j] == best && e < best_e))) { best = v[j]; best_e = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;      // remove the winner
      if (lane == s) { sel_w = best; sel_e = best_e; }
      wsum += best;
    }
    if (lane < k) {
      weights[(size_t)t * k + lane] = norm_topk ? sel_w / wsum : sel_w;
      experts[(size_t)t * k + lane] = sel_e;
      if (counts != nullptr) atomicAdd(counts + sel_e, 1);
    }
  }
}

}  // namespace b200

using namespace b200;

// logits fp32 [T, E] (E <= 256, k <= 32). probs [T, E], counts [E] and prob_sums [E] are optional (counts / prob_sums
// must be zeroed by the caller).
extern "C" int b200_moe_route(const float* logits, int T, int E, int k, int norm_topk, float* probs, float* weights,
                              long long* experts, int* counts, float* prob_sums, void* stream) {
  if (T <= 0) return 0;
  if (E > 32 * ROUTE_MAX_PER_LANE || k < 1 || k > 32 || k > E) return -10;
  const int blocks = (int)((((long long)T * 32 + 255) / 256) < 148 * 8 ? (((long long)T * 32 + 255) / 256) : 148 * 8);
  moe_route_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, T, E, k, norm_topk, probs, weights,
                                                                               experts, counts, prob_sums);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
