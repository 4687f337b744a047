// RL-specific fused kernels: PPO clipped policy loss (+KL penalty, importance-sampling correction, metrics and the
// gradient w.r.t. the log-probs in one pass), clipped value loss, reward shaping + GAE / discounted returns,
// masked whitening. They replace the chains of small PyTorch ops in the reference's
// openrlhf/models/loss.py:116-269, openrlhf/models/utils.py:64-126 and the Python loops over the response length in
// openrlhf/trainer/ppo_utils/experience_maker.py:332-411.
#include "ptx.cuh"

namespace b200 {

template <int THREADS>
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

struct PpoParams {
  const float* logp;       // [N] new log-probs
  const float* old_logp;   // [N]
  const float* adv;        // [N]
  const float* weight;     // [N] aggregation weight of each token (mask / normaliser), 0 on padding
  const float* mask;       // [N] 0/1 action mask (for the metrics)
  const float* ref_logp;   // [N] or null: reference log-probs for the KL loss term
  const float* roll_logp;  // [N] or null: rollout-engine log-probs (importance-sampling correction, vllm_kl metric)
  float* dlogp;            // [N] gradient of the total loss w.r.t. logp
  float* acc;              // [8]: policy_loss, kl_loss, clip_cnt, ppo_kl_sum, vllm_kl_sum, mask_sum, kl_masked_sum, -
  long long n;
  float eps_low, eps_high, dual_clip;  // dual_clip <= 1 disables
  float kl_coef;
  int kl_estimator;  // 1,2,3
  int is_mode;       // 0 none, 1 tis (clamp), 2 icepop (zero outside)
  float is_lo, is_hi;
};

__global__ void __launch_bounds__(256) ppo_loss_kernel(const PpoParams p) {
  __shared__ float red[32];
  float a_loss = 0.f, a_kl = 0.f, a_clip = 0.f, a_pkl = 0.f, a_vkl = 0.f, a_mask = 0.f, a_klm = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.n; i += (long long)gridDim.x * blockDim.x) {
    const float w = p.weight[i];
    const float mk = p.mask[i];
    const float lp = p.logp[i], old = p.old_logp[i], A = p.adv[i];
    const float lr_raw = lp - old;
    const float lr = fminf(fmaxf(lr_raw, -20.f), 20.f);
    const float ratio = __expf(lr);
    const float dratio = (lr_raw > -20.f && lr_raw < 20.f) ? ratio : 0.f;
    const float lo = 1.f - p.eps_low, hi = 1.f + p.eps_high;
    const float rc = fminf(fmaxf(ratio, lo), hi);
    const float s1 = ratio * A, s2 = rc * A;
    float loss, g;  // loss = -min(s1, s2); g = dloss/dlogp
    if (s1 <= s2) {
      loss = -s1;
      g = -A * dratio;
    } else {
      loss = -s2;
      g = (ratio >= lo && ratio <= hi) ? -A * dratio : 0.f;
    }
    if (p.dual_clip > 1.f && A < 0.f) {
      const float floor_v = p.dual_clip * A;  // negative
      if (-loss < floor_v) {                  // min(s1,s2) < c*A  ->  loss = -c*A, no gradient
        loss = -floor_v;
        g = 0.f;
      }
    }
    float isw = 1.f;
    float vkl = 0.f;
    if (p.roll_logp != nullptr) {
      const float d = old - p.roll_logp[i];
      vkl = -d;  // rollout - old
      if (p.is_mode != 0) {
        const float wr = __expf(d);
        if (p.is_mode == 1) isw = fminf(fmaxf(wr, p.is_lo), p.is_hi);
        else isw = (wr >= p.is_lo && wr <= p.is_hi) ? wr : 0.f;
      }
    }
    loss *= isw;
    g *= isw;
    float kl = 0.f, gkl = 0.f;
    if (p.ref_logp != nullptr) {
      const float d = lp - p.ref_logp[i];
      if (p.kl_estimator == 1) { kl = d; gkl = 1.f; }
      else if (p.kl_estimator == 2) { kl = 0.5f * d * d; gkl = d; }
      else { const float e = __expf(-d); kl = e - 1.f + d; gkl = 1.f - e; }
      if (kl > 10.f) { kl = 10.f; gkl = 0.f; }
      if (kl < -10.f) { kl = -10.f; gkl = 0.f; }
    }
    p.dlogp[i] = w * (g + p.kl_coef * gkl);
    a_loss += w * loss;
    a_kl += w * kl;
    a_clip += (s2 < s1) ? mk : 0.f;
    a_pkl += -lr_raw * mk;
    a_vkl += vkl * mk;
    a_mask += mk;
    a_klm += kl * mk;
  }
  float v[7] = {a_loss, a_kl, a_clip, a_pkl, a_vkl, a_mask, a_klm};
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    float s = block_sum_f<256>(v[k], red);
    if (threadIdx.x == 0) atomicAdd(p.acc + k, s);
  }
}

// Clipped value loss: 0.5 * sum w * max((clip(v, old +- eps) - R)^2, (v - R)^2); eps <= 0 disables clipping.
__global__ void __launch_bounds__(256)
value_loss_kernel(const float* __restrict__ values, const float* __restrict__ old_values,
                  const float* __restrict__ returns, const float* __restrict__ weight, float* __restrict__ dvalues,
                  float* __restrict__ acc, long long n, float clip_eps) {
  __shared__ float red[32];
  float a = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = values[i], R = returns[i], w = weight[i];
    float loss = (v - R) * (v - R), g = 2.f * (v - R);
    if (clip_eps > 0.f) {
      const float ov = old_values[i];
      const float vc = ov + fminf(fmaxf(v - ov, -clip_eps), clip_eps);
      const float lc = (vc - R) * (vc - R);
      if (lc > loss) {
        loss = lc;
        g = (v - ov > -clip_eps && v - ov < clip_eps) ? 2.f * (vc - R) : 0.f;
      } else if (lc == loss) {
        g = 0.5f * g + 0.5f * ((v - ov > -clip_eps && v - ov < clip_eps) ? 2.f * (vc - R) : 0.f);
      }
    }
    dvalues[i] = 0.5f * w * g;
    a += 0.5f * w * loss;
  }
  a = block_sum_f<256>(a, red);
  if (threadIdx.x == 0) atomicAdd(acc, a);
}

// Reward shaping + GAE or discounted returns; one warp per sequence, reverse scan in chunks of 32.
//   reward_t = -beta * kl_t (+ clamp(r) at the last action position); masked by action_mask
//   gae:      delta_t = r_t + gamma V_{t+1} - V_t; A_t = delta_t + gamma*lambda A_{t+1}; returns = A + V
//   otherwise R_t = r_t + gamma R_{t+1}; advantages = returns
__global__ void __launch_bounds__(128)
gae_kernel(const float* __restrict__ values /*null -> cumulative returns*/, const float* __restrict__ kl /*or null*/,
           const float* __restrict__ seq_reward, const float* __restrict__ mask, float* __restrict__ adv,
           float* __restrict__ ret, float* __restrict__ reward_sum, int B, int A, float beta, float gamma, float lambd,
           float clip_lo, float clip_hi) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const float* mk = mask + (size_t)warp * A;
  // last action index
  int last = -1;
  for (int base = 0; base < A; base += 32) {
    int t = base + lane;
    int cand = (t < A && mk[t] != 0.f) ? t : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = max(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    last = max(last, cand);
  }
  const float r_seq = fminf(fmaxf(seq_reward[warp], clip_lo), clip_hi);
  const bool gae = values != nullptr;
  const float c = gae ? gamma * lambd : gamma;
  float cpow[6];  // c^(1,2,4,8,16,32)
  cpow[0] = c;
#pragma unroll
  for (int k = 1; k < 6; ++k) cpow[k] = cpow[k - 1] * cpow[k - 1];
  float carry = 0.f;      // A_{t+1} (or R_{t+1}) entering the chunk from the right
  float v_next_carry = 0.f;
  float rsum = 0.f;
  const int nchunks = (A + 31) / 32;
  for (int ch = nchunks - 1; ch >= 0; --ch) {
    const int t = ch * 32 + lane;
    const bool in = t < A;
    const float m = in ? mk[t] : 0.f;
    float r = 0.f;
    if (in) {
      r = (kl ? -beta * kl[(size_t)warp * A + t] : 0.f) + (t == last ? r_seq : 0.f);
      r *= m;
    }
    rsum += r;
    float x;
    if (gae) {
      const float v = in ? values[(size_t)warp * A + t] * m : 0.f;
      float vn = __shfl_down_sync(0xffffffffu, v, 1);
      if (lane == 31) vn = v_next_carry;
      x = r + gamma * vn - v;
      v_next_carry = __shfl_sync(0xffffffffu, v, 0);
    } else {
      x = r;
    }
    // suffix scan: x_j <- x_j + c^d * x_{j+d}
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      const int d = 1 << k;
      float y = __shfl_down_sync(0xffffffffu, x, d);
      if (lane + d < 32) x += cpow[k] * y;
    }
    // carry from the chunk to the right: c^(32-lane) * carry
    float cp = 1.f;
    {
      int e = 32 - lane;
#pragma unroll
      for (int k = 0; k < 6; ++k)
        if (e & (1 << k)) cp *= cpow[k];
    }
    x += cp * carry;
    carry = __shfl_sync(0xffffffffu, x, 0);
    if (in) {
      if (gae) {
        const float v = values[(size_t)warp * A + t] * m;
        adv[(size_t)warp * A + t] = x;
        ret[(size_t)warp * A + t] = x + v;
      } else {
        adv[(size_t)warp * A + t] = x;
        ret[(size_t)warp * A + t] = x;
      }
    }
  }
  rsum = warp_sum(rsum);
  if (lane == 0 && reward_sum) reward_sum[warp] = rsum;
}

// Masked statistics: acc[0] += sum(x*m), acc[1] += sum(x*x*m), acc[2] += sum(m)
__global__ void __launch_bounds__(256)
masked_stats_kernel(const float* __restrict__ x, const float* __restrict__ m, long long n, float* __restrict__ acc) {
  __shared__ float red[32];
  float s = 0.f, ss = 0.f, cnt = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float mk = m[i], v = x[i];
    s += v * mk;
    ss += v * v * mk;
    cnt += mk;
  }
  s = block_sum_f<256>(s, red);
  ss = block_sum_f<256>(ss, red);
  cnt = block_sum_f<256>(cnt, red);
  if (threadIdx.x == 0) {
    atomicAdd(acc, s);
    atomicAdd(acc + 1, ss);
    atomicAdd(acc + 2, cnt);
  }
}
// x <- (x - mean) * rsqrt(max(var, 1e-8)) with mean/var from acc (biased, over masked entries); std_norm=0 keeps only
// the mean subtraction (openrlhf/trainer/ppo_utils/experience_maker.py:314-328).
__global__ void whiten_apply_kernel(float* __restrict__ x, long long n, const float* __restrict__ acc, int std_norm) {
  const float cnt = fmaxf(acc[2], 1.f);
  const float mean = acc[0] / cnt;
  const float var = fmaxf(acc[1] / cnt - mean * mean, 0.f);
  const float rs = std_norm ? rsqrtf(fmaxf(var, 1e-8f)) : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = (x[i] - mean) * rs;
}

static inline int grid_for(long long work, int threads, int cap = 148 * 4) {
  long long b = (work + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace b200

using namespace b200;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -3)

extern "C" int b200_ppo_loss(const float* logp, const float* old_logp, const float* adv, const float* weight,
                             const float* mask, const float* ref_logp, const float* roll_logp, float* dlogp,
                             float* acc, long long n, float eps_low, float eps_high, float dual_clip, float kl_coef,
                             int kl_estimator, int is_mode, float is_lo, float is_hi, void* stream) {
  if (n <= 0) return 0;
  PpoParams p{logp, old_logp, adv, weight, mask, ref_logp, roll_logp, dlogp, acc, n, eps_low, eps_high, dual_clip,
              kl_coef, kl_estimator, is_mode, is_lo, is_hi};
  ppo_loss_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(p);
  return LAUNCH_OK();
}
extern "C" int b200_value_loss(const float* values, const float* old_values, const float* returns,
                               const float* weight, float* dvalues, float* acc, long long n, float clip_eps,
                               void* stream) {
  if (n <= 0) return 0;
  value_loss_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(values, old_values, returns, weight, dvalues, acc, n,
                                                                  clip_eps);
  return LAUNCH_OK();
}
extern "C" int b200_gae(const float* values, const float* kl, const float* seq_reward, const float* mask, float* adv,
                        float* ret, float* reward_sum, int B, int A, float beta, float gamma, float lambd,
                        float clip_lo, float clip_hi, void* stream) {
  if (B <= 0 || A <= 0) return 0;
  const int warps_per_block = 4;
  gae_kernel<<<(B + warps_per_block - 1) / warps_per_block, 128, 0, STREAM(stream)>>>(
      values, kl, seq_reward, mask, adv, ret, reward_sum, B, A, beta, gamma, lambd, clip_lo, clip_hi);
  return LAUNCH_OK();
}
extern "C" int b200_masked_stats(const float* x, const float* m, long long n, float* acc, void* stream) {
  if (n <= 0) return 0;
  masked_stats_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(x, m, n, acc);
  return LAUNCH_OK();
}
extern "C" int b200_whiten_apply(float* x, long long n, const float* acc, int std_norm, void* stream) {
  if (n <= 0) return 0;
  whiten_apply_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(x, n, acc, std_norm);
  return LAUNCH_OK();
}
