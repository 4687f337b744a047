// Token sampler for the rollout engine: temperature, top-k, top-p, an inverse-CDF draw (one Philox uniform per
// (seed, sequence, step)) and the log-prob of the drawn token under the processed distribution, one CTA per sequence.
// Stands in for vLLM's sampler as configured by the reference (SamplingParams with temperature / top_p / top_k and
// logprobs of the sampled token: openrlhf/trainer/ppo_utils/samples_generator.py:203-211,
// openrlhf/trainer/ray/vllm_engine.py:295-300 selects "processed_logprobs").
#include <curand_kernel.h>

#include "ptx.cuh"

namespace b200 {

constexpr int SAMPLE_THREADS = 1024;

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) {
    t = warp_max(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// e[k] = exp((z[j+k] - mx) * inv_t) if that value passes the keep threshold and j + k < end, else 0. j is a multiple
// of 8; one 16-byte load when the row is bf16 and 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load8_kept_exp(const T* z, int j, int end, float mx, float inv_t, float thr, bool vec,
                                               float* e) {
  float x[8];
  if (vec && j + 8 <= end) {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(z) + j);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __bfloat1622float2(h[q]);
      x[2 * q] = f.x;
      x[2 * q + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = (j + k < end) ? load_logit(z, j + k) : -INFINITY;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float v = (x[k] - mx) * inv_t;
    e[k] = (j + k < end && v >= thr) ? __expf(v) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const T* __restrict__ logits, int ld, int V, const float* __restrict__ temperature, float temp_scalar,
              int top_k, float top_p, unsigned long long seed, const long long* __restrict__ step_ptr,
              long long step_scalar, long long* __restrict__ out_tok, float* __restrict__ out_logp,
              const int* __restrict__ active, const int* __restrict__ top_k_rows,
              const float* __restrict__ top_p_rows) {
  __shared__ float red[32];
  __shared__ float s_best[32];
  __shared__ int s_idx[32];
  const int row = blockIdx.x;
  if (active != nullptr && active[row] == 0) return;
  // per-request nucleus settings (one value per row) take precedence over the launch-wide scalars
  if (top_k_rows != nullptr) top_k = top_k_rows[row];
  if (top_p_rows != nullptr) top_p = top_p_rows[row];
  const T* z = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : temp_scalar;
  const bool greedy = temp <= 1e-6f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  const long long step = step_ptr ? *step_ptr : step_scalar;

  float mx = -INFINITY;
  if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(z) & 15) == 0) {
    const int nvec = V >> 3;                       // 16-byte loads over the aligned part, scalar tail
    for (int i = threadIdx.x; i < nvec; i += SAMPLE_THREADS) {
      const uint4 u = reinterpret_cast<const uint4*>(z)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        mx = fmaxf(mx, fmaxf(f.x, f.y));
      }
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, load_logit(z, i));
  } else {
    for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, load_logit(z, i));
  }
  mx = block_reduce_max(mx, red);

  // threshold in x = (z - max) * inv_t space; keep x >= thr
  float thr = -INFINITY;
  if (!greedy && ((top_k > 0 && top_k < V) || top_p < 1.f)) {
    float lo_u = 0.f;  // keep-set threshold in u = exp(x) in [0, 1]
    if (top_k > 0 && top_k < V) {
      float lo = 0.f, hi = 1.f;
      for (int it = 0; it < 26; ++it) {
        const float mid = 0.5f * (lo + hi);
        float c = 0.f;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS)
          c += (__expf((load_logit(z, i) - mx) * inv_t) >= mid) ? 1.f : 0.f;
        c = block_reduce_sum(c, red);
        if (c >= (float)top_k) lo = mid; else hi = mid;
      }
      lo_u = lo;
    }
    if (top_p < 1.f) {
      float mass_all = 0.f;
      for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
        const float u = __expf((load_logit(z, i) - mx) * inv_t);
        mass_all += (u >= lo_u) ? u : 0.f;
      }
      mass_all = block_reduce_sum(mass_all, red);
      const float target = top_p * mass_all;
      float lo = lo_u, hi = 1.f;
      for (int it = 0; it < 26; ++it) {
        const float mid = 0.5f * (lo + hi);
        float m = 0.f;
        for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
          const float u = __expf((load_logit(z, i) - mx) * inv_t);
          m += (u >= mid) ? u : 0.f;
        }
        m = block_reduce_sum(m, red);
        if (m >= target) lo = mid; else hi = mid;
      }
      lo_u = lo;
    }
    thr = lo_u > 0.f ? __logf(lo_u) : -INFINITY;
  }

  if (!greedy) {
    // ---- inverse-CDF draw from the kept set: one uniform per (row, step). Warp w owns the contiguous vocabulary
    // segment [w*S, (w+1)*S); pass 1 gives every warp's probability mass, thread 0 picks the warp that holds the
    // target quantile, and that warp walks its segment once more with a running prefix sum.
    __shared__ float s_wsum[SAMPLE_THREADS / 32];
    __shared__ float s_resid, s_total;
    __shared__ int s_warp;
    constexpr int NW = SAMPLE_THREADS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = ((V + NW - 1) / NW + 255) / 256 * 256;
    const int seg0 = min(V, warp * S), seg1 = min(V, seg0 + S);
    const bool vec = sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(z) & 15) == 0;
    float acc = 0.f;
    for (int j = seg0 + lane * 8; j < seg1; j += 256) {
      float e[8];
      load8_kept_exp(z, j, seg1, mx, inv_t, thr, vec, e);
      acc += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
    }
    acc = warp_sum(acc);
    if (lane == 0) s_wsum[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int w = 0; w < NW; ++w) total += s_wsum[w];
      curandStatePhilox4_32_10_t rng;
      curand_init(seed, (unsigned long long)row, (unsigned long long)step, &rng);
      const float target = curand_uniform(&rng) * total;      // uniform in (0, 1]
      int sel = -1, last = 0;
      float pre = 0.f;
      for (int w = 0; w < NW; ++w) {
        if (s_wsum[w] > 0.f) {
          last = w;
          if (sel < 0 && pre + s_wsum[w] >= target) { sel = w; s_resid = target - pre; }
        }
        pre += s_wsum[w];
      }
      if (sel < 0) { sel = last; s_resid = s_wsum[last]; }     // rounding: the quantile fell past the last mass
      s_warp = sel;
      s_total = total;
    }
    __syncthreads();
    if (warp == s_warp) {
      float resid = s_resid;
      int chosen = -1, last_kept = -1;
      for (int j0 = seg0; j0 < seg1 && chosen < 0; j0 += 256) {
        const int j = j0 + lane * 8;
        float e[8];
        if (j < seg1) {
          load8_kept_exp(z, j, seg1, mx, inv_t, thr, vec, e);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) e[k] = 0.f;
        }
        int lk = -1;
        float ls = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          ls += e[k];
          if (e[k] > 0.f) lk = j + k;
        }
        float cum = ls;                                        // inclusive prefix over lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, cum, o);
          if (lane >= o) cum += t;
        }
        const float tot = __shfl_sync(0xffffffffu, cum, 31);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
        last_kept = max(last_kept, lk);
        if (tot > 0.f && resid <= tot) {
          const unsigned m = __ballot_sync(0xffffffffu, ls > 0.f && cum >= resid);
          if (m != 0) {
            const int src = __ffs(m) - 1;
            int pick = -1;
            if (lane == src) {
              const float r = resid - (cum - ls);
              float c = 0.f;
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                c += e[k];
                if (e[k] > 0.f) {
                  if (pick < 0 || c - e[k] < r) pick = j + k;   // last kept element whose prefix starts below r
                }
              }
            }
            chosen = __shfl_sync(0xffffffffu, pick, src);
          }
        }
        if (chosen < 0) resid -= tot;
      }
      if (chosen < 0) chosen = max(last_kept, 0);
      if (lane == 0) {
        out_tok[row] = chosen;
        if (out_logp) out_logp[row] = (load_logit(z, chosen) - mx) * inv_t - __logf(s_total);
      }
    }
    return;
  }
  // ---- greedy: arg-max of the logits; the reported log-prob is under temperature 1
  float sum = 0.f, best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float x = (load_logit(z, i) - mx) * inv_t;
    sum += __expf(x);
    if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
  }
  sum = block_reduce_sum(sum, red);
  // argmax over the block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_best[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = s_best[threadIdx.x];
    best_i = s_idx[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    if (threadIdx.x == 0) {
      out_tok[row] = best_i;
      if (out_logp) {
        // greedy reports the log-prob under temperature 1 (sum was computed with inv_t = 1 in that case)
        out_logp[row] = (load_logit(z, best_i) - mx) * inv_t - __logf(sum);
      }
    }
  }
}

// Log-prob of given tokens under softmax(logits / T): out[t] = z[t, y_t]/T - logsumexp(z[t,:]/T), and optionally the
// entropy of softmax(z) (untempered, as in openrlhf/models/actor.py:269-285). One CTA per row.
template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
logprob_rows_kernel(const T* __restrict__ logits, int ld, int V, const long long* __restrict__ labels, float inv_t,
                    float* __restrict__ out_logp, float* __restrict__ out_entropy, float* __restrict__ out_lse) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* z = logits + (size_t)row * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) mx = fmaxf(mx, load_logit(z, i));
  mx = block_reduce_max(mx, red);
  float s = 0.f, s1 = 0.f, sz = 0.f;
  for (int i = threadIdx.x; i < V; i += SAMPLE_THREADS) {
    const float v = load_logit(z, i) - mx;
    s += __expf(v * inv_t);
    if (out_entropy) {
      const float e = __expf(v);
      s1 += e;
      sz += e * v;
    }
  }
  s = block_reduce_sum(s, red);
  if (out_entropy) {
    s1 = block_reduce_sum(s1, red);
    sz = block_reduce_sum(sz, red);
  }
  if (threadIdx.x == 0) {
    long long y = labels[row];
    y = y < 0 ? 0 : (y >= V ? V - 1 : y);
    out_logp[row] = (load_logit(z, (int)y) - mx) * inv_t - __logf(s);
    if (out_lse) out_lse[row] = mx * inv_t + __logf(s);
    if (out_entropy) out_entropy[row] = __logf(s1) - sz / s1;
  }
}


// In place on bf16 logits: z <- g * inv_t * (onehot(label) - softmax(z * inv_t)); lse = logsumexp(z * inv_t) per row.
__global__ void __launch_bounds__(256)
logprob_bwd_rows_kernel(__nv_bfloat16* __restrict__ logits, int T, int V, int ld, const long long* __restrict__ labels,
                        const float* __restrict__ lse_in, const float* __restrict__ dlogp, float inv_t) {
  const int nvec = V >> 3;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    const long long y = labels[t];      // outside [0, V): no one-hot term in this row (vocabulary-parallel shards)
    __nv_bfloat16* row = logits + (size_t)t * ld;
    const float lse = lse_in[t];
    const float g = dlogp[t] * inv_t;
    uint4 u = reinterpret_cast<uint4*>(row)[v];
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
    float o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h2[i]);
      o[2 * i] = -g * __expf(f.x * inv_t - lse);
      o[2 * i + 1] = -g * __expf(f.y * inv_t - lse);
    }
    const int c0 = v * 8;
    if (y >= c0 && y < c0 + 8) o[y - c0] += g;
    uint4 w;
    w.x = pack_bf16x2(o[0], o[1]); w.y = pack_bf16x2(o[2], o[3]); w.z = pack_bf16x2(o[4], o[5]); w.w = pack_bf16x2(o[6], o[7]);
    reinterpret_cast<uint4*>(row)[v] = w;
  }
}


// One decode step's bookkeeping for all batch rows in one launch (replaces ~35 small elementwise launches per step):
// append the sampled token and its log-prob, detect EOS / length stops, advance position and context length, and
// compute the KV slot of the next token from the block table.
__global__ void decode_advance_kernel(int B, const long long* __restrict__ next_tok, const float* __restrict__ next_lp,
                                      long long* __restrict__ tok, int* __restrict__ pos, int* __restrict__ seq_lens,
                                      int* __restrict__ slots, int* __restrict__ active, int* __restrict__ gen_count,
                                      long long* __restrict__ out_tokens, float* __restrict__ out_logprobs, int out_ld,
                                      const int* __restrict__ min_tok, const int* __restrict__ max_tok,
                                      const unsigned char* __restrict__ ignore_eos, long long eos,
                                      const int* __restrict__ block_table, int max_pages, int page_size,
                                      long long* __restrict__ step_counter) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r == 0) *step_counter += 1;
  if (r >= B) return;
  const bool act = active[r] != 0;
  int p = pos[r];
  if (act) {
    const long long nt = next_tok[r];
    const int g = min(gen_count[r], out_ld - 1);
    out_tokens[(size_t)r * out_ld + g] = nt;
    out_logprobs[(size_t)r * out_ld + g] = next_lp[r];
    const int gc = gen_count[r] + 1;
    gen_count[r] = gc;
    const bool hit_eos = nt == eos && !ignore_eos[r] && gc >= min_tok[r];
    const bool still = !(hit_eos || gc >= max_tok[r]);
    tok[r] = nt;
    if (still) {
      p += 1;
      pos[r] = p;
      seq_lens[r] += 1;
    }
    active[r] = still ? 1 : 0;
  }
  const int page = block_table[(size_t)r * max_pages + min(p / page_size, max_pages - 1)];
  slots[r] = page * page_size + p % page_size;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_sample(const void* logits, int is_bf16, int B, int V, int ld, const float* temperature,
                           float temp_scalar, int top_k, float top_p, unsigned long long seed,
                           const long long* step_ptr, long long step_scalar, long long* out_tok, float* out_logp,
                           const int* active, const int* top_k_rows, const float* top_p_rows, void* stream_) {
  if (B <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, SAMPLE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, V, temperature,
                                                               temp_scalar, top_k, top_p, seed, step_ptr, step_scalar,
                                                               out_tok, out_logp, active, top_k_rows, top_p_rows);
  else
    sample_kernel<float><<<B, SAMPLE_THREADS, 0, st>>>((const float*)logits, ld, V, temperature, temp_scalar, top_k,
                                                       top_p, seed, step_ptr, step_scalar, out_tok, out_logp, active,
                                                       top_k_rows, top_p_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_logprob_rows(const void* logits, int is_bf16, int T, int V, int ld, const long long* labels,
                                 float temperature, float* out_logp, float* out_entropy, float* out_lse, void* stream_) {
  if (T <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  const float inv_t = 1.f / temperature;
  if (is_bf16)
    logprob_rows_kernel<__nv_bfloat16><<<T, SAMPLE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, ld, V, labels, inv_t,
                                                                     out_logp, out_entropy, out_lse);
  else
    logprob_rows_kernel<float><<<T, SAMPLE_THREADS, 0, st>>>((const float*)logits, ld, V, labels, inv_t, out_logp,
                                                             out_entropy, out_lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_logprob_bwd_rows(void* logits, int T, int V, int ld, const long long* labels, const float* lse,
                                     const float* dlogp, float inv_t, void* stream_) {
  if (T <= 0) return 0;
  if (V % 8 || ld % 8) return -10;
  long long work = (long long)T * (V / 8);
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  logprob_bwd_rows_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (__nv_bfloat16*)logits, T, V, ld, labels, lse, dlogp, inv_t);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_decode_advance(int B, const long long* next_tok, const float* next_lp, long long* tok, int* pos,
                                   int* seq_lens, int* slots, int* active, int* gen_count, long long* out_tokens,
                                   float* out_logprobs, int out_ld, const int* min_tok, const int* max_tok,
                                   const void* ignore_eos, long long eos, const int* block_table, int max_pages,
                                   int page_size, long long* step_counter, void* stream_) {
  if (B <= 0) return 0;
  decode_advance_kernel<<<(B + 127) / 128, 128, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      B, next_tok, next_lp, tok, pos, seq_lens, slots, active, gen_count, out_tokens, out_logprobs, out_ld, min_tok,
      max_tok, reinterpret_cast<const unsigned char*>(ignore_eos), eos, block_table, max_pages, page_size, step_counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
