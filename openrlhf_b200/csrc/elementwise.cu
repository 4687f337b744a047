// Memory-bound transformer ops for packed token streams: RMSNorm, RoPE, SwiGLU, embedding, fused AdamW.
// All kernels use 128-bit accesses and fp32 arithmetic; hidden sizes must be multiples of 8.
// They stand in for the PyTorch elementwise kernels HF Transformers launches under the reference
// (RMSNorm / rotary / MLP activation of transformers' Llama and Qwen2 blocks, nn.Embedding) and for
// DeepSpeed FusedAdam (openrlhf/utils/deepspeed/deepspeed.py:295-429 builds the optimizer).
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace b200 {

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
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

// ------------------------------------------------------------------ RMSNorm
// y = bf16(bf16(x * rstd) * w): same rounding points as the HF modules (normalise in fp32, cast, scale).
// Optional fused residual add: if `res` is given, h = x + res is written to `h_out` and normalised.
constexpr int NORM_THREADS = 256;
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int T, int H, int ldx, int ldy,
                   float eps) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  extern __shared__ uint4 row_cache[];  // H/8 vectors
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * ldx) : nullptr;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      uint4 u = xr[v];
      float f[8];
      unpack8(u, f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i] + g[i]);
        u = pack8(f);
        reinterpret_cast<uint4*>(h_out + (size_t)row * ldx)[v] = u;
      }
      row_cache[v] = u;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum<NORM_THREADS>(ss, red);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float f[8], g[8];
      unpack8(row_cache[v], f);
      unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i] * rstd) * g[i];
      yr[v] = pack8(f);
    }
    __syncthreads();
  }
}

// Warp-per-row variant for H <= 32 * 8 * MAXV: the row stays in registers, the reduction is a shuffle, and a warp has
// all of its row's loads in flight at once (one CTA per row with a block-wide reduction left too few bytes in flight
// per SM to approach the HBM rate).
template <int MAXV>
__global__ void __launch_bounds__(512)
rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                        __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int T, int H, int ldx, int ldy,
                        float eps) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  const int nvec = H >> 3;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < T; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * ldx) : nullptr;
    uint4 c[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) c[i] = xr[v];
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float f[8];
        unpack8(c[i], f);
        if (rr) {
          float g[8];
          unpack8(rr[v], g);
#pragma unroll
          for (int q = 0; q < 8; ++q) f[q] = round_bf16(f[q] + g[q]);
          c[i] = pack8(f);
          reinterpret_cast<uint4*>(h_out + (size_t)row * ldx)[v] = c[i];
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += f[q] * f[q];
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float f[8], g[8];
        unpack8(c[i], f);
        unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] = round_bf16(f[q] * rstd) * g[q];
        yr[v] = pack8(f);
      }
    }
  }
}

// Backward, warp per row (H <= 2048): x and dy of the row stay in registers between the dot product and the dx pass,
// each lane accumulates the weight gradient of its own columns in registers over all of the warp's rows; the CTA's
// warps are summed in shared memory and one atomic per column and CTA reaches the fp32 gradient.
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                        const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw, int T, int H) {
  extern __shared__ float dw_acc[];  // H floats
  const int nvec = H >> 3;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dw_acc[i] = 0.f;
  __syncthreads();
  float acc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[i][q] = 0.f;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < T; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    uint4 cx[MAXV], cd[MAXV];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        cx[i] = xr[v];
        cd[i] = dyr[v];
      }
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float fx[8], fd[8], fw[8];
        unpack8(cx[i], fx);
        unpack8(cd[i], fd);
        unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
#pragma unroll
        for (int q = 0; q < 8; ++q) dot += fd[q] * fw[q] * fx[q];
      }
    }
    dot = warp_sum(dot);
    const float cc = dot * rstd * rstd * rstd / (float)H;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float fx[8], fd[8], fw[8], o[8];
        unpack8(cx[i], fx);
        unpack8(cd[i], fd);
        unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
        if (dres_in) unpack8(reinterpret_cast<const uint4*>(dres_in + (size_t)row * H)[v], o);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float g = fd[q] * fw[q] * rstd - fx[q] * cc;
          o[q] = dres_in ? o[q] + g : g;
          acc[i][q] += fd[q] * round_bf16(fx[q] * rstd);
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * H)[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
#pragma unroll
      for (int q = 0; q < 8; ++q) atomicAdd(&dw_acc[v * 8 + q], acc[i][q]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) atomicAdd(dw + i, dw_acc[i]);
}

// dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x)  (+ dres_in);  dw += sum_rows dy * (x*rstd)
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw, int T, int H) {
  extern __shared__ float dw_acc[];  // H floats
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int i = threadIdx.x; i < H; i += NORM_THREADS) dw_acc[i] = 0.f;
  __syncthreads();
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float fx[8], fd[8], fw[8];
      unpack8(xr[v], fx);
      unpack8(dyr[v], fd);
      unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += fd[i] * fw[i] * fx[i];
    }
    dot = block_sum<NORM_THREADS>(dot, red);
    const float c = dot * rstd * rstd * rstd / (float)H;
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float fx[8], fd[8], fw[8], o[8];
      unpack8(xr[v], fx);
      unpack8(dyr[v], fd);
      unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
      if (dres_in) unpack8(reinterpret_cast<const uint4*>(dres_in + (size_t)row * H)[v], o);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float g = fd[i] * fw[i] * rstd - fx[i] * c;
        o[i] = dres_in ? o[i] + g : g;
        dw_acc[v * 8 + i] += fd[i] * round_bf16(fx[i] * rstd);  // each (v,i) is owned by one thread
      }
      reinterpret_cast<uint4*>(dx + (size_t)row * H)[v] = pack8(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += NORM_THREADS) atomicAdd(dw + i, dw_acc[i]);
}

// ------------------------------------------------------------------ RoPE (rotate-half layout), in place
// qkv: [T, ld] with q heads then k heads at the start of each row; head_dim = 2*half. cos_sin: [max_pos, half] float2.
// sign = +1 forward, -1 backward (the transpose of a rotation is the rotation by the negative angle).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                            const float2* __restrict__ cos_sin, int T, int n_heads, int half, int ld, float sign,
                            int max_pos) {
  const int pairs_per_row = n_heads * half;
  const long long total = (long long)T * pairs_per_row / 2;  // two adjacent pairs per thread
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / (pairs_per_row / 2));
    const int r = (int)(idx % (pairs_per_row / 2)) * 2;
    const int head = r / half, i = r % half;
    int p = pos[t];
    p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
    __nv_bfloat16* base = qkv + (size_t)t * ld + head * 2 * half;
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(base + i);
    __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(base + i + half);
    const float2 cs0 = cos_sin[(size_t)p * half + i], cs1 = cos_sin[(size_t)p * half + i + 1];
    float2 l = __bfloat1622float2(lo), h = __bfloat1622float2(hi);
    float2 ol, oh;
    ol.x = l.x * cs0.x - sign * h.x * cs0.y;
    oh.x = h.x * cs0.x + sign * l.x * cs0.y;
    ol.y = l.y * cs1.x - sign * h.y * cs1.y;
    oh.y = h.y * cs1.x + sign * l.y * cs1.y;
    *reinterpret_cast<__nv_bfloat162*>(base + i) = __floats2bfloat162_rn(ol.x, ol.y);
    *reinterpret_cast<__nv_bfloat162*>(base + i + half) = __floats2bfloat162_rn(oh.x, oh.y);
  }
}

// ------------------------------------------------------------------ SwiGLU: y = silu(g) * u, gu = [g | u]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long long T,
                                  int F) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  const int nvec = F >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = (int)(idx % nvec);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8];
    unpack8(row[v], g);
    unpack8(row[nvec + v], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
    reinterpret_cast<uint4*>(y + t * F)[v] = pack8(g);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int nvec = F >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int v = (int)(idx % nvec);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[v], g);
    unpack8(row[nvec + v], u);
    unpack8(reinterpret_cast<const uint4*>(dy + t * F)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = 1.f / (1.f + __expf(-g[i]));
      du[i] = d[i] * g[i] * s;
      dg[i] = d[i] * u[i] * s * (1.f + g[i] * (1.f - s));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * F);
    orow[v] = pack8(dg);
    orow[nvec + v] = pack8(du);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int V) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  const int nvec = H >> 3;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    reinterpret_cast<uint4*>(out + (size_t)t * H)[v] = reinterpret_cast<const uint4*>(table + (size_t)id * H)[v];
  }
}
// grad_table (fp32) += scatter of dout rows.
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ grad_table, int T, int H, int V) {
  const int nvec = H >> 3;
  const long long total = (long long)T * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / nvec), v = (int)(idx % nvec);
    long long id = ids[t];
    if (id < 0 || id >= V) continue;
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(dout + (size_t)t * H)[v], f);
    float* g = grad_table + (size_t)id * H + v * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) atomicAdd(g + i, f[i]);
  }
}

// ------------------------------------------------------------------ optimizer
// Sum of squares of an fp32 buffer, accumulated into *out (caller zeroes it).
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n4 << 2; i < n; ++i) s += g[i] * g[i];
  s = block_sum<256>(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}
// scalars[0] = sum of squares (all ranks) -> scalars[1] = grad norm, scalars[2] = clip coefficient * grad_scale
__global__ void clip_coef_kernel(float* scalars, float max_norm, float grad_scale) {
  const float norm = sqrtf(scalars[0]) * grad_scale;
  scalars[1] = norm;
  float c = (max_norm > 0.f && norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.f;
  if (!isfinite(norm)) c = 0.f;
  scalars[2] = c * grad_scale;
}
// AdamW on fp32 master weights; writes the bf16 working copy; optionally zeroes the gradient.
// scale_ptr (device) multiplies the gradient (clip coefficient x 1/accumulation); step sizes come precomputed.
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                             const float* __restrict__ scale_ptr, float lr, float beta1, float beta2, float eps,
                             float wd, float bc1, float bc2, int zero_grad) {
  const float gs = scale_ptr ? *scale_ptr : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float g = grad[i] * gs;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi / bc2) + eps;
    p = p * (1.f - lr * wd) - lr * (mi / bc1) / denom;
    master[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(p);
    if (zero_grad) grad[i] = 0.f;
  }
}
// dst = beta * dst + (1 - beta) * src (EMA of the policy: openrlhf/utils/deepspeed/deepspeed.py:503-517)
__global__ void ema_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n, float beta) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = beta * dst[i] + (1.f - beta) * src[i];
}
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

static inline int grid_for(long long work, int threads, int cap = 148 * 8) {
  long long b = (work + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace b200

using namespace b200;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? 0 : -3)

extern "C" int b200_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                                int T, int H, int ldx, int ldy, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || ldx % 8 || ldy % 8 || H > 16384) return -10;
  if (H <= 32 * 8 * 24 && T >= 512) {
    // warp per row, 16 rows per CTA, two CTAs per SM in flight
    const int ctas = (T + 15) / 16 < 148 * 2 ? (T + 15) / 16 : 148 * 2;
#define B200_NORM_FWD(MAXV_)                                                                                      \
    return launch_pdl(rmsnorm_fwd_warp_kernel<MAXV_>, dim3(ctas), dim3(512), (size_t)0, STREAM(stream),            \
                      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,                 \
                      (__nv_bfloat16*)y, (__nv_bfloat16*)h_out, rstd, T, H, ldx, ldy, eps) == cudaSuccess ? 0 : -3;
    if (H <= 32 * 8 * 8) { B200_NORM_FWD(8) }
    if (H <= 32 * 8 * 16) { B200_NORM_FWD(16) }
    B200_NORM_FWD(24)
#undef B200_NORM_FWD
  }
  int grid = T < 148 * 8 ? T : 148 * 8;
  return launch_pdl(rmsnorm_fwd_kernel, dim3(grid), dim3(NORM_THREADS), (size_t)(H / 8) * sizeof(uint4), STREAM(stream),
                    (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                    (__nv_bfloat16*)h_out, rstd, T, H, ldx, ldy, eps) == cudaSuccess ? 0 : -3;
}
extern "C" int b200_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres_in,
                                void* dx, float* dw, int T, int H, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 || H > 11264) return -10;
  if (H <= 32 * 8 * 8 && T >= 512) {
    const int ctas = (T + 7) / 8 < 148 ? (T + 7) / 8 : 148;   // 254 registers per thread: one CTA per SM
    rmsnorm_bwd_warp_kernel<8><<<ctas, 256, H * sizeof(float), STREAM(stream)>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (const __nv_bfloat16*)dres_in,
        (__nv_bfloat16*)dx, dw, T, H);
    return LAUNCH_OK();
  }
  int grid = T < 148 * 2 ? T : 148 * 2;
  rmsnorm_bwd_kernel<<<grid, NORM_THREADS, H * sizeof(float), STREAM(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (const __nv_bfloat16*)dres_in,
      (__nv_bfloat16*)dx, dw, T, H);
  return LAUNCH_OK();
}
extern "C" int b200_rope(void* qkv, const int* pos, const void* cos_sin, int T, int n_heads, int head_dim, int ld,
                         float sign, int max_pos, void* stream) {
  if (T <= 0) return 0;
  if (head_dim % 4 || ld % 2) return -10;
  long long work = (long long)T * n_heads * (head_dim / 2) / 2;
  rope_kernel<<<grid_for(work, 256), 256, 0, STREAM(stream)>>>((__nv_bfloat16*)qkv, pos, (const float2*)cos_sin, T,
                                                               n_heads, head_dim / 2, ld, sign, max_pos);
  return LAUNCH_OK();
}
extern "C" int b200_swiglu_fwd(const void* gu, void* y, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  return launch_pdl(swiglu_fwd_kernel, dim3(grid_for(T * (F / 8), 256, 148 * 16)), dim3(256), (size_t)0, STREAM(stream),
                    (const __nv_bfloat16*)gu, (__nv_bfloat16*)y, T, F) == cudaSuccess ? 0 : -3;
}
extern "C" int b200_swiglu_bwd(const void* gu, const void* dy, void* dgu, long long T, int F, void* stream) {
  if (T <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256, 148 * 16), 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dgu, T, F);
  return LAUNCH_OK();
}
extern "C" int b200_embedding_fwd(const long long* ids, const void* table, void* out, int T, int H, int V,
                                  void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  return launch_pdl(embedding_fwd_kernel, dim3(grid_for((long long)T * (H / 8), 256, 148 * 16)), dim3(256), (size_t)0,
                    STREAM(stream), ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, V) == cudaSuccess ? 0 : -3;
}
extern "C" int b200_embedding_bwd(const long long* ids, const void* dout, float* grad_table, int T, int H, int V,
                                  void* stream) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  embedding_bwd_kernel<<<grid_for((long long)T * (H / 8), 256, 148 * 16), 256, 0, STREAM(stream)>>>(
      ids, (const __nv_bfloat16*)dout, grad_table, T, H, V);
  return LAUNCH_OK();
}
extern "C" int b200_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return -12;
  sumsq_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, STREAM(stream)>>>(g, n, out);
  return LAUNCH_OK();
}
extern "C" int b200_clip_coef(float* scalars, float max_norm, float grad_scale, void* stream) {
  clip_coef_kernel<<<1, 1, 0, STREAM(stream)>>>(scalars, max_norm, grad_scale);
  return LAUNCH_OK();
}
extern "C" int b200_adamw(float* master, float* m, float* v, float* grad, void* param_bf16, long long n,
                          const float* scale_ptr, float lr, float beta1, float beta2, float eps, float wd, int step,
                          int zero_grad, void* stream) {
  if (n <= 0) return 0;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  adamw_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, STREAM(stream)>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16,
                                                                       n, scale_ptr, lr, beta1, beta2, eps, wd, bc1,
                                                                       bc2, zero_grad);
  return LAUNCH_OK();
}
extern "C" int b200_ema(float* dst, const float* src, long long n, float beta, void* stream) {
  if (n <= 0) return 0;
  ema_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, STREAM(stream)>>>(dst, src, n, beta);
  return LAUNCH_OK();
}
extern "C" int b200_cast_f32_bf16(const float* src, void* dst, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, STREAM(stream)>>>(src, (__nv_bfloat16*)dst, n);
  return LAUNCH_OK();
}

// ------------------------------------------------------------------ fused decode-path kernels
namespace b200 {

// h = bf16(sum_s ws[s] (+ residual)); x = rmsnorm(h) * w. One block per row. Finishes a split-K GEMM and runs the
// following RMSNorm in the same pass (rollout decode loop: o_proj / down_proj -> next norm).
__global__ void __launch_bounds__(NORM_THREADS)
splitk_reduce_rmsnorm_kernel(const float* __restrict__ ws, int splits, long long slab,
                             const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                             __nv_bfloat16* __restrict__ h_out, __nv_bfloat16* __restrict__ x_out, int M, int N,
                             float eps) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  extern __shared__ uint4 row_cache[];
  __shared__ float red[32];
  const int nvec = N >> 3;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float f[8];
      const float4* base = reinterpret_cast<const float4*>(ws + (size_t)row * N) + 2 * v;
      float4 a = base[0], b = base[1];
      for (int s = 1; s < splits; ++s) {
        const float4* bs = reinterpret_cast<const float4*>(ws + (size_t)s * slab + (size_t)row * N) + 2 * v;
        const float4 c = bs[0], d = bs[1];
        a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
        b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
      }
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      if (residual != nullptr) {
        float g[8];
        unpack8(reinterpret_cast<const uint4*>(residual + (size_t)row * N)[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i]);
      const uint4 u = pack8(f);
      reinterpret_cast<uint4*>(h_out + (size_t)row * N)[v] = u;
      row_cache[v] = u;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum<NORM_THREADS>(ss, red);
    const float rstd = rsqrtf(ss / (float)N + eps);
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float f[8], g[8];
      unpack8(row_cache[v], f);
      unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i] * rstd) * g[i];
      reinterpret_cast<uint4*>(x_out + (size_t)row * N)[v] = pack8(f);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ fp8 (e4m3) per-tensor quantisation
// amax_bits: non-negative float bit pattern (integer max == float max for non-negative floats), zeroed by the caller.
__global__ void __launch_bounds__(256)
absmax_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long n, unsigned int* __restrict__ amax_bits) {
  __shared__ float red[32];
  float m = 0.f;
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(f[k]));
  }
  for (long long i = (nvec << 3) + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(x[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    m = warp_max(m);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
  }
}

// q = e4m3(x / scale), scale = amax / 448 (written to scale_out for the GEMM's alpha). n multiple of 8.
__global__ void __launch_bounds__(256)
quantize_e4m3_kernel(const __nv_bfloat16* __restrict__ x, long long n, const unsigned int* __restrict__ amax_bits,
                     unsigned char* __restrict__ q, float* __restrict__ scale_out) {
  const float amax = fmaxf(__uint_as_float(*amax_bits), 1e-12f);
  const float scale = amax / 448.f, inv = 448.f / amax;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
    unsigned long long out = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      out |= (unsigned long long)__nv_cvt_float_to_fp8(f[k] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * k);
    reinterpret_cast<unsigned long long*>(q)[i] = out;
  }
}

// Tensor-parallel version of the kernel above: the row-parallel projection (o_proj / down_proj) of every TP rank left
// its split-K slabs in a symmetric workspace; each rank reads ALL ranks' slabs (peer loads, fixed order rank 0..n-1, so
// every rank gets bit-identical sums), adds the residual and runs the next RMSNorm. The all-reduce of the row-parallel
// linear is thereby part of the reduction the decode loop performs anyway.
struct WsTable {
  const float* p[8];
};
__global__ void __launch_bounds__(NORM_THREADS)
tp_reduce_rmsnorm_kernel(WsTable ws, int world, int splits, long long slab, const __nv_bfloat16* __restrict__ residual,
                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                         __nv_bfloat16* __restrict__ x_out, int M, int N, float eps) {
  extern __shared__ uint4 row_cache[];
  __shared__ float red[32];
  const int nvec = N >> 3;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      for (int r = 0; r < world; ++r) {
        for (int s = 0; s < splits; ++s) {
          const float4* bs = reinterpret_cast<const float4*>(ws.p[r] + (size_t)s * slab + (size_t)row * N) + 2 * v;
          const float4 c = bs[0], d = bs[1];
          a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
          b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
        }
      }
      float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      if (residual != nullptr) {
        float g[8];
        unpack8(reinterpret_cast<const uint4*>(residual + (size_t)row * N)[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i]);
      const uint4 u = pack8(f);
      reinterpret_cast<uint4*>(h_out + (size_t)row * N)[v] = u;
      row_cache[v] = u;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum<NORM_THREADS>(ss, red);
    const float rstd = rsqrtf(ss / (float)N + eps);
    for (int v = threadIdx.x; v < nvec; v += NORM_THREADS) {
      float f[8], g[8];
      unpack8(row_cache[v], f);
      unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i] * rstd) * g[i];
      reinterpret_cast<uint4*>(x_out + (size_t)row * N)[v] = pack8(f);
    }
    __syncthreads();
  }
}

// Finishes the split-K qkv projection (sum of slabs + bias), applies RoPE to q and k, writes q compactly and k, v
// into the paged KV cache. head_dim 128.
__global__ void rope_kvwrite_splitk_kernel(const float* __restrict__ ws, int splits, long long slab,
                                           const __nv_bfloat16* __restrict__ bias, const int* __restrict__ pos,
                                           const int* __restrict__ slots, const float2* __restrict__ cos_sin,
                                           __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                           __nv_bfloat16* __restrict__ v_cache, int T, int Hq, int Hkv, int max_pos) {
  pdl_launch_dependents();   // successors may start their prologue / weight fetch now; they wait for this grid
  pdl_wait();
  constexpr int HALF = 64;
  const int heads = Hq + 2 * Hkv;
  const int ld = heads * 128;
  const long long total = (long long)T * heads * (HALF / 2);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % (HALF / 2)) * 2;
    const int head = (int)((idx / (HALF / 2)) % heads);
    const int t = (int)(idx / ((long long)(HALF / 2) * heads));
    const size_t off = (size_t)t * ld + head * 128 + i;
    float2 lo = *reinterpret_cast<const float2*>(ws + off);
    float2 hi = *reinterpret_cast<const float2*>(ws + off + HALF);
    for (int s = 1; s < splits; ++s) {
      const float2 a = *reinterpret_cast<const float2*>(ws + (size_t)s * slab + off);
      const float2 b = *reinterpret_cast<const float2*>(ws + (size_t)s * slab + off + HALF);
      lo.x += a.x; lo.y += a.y; hi.x += b.x; hi.y += b.y;
    }
    if (bias != nullptr) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bias + head * 128 + i));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bias + head * 128 + i + HALF));
      lo.x += a.x; lo.y += a.y; hi.x += b.x; hi.y += b.y;
    }
    // the unfused path rounds the projection to bf16 before the rotation: keep the same rounding points
    lo.x = round_bf16(lo.x); lo.y = round_bf16(lo.y); hi.x = round_bf16(hi.x); hi.y = round_bf16(hi.y);
    __nv_bfloat16* dst;
    if (head < Hq) {
      dst = q_out + ((size_t)t * Hq + head) * 128;
    } else {
      const int slot = slots[t];
      if (slot < 0) continue;
      if (head < Hq + Hkv) dst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * 128;
      else dst = v_cache + ((size_t)slot * Hkv + (head - Hq - Hkv)) * 128;
    }
    if (head < Hq + Hkv) {
      int pp = pos[t];
      pp = pp < 0 ? 0 : (pp >= max_pos ? max_pos - 1 : pp);
      const float2 c0 = cos_sin[(size_t)pp * HALF + i], c1 = cos_sin[(size_t)pp * HALF + i + 1];
      float2 ol, oh;
      ol.x = lo.x * c0.x - hi.x * c0.y;
      oh.x = hi.x * c0.x + lo.x * c0.y;
      ol.y = lo.y * c1.x - hi.y * c1.y;
      oh.y = hi.y * c1.x + lo.y * c1.y;
      lo = ol;
      hi = oh;
    }
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(lo.x, lo.y);
    *reinterpret_cast<__nv_bfloat162*>(dst + i + HALF) = __floats2bfloat162_rn(hi.x, hi.y);
  }
}

}  // namespace b200

extern "C" int b200_splitk_reduce_rmsnorm(const float* ws, int splits, const void* residual, const void* w, void* h_out,
                                          void* x_out, int M, int N, float eps, void* stream) {
  if (M <= 0) return 0;
  if (N % 8 || N > 16384) return -10;
  int grid = M < 148 * 8 ? M : 148 * 8;
  return launch_pdl(splitk_reduce_rmsnorm_kernel, dim3(grid), dim3(NORM_THREADS), (size_t)(N / 8) * sizeof(uint4),
                    STREAM(stream), ws, splits, (long long)M * N, (const __nv_bfloat16*)residual,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, M, N, eps) == cudaSuccess ? 0 : -3;
}
extern "C" int b200_rope_kvwrite_splitk(const float* ws, int splits, const void* bias, const int* pos, const int* slots,
                                        const void* cos_sin, void* q_out, void* k_cache, void* v_cache, int T, int Hq,
                                        int Hkv, int max_pos, void* stream) {
  if (T <= 0) return 0;
  long long work = (long long)T * (Hq + 2 * Hkv) * 32;
  return launch_pdl(rope_kvwrite_splitk_kernel, dim3(grid_for(work, 256, 148 * 16)), dim3(256), (size_t)0, STREAM(stream),
                    ws, splits, (long long)T * (Hq + 2 * Hkv) * 128, (const __nv_bfloat16*)bias, pos, slots,
                    (const float2*)cos_sin, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T,
                    Hq, Hkv, max_pos) == cudaSuccess ? 0 : -3;
}

extern "C" int b200_tp_reduce_rmsnorm(const void* const* ws_ptrs, int world, int splits, const void* residual,
                                      const void* w, void* h_out, void* x_out, int M, int N, float eps, void* stream) {
  if (M <= 0) return 0;
  if (N % 8 || N > 16384 || world < 1 || world > 8) return -10;
  WsTable t;
  for (int i = 0; i < 8; ++i) t.p[i] = i < world ? reinterpret_cast<const float*>(ws_ptrs[i]) : nullptr;
  int grid = M < 148 * 8 ? M : 148 * 8;
  tp_reduce_rmsnorm_kernel<<<grid, NORM_THREADS, (size_t)(N / 8) * sizeof(uint4), STREAM(stream)>>>(
      t, world, splits, (long long)M * N, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w,
      (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, M, N, eps);
  return LAUNCH_OK();
}

// x bf16 [n] (n multiple of 8) -> q e4m3 [n] and the de-quantisation scale (amax / 448). amax_bits: 4-byte scratch.
extern "C" int b200_quantize_e4m3(const void* x, long long n, void* q, float* scale_out, unsigned int* amax_bits,
                                  void* stream) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  if (cudaMemsetAsync(amax_bits, 0, 4, STREAM(stream)) != cudaSuccess) return -3;
  const int grid = grid_for(n / 8, 256, 148 * 8);
  absmax_bf16_kernel<<<grid, 256, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, n, amax_bits);
  quantize_e4m3_kernel<<<grid, 256, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, n, amax_bits, (unsigned char*)q,
                                                          scale_out);
  return LAUNCH_OK();
}
