// In-kernel NVLink collectives over symmetric (peer-mapped) buffers for the ZeRO engine and weight resharding.
//
//   symm_barrier      epoch-numbered flag barrier across ranks; every wait is bounded and reports through a status word
//   zero_reduce       reduce-scatter fused with scaling and the gradient-norm partial: the shard owner pulls its slice
//                     of every peer's fp32 gradient buffer (P2P loads, or one NVLS multimem.ld_reduce per 16 B), sums in
//                     rank order, writes the reduced shard locally and accumulates sum(g^2)
//   zero_adam_gather  fused AdamW on the owned fp32 master shard + bf16 cast + all-gather: the new bf16 values are
//                     stored straight into every peer's parameter buffer (P2P stores or one NVLS multimem.st)
//   reshard_copy      plan-driven gather of weight pieces (from local or peer buffers) into another layout
//
// Together they replace DeepSpeed's bucketed NCCL reduce-scatter -> FusedAdam -> all-gather sequence
// (engine.backward / engine.step at openrlhf/utils/deepspeed/deepspeed.py:177-194) and the per-parameter
// gather + broadcast weight sync of openrlhf/trainer/ray/ppo_actor.py:408-489.
// No TMA is involved here: all remote traffic is plain ld/st/multimem issued by the consuming or producing thread.
#include <algorithm>

#include "ptx.cuh"

namespace b200 {

constexpr int MAX_PEERS = 16;

struct PeerTable {
  void* ptr[MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Each rank writes `epoch` into slot [channel][rank] of every peer's signal pad, then waits until all slots of its own
// pad reach `epoch`. Epochs only grow, so no slot ever needs resetting. wait_limit_ns bounds the wait.
__global__ void symm_barrier_kernel(PeerTable pads, int rank, int world, int channel, unsigned int epoch,
                                    unsigned long long wait_limit_ns, int* status) {
  const int t = threadIdx.x;
  __threadfence_system();
  if (t < world) {
    unsigned int* remote = reinterpret_cast<unsigned int*>(pads.ptr[t]) + channel * MAX_PEERS + rank;
    st_release_sys(remote, epoch);
  }
  if (t < world) {
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pads.ptr[rank]) + channel * MAX_PEERS + t;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      const unsigned int v = ld_acquire_sys(mine);
      if ((int)(v - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > wait_limit_ns) {
        atomicCAS(status, 0, ERR_TIMEOUT_FLAG);
        atomicExch(status + 1, t);  // which peer never arrived
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
}

// The same barrier for use inside CUDA graphs: the epoch is not a launch argument (which a replay could not change)
// but a device-side counter this kernel advances itself. Every rank replays the same graphs in lockstep, so the
// counters stay equal.
__global__ void symm_barrier_dev_kernel(PeerTable pads, int rank, int world, int channel, unsigned int* epoch_counter,
                                        unsigned long long wait_limit_ns, int* status) {
  __shared__ unsigned int s_epoch;
  const int t = threadIdx.x;
  if (t == 0) {
    s_epoch = *epoch_counter + 1;
    *epoch_counter = s_epoch;
  }
  __syncthreads();
  const unsigned int epoch = s_epoch;
  __threadfence_system();
  if (t < world) {
    unsigned int* remote = reinterpret_cast<unsigned int*>(pads.ptr[t]) + channel * MAX_PEERS + rank;
    st_release_sys(remote, epoch);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pads.ptr[rank]) + channel * MAX_PEERS + t;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      const unsigned int v = ld_acquire_sys(mine);
      if ((int)(v - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > wait_limit_ns) {
        atomicCAS(status, 0, ERR_TIMEOUT_FLAG);
        atomicExch(status + 1, t);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
}

// reduced[i] = scale * sum_r grad_r[lo + i]; scalars[0] += sum reduced^2. n is a multiple of 4.
__global__ void __launch_bounds__(256)
zero_reduce_kernel(PeerTable grads, int world, long long lo, long long n, float scale, float* __restrict__ reduced,
                   float* __restrict__ scalars) {
  __shared__ float red[8];
  float ss = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[r]) + lo)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(reduced)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(scalars, t);
  }
}

// Same reduction through the NVSwitch: one multimem.ld_reduce returns the sum over all ranks of 4 floats.
__global__ void __launch_bounds__(256)
zero_reduce_nvls_kernel(const float* __restrict__ mc_grad, long long lo, long long n, float scale,
                        float* __restrict__ reduced, float* __restrict__ scalars) {
  __shared__ float red[8];
  float ss = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc;
    const float* addr = mc_grad + lo + i * 4;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                 : "l"(addr)
                 : "memory");
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(reduced)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(scalars, t);
  }
}

// AdamW on the owned shard, then the bf16 result goes to every rank's parameter buffer at [lo, lo+n).
// scalars[2] = clip coefficient x gradient scale (device scalar, no host round trip). n multiple of 8.
__global__ void __launch_bounds__(256)
zero_adam_gather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                        const float* __restrict__ g, PeerTable params, __nv_bfloat16* mc_param, int world, long long lo,
                        long long n, const float* __restrict__ scalars, float lr, float beta1, float beta2, float eps,
                        float wd, float bc1, float bc2, const unsigned char* __restrict__ decay_mask) {
  const float gs = scalars[2];
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float p[8], mm[8], vv[8], gg[8];
    *reinterpret_cast<float4*>(p) = reinterpret_cast<const float4*>(master)[2 * i];
    *reinterpret_cast<float4*>(p + 4) = reinterpret_cast<const float4*>(master)[2 * i + 1];
    *reinterpret_cast<float4*>(mm) = reinterpret_cast<const float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<const float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(v)[2 * i + 1];
    *reinterpret_cast<float4*>(gg) = reinterpret_cast<const float4*>(g)[2 * i];
    *reinterpret_cast<float4*>(gg + 4) = reinterpret_cast<const float4*>(g)[2 * i + 1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = gg[k] * gs;
      mm[k] = beta1 * mm[k] + (1.f - beta1) * gk;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gk * gk;
      const float decay = (decay_mask == nullptr || decay_mask[i * 8 + k]) ? (1.f - lr * wd) : 1.f;
      p[k] = p[k] * decay - lr * (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps);
    }
    reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(p);
    reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(p + 4);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]);
    o.w = pack_bf16x2(p[6], p[7]);
    if (mc_param != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_param + lo + i * 8),
                   "f"(__uint_as_float(o.x)), "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)),
                   "f"(__uint_as_float(o.w))
                   : "memory");
    } else {
#pragma unroll 4
      for (int r = 0; r < world; ++r)
        reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[r]) + lo)[i] = o;
    }
  }
}

// One block per plan entry: copy `rows` rows of `row_elems` bf16 from (src rank buffer + src_off, stride src_ld) to
// (dst + dst_off, stride dst_ld). row_elems, offsets and strides are multiples of 8 elements.
struct ReshardEntry {
  long long src_off, dst_off;
  int rows, row_elems, src_ld, dst_ld, src_rank, pad;
};
__global__ void __launch_bounds__(256)
reshard_copy_kernel(const ReshardEntry* __restrict__ plan, PeerTable srcs, __nv_bfloat16* __restrict__ dst) {
  const ReshardEntry e = plan[blockIdx.x];
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(srcs.ptr[e.src_rank]) + e.src_off;
  __nv_bfloat16* out = dst + e.dst_off;
  const int vec_per_row = e.row_elems >> 3;
  const long long total = (long long)e.rows * vec_per_row;
  const long long stride = (long long)gridDim.y * blockDim.x;
  long long i = blockIdx.y * (long long)blockDim.x + threadIdx.x;
  // four independent 16-byte loads in flight per thread: a launch with few blocks (a copy that shares the GPU with
  // compute kernels) still covers the NVLink latency
  for (; i + 3 * stride < total; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long j = i + u * stride;
      const int r = (int)(j / vec_per_row), c = (int)(j % vec_per_row);
      v[u] = reinterpret_cast<const uint4*>(src + (size_t)r * e.src_ld)[c];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long j = i + u * stride;
      const int r = (int)(j / vec_per_row), c = (int)(j % vec_per_row);
      reinterpret_cast<uint4*>(out + (size_t)r * e.dst_ld)[c] = v[u];
    }
  }
  for (; i < total; i += stride) {
    const int r = (int)(i / vec_per_row), c = (int)(i % vec_per_row);
    reinterpret_cast<uint4*>(out + (size_t)r * e.dst_ld)[c] = reinterpret_cast<const uint4*>(src + (size_t)r * e.src_ld)[c];
  }
}


// Context-parallel attention backward, second half: every rank holds partial dK / dV sums for ALL rows of the packed
// stream it attended to (dkv_g [T_total, cols] fp32). The owner of rows [rank*rows_per_rank, +rows_per_rank) pulls the
// partials of the ranks >= its own (causal attention: earlier ranks never see its keys) over NVLink, adds them and
// writes the sum into its local accumulator (row stride out_ld, first column out_col0). One pass, every byte crosses
// the link once.
__global__ void __launch_bounds__(256)
cp_dkv_reduce_kernel(PeerTable parts, int world, int rank, int rows_per_rank, int cols, float* __restrict__ out,
                     int out_ld, int out_col0) {
  const int vec_per_row = cols >> 2;
  const long long total = (long long)rows_per_rank * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row), c = (int)(i % vec_per_row);
    const size_t src = ((size_t)rank * rows_per_rank + r) * cols + (size_t)c * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int pr = rank; pr < world; ++pr) {
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(parts.ptr[pr]) + src);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)r * out_ld + out_col0 + c * 4) = acc;
  }
}


// ---------------------------------------------------------------------------------------------- expert parallelism
// Dispatch: routed row i = (token i / k, slot i % k) goes to row dest_row[i] of the receive buffer of rank
// dest_rank[i] (peer stores, 16 bytes per lane), optionally scaled (backward of the weighted combine). One warp per row.
__global__ void __launch_bounds__(256)
ep_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest_rank,
                  const int* __restrict__ dest_row, const float* __restrict__ scale, PeerTable bufs, int rows, int k,
                  int H) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vec = H >> 3;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < rows; i += warps) {
    const int r = dest_rank[i];
    if (r < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * H);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.ptr[r]) + (size_t)dest_row[i] * H);
    const float sc = scale != nullptr ? scale[i] : 1.f;
    for (int c = lane; c < vec; c += 32) {
      uint4 v = src[c];
      if (scale != nullptr) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(h[q]);
          h[q] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      dst[c] = v;
    }
  }
}

// Combine: out[t] = sum_slot w[t,slot] * buf[dest_rank[t,slot]][dest_row[t,slot]] (peer loads, fp32 accumulation; the
// pull makes the sum order fixed, so the result is deterministic). Optionally also keeps the pulled rows
// (rows_out [T*k, H]) and, given dy [T, H], writes dots[t,slot] = <dy[t], row> (the gradient of the routing weight).
__global__ void __launch_bounds__(256)
ep_gather_kernel(PeerTable bufs, const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                 const float* __restrict__ w, __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ rows_out,
                 const __nv_bfloat16* __restrict__ dy, float* __restrict__ dots, int T, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int vec = H >> 3;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int c = lane; c < vec; c += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < k; ++s) {
        const int i = t * k + s;
        const int r = dest_rank[i];
        if (r < 0) continue;
        const uint4 v = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.ptr[r]) +
                                                       (size_t)dest_row[i] * H)[c];
        if (rows_out != nullptr) reinterpret_cast<uint4*>(rows_out + (size_t)i * H)[c] = v;
        const float ws = w != nullptr ? w[i] : 1.f;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float2 f = __bfloat1622float2(h[q]);
          acc[2 * q] += ws * f.x;
          acc[2 * q + 1] += ws * f.y;
        }
      }
      if (out != nullptr) {
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = o;
      }
    }
    if (dots != nullptr) {
      for (int s = 0; s < k; ++s) {
        const int i = t * k + s;
        const int r = dest_rank[i];
        float d = 0.f;
        if (r >= 0) {
          const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(bufs.ptr[r]) + (size_t)dest_row[i] * H;
          for (int c = lane; c < vec; c += 32) {
            const uint4 a = reinterpret_cast<const uint4*>(row)[c];
            const uint4 b = reinterpret_cast<const uint4*>(dy + (size_t)t * H)[c];
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float2 fa = __bfloat1622float2(ha[q]), fb = __bfloat1622float2(hb[q]);
              d += fa.x * fb.x + fa.y * fb.y;
            }
          }
        }
        d = warp_sum(d);
        if (lane == 0) dots[i] = d;
      }
    }
  }
}

}  // namespace b200

using namespace b200;

static PeerTable make_table(const void* const* ptrs, int world) {
  PeerTable t;
  for (int i = 0; i < MAX_PEERS; ++i) t.ptr[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

extern "C" int b200_symm_barrier(const void* const* pad_ptrs, int rank, int world, int channel, unsigned int epoch,
                                 double wait_limit_s, int* status, void* stream) {
  if (world > MAX_PEERS || channel < 0 || channel >= 8) return -10;
  symm_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_table(pad_ptrs, world), rank, world, channel, epoch, (unsigned long long)(wait_limit_s * 1e9), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_zero_reduce(const void* const* grad_ptrs, const void* mc_grad, int world, long long lo,
                                long long n, float scale, float* reduced, float* scalars, int sms, void* stream) {
  if (world > MAX_PEERS || (n & 3) || (lo & 3)) return -10;
  int grid = sms > 0 ? sms : 148 * 4;
  if (mc_grad != nullptr)
    zero_reduce_nvls_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float*>(mc_grad), lo, n, scale, reduced, scalars);
  else
    zero_reduce_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_table(grad_ptrs, world), world, lo,
                                                                                 n, scale, reduced, scalars);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_zero_adam_gather(float* master, float* m, float* v, const float* g, const void* const* param_ptrs,
                                     void* mc_param, int world, long long lo, long long n, const float* scalars,
                                     float lr, float beta1, float beta2, float eps, float wd, int step,
                                     const unsigned char* decay_mask, int sms, void* stream) {
  if (world > MAX_PEERS || (n & 7) || (lo & 7)) return -10;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  int grid = sms > 0 ? sms : 148 * 4;
  zero_adam_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      master, m, v, g, make_table(param_ptrs, world), reinterpret_cast<__nv_bfloat16*>(mc_param), world, lo, n, scalars,
      lr, beta1, beta2, eps, wd, bc1, bc2, decay_mask);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// max_ctas > 0 caps the launch at about that many blocks: a copy that runs next to compute kernels (ZeRO-3 layer
// gathers under the previous layer's GEMMs) must leave thread slots on every SM free, or the compute stream's kernels
// cannot become resident until the copy's blocks retire. 0: fill the GPU.
extern "C" int b200_reshard_copy_budget(const void* plan_dev, int n_entries, const void* const* src_ptrs, int world,
                                        void* dst, int max_ctas, void* stream) {
  if (n_entries <= 0) return 0;
  if (world > MAX_PEERS) return -10;
  // enough blocks per entry to fill the GPU even when a plan has only a handful of large entries
  const int want = max_ctas > 0 ? max_ctas : 148 * 8;
  int gy = (want + n_entries - 1) / n_entries;
  const int gy_min = max_ctas > 0 ? 1 : 8;
  gy = gy < gy_min ? gy_min : (gy > 1024 ? 1024 : gy);
  dim3 grid(n_entries, gy);
  reshard_copy_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const ReshardEntry*>(plan_dev), make_table(src_ptrs, world), reinterpret_cast<__nv_bfloat16*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int b200_reshard_copy(const void* plan_dev, int n_entries, const void* const* src_ptrs, int world, void* dst,
                                 void* stream) {
  return b200_reshard_copy_budget(plan_dev, n_entries, src_ptrs, world, dst, 0, stream);
}

extern "C" int b200_cp_dkv_reduce(const void* const* part_ptrs, int world, int rank, int rows_per_rank, int cols,
                                  float* out, int out_ld, int out_col0, void* stream) {
  if (world > MAX_PEERS || (cols & 3) || (out_ld & 3) || (out_col0 & 3)) return -10;
  cp_dkv_reduce_kernel<<<148 * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_table(part_ptrs, world), world, rank, rows_per_rank, cols, out, out_ld, out_col0);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_ep_scatter(const void* x, const int* dest_rank, const int* dest_row, const float* scale,
                               const void* const* buf_ptrs, int world, int rows, int k, int H, void* stream) {
  if (world > MAX_PEERS || (H & 7) || k < 1) return -10;
  if (rows <= 0) return 0;
  const int blocks = (int)std::min<long long>(((long long)rows * 32 + 255) / 256, 148 * 8);
  ep_scatter_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), dest_rank, dest_row, scale, make_table(buf_ptrs, world), rows, k, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_ep_gather(const void* const* buf_ptrs, int world, const int* dest_rank, const int* dest_row,
                              const float* w, void* out, void* rows_out, const void* dy, float* dots, int T, int k,
                              int H, void* stream) {
  if (world > MAX_PEERS || (H & 7) || k < 1) return -10;
  if (T <= 0) return 0;
  const int blocks = (int)std::min<long long>(((long long)T * 32 + 255) / 256, 148 * 8);
  ep_gather_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_table(buf_ptrs, world), dest_rank, dest_row, w, reinterpret_cast<__nv_bfloat16*>(out),
      reinterpret_cast<__nv_bfloat16*>(rows_out), reinterpret_cast<const __nv_bfloat16*>(dy), dots, T, k, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int b200_symm_barrier_dev(const void* const* pad_ptrs, int rank, int world, int channel,
                                     unsigned int* epoch_counter, double wait_limit_s, int* status, void* stream) {
  if (world > MAX_PEERS || channel < 0 || channel >= 8) return -10;
  symm_barrier_dev_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_table(pad_ptrs, world), rank, world, channel, epoch_counter, (unsigned long long)(wait_limit_s * 1e9), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
