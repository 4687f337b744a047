// Paged-KV decode attention on tcgen05 with swapped operands, plus the RoPE + KV-cache write kernel that feeds it.
//
// One CTA handles one (sequence, kv-head, kv-split). The KV page (128 tokens x 128 dims) is the M side of the MMAs,
// the G = Hq/Hkv query heads that share the kv-head are the N side (padded to 16):
//     S^T[kv,16]  = K_page[kv,hd] * Q^T[hd,16]        (A = K, K-major;   B = Q, K-major)
//     O^T[hd,16] += V_page^T[hd,kv] * P^T[kv,16]      (A = V, MN-major;  B = P, K-major)
// so no tensor-core work is spent on padding rows, each softmax thread owns one kv token (16 values), and the kernel
// is bound by the KV bytes it streams; two CTAs are resident per SM so that one CTA's loads overlap the other's math. Takes the place of vLLM's paged decode attention in
// the reference's rollout path (openrlhf/trainer/ray/vllm_engine.py:155-179 drives vLLM's engine).
#include "ptx.cuh"

namespace b200 {

constexpr int PAGE = 128;   // tokens per KV page == kv tile
constexpr int HD = 128;     // head dim
constexpr int NPAD = 16;    // query heads per kv head, padded
// one K and one V buffer per CTA; two CTAs share an SM and interleave their loads
constexpr int KV_TILE_BYTES = PAGE * HD * 2;  // 32 KB for K, same for V

struct DecodeParams {
  const int* block_table;  // [B, max_pages]
  const int* seq_lens;     // [B] tokens in the cache, including the current one
  __nv_bfloat16* out;      // [B, Hq, HD]
  float* part_o;           // [B, Hq, splits, HD]  (splits > 1)
  float* part_ml;          // [B, Hq, splits, 2]
  int B, Hq, Hkv, max_pages, splits;
  float scale_log2;        // softmax scale * log2(e)
  int* status;
  int early_trigger;       // the grid fits in one wave (two CTAs per SM): dependents may be released at once
};

struct DecSmem {
  static constexpr int Q_OFF = 0;                         // 2 panels x 16 rows x 128 B
  static constexpr int P_OFF = 4096;                      // 2 buffers x (2 panels x 16 rows x 128 B)
  static constexpr int K_OFF = 12288;                     // K page, 32 KB
  static constexpr int V_OFF = K_OFF + KV_TILE_BYTES;     // V page, 32 KB
  static constexpr int BAR_OFF = V_OFF + KV_TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 1024 + 1024;
};

// Pipeline: the MMA warp issues S(j+1) before it waits for P(j), so the score MMA of the next page runs while the
// softmax warps work on the current one, and the P*V MMA of page j runs while they work on page j+1. S and P are
// double-buffered (TMEM columns [0,16) / [16,32), shared-memory P buffers 0 / 1). The running output O (TMEM
// columns [32,48)) is rescaled only when a head's maximum grew by more than 2^8 since the reference maximum was
// last moved, which needs the previous P*V to have finished (pv_done); otherwise nothing waits on the tensor pipe.
__global__ void __launch_bounds__(192, 2)
attn_decode_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DecSmem::BAR_OFF);
  uint64_t* k_full = bars;        // K and V have their own full / empty pairs: the next K page is fetched while the
  uint64_t* k_empty = bars + 1;   // softmax and the P*V product of the current page are still running
  uint64_t* v_full = bars + 2;
  uint64_t* v_empty = bars + 3;
  uint64_t* q_full = bars + 4;
  uint64_t* s_full = q_full + 1;               // [2]
  uint64_t* p_full = q_full + 3;               // [2]
  uint64_t* pv_done = q_full + 5;
  uint64_t* o_full = q_full + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 7);
  float* red = reinterpret_cast<float*>(q_full + 8);  // [2][4][16] floats: per-warp partial max (two parities)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  // prologue first: it touches nothing an earlier kernel produces, so under programmatic dependent launch it runs
  // while the predecessor is still working
  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_full, 1);
    mbar_fence_init();
  }
  // both P buffers start as zeros: rows of heads beyond G are never written and must stay finite
  for (int i = threadIdx.x; i < 8192 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + DecSmem::P_OFF)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // 2 x 16 columns
  const uint32_t tmem_o = tmem_base + 32;   // 16 columns
  if (p.early_trigger) pdl_launch_dependents();
  pdl_wait();   // seq_lens / block_table / q / the KV cache come from earlier kernels of the stream
  const int len = p.seq_lens[b];
  const int n_tiles_all = (len + PAGE - 1) / PAGE;
  const int tiles_per_split = (n_tiles_all + p.splits - 1) / p.splits;
  const int tile0 = split * tiles_per_split;
  const int tile1 = min(n_tiles_all, tile0 + tiles_per_split);
  const int n_tiles = max(tile1 - tile0, 0);


  if (n_tiles > 0) {
    if (warp == 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tma_k);
        tma_prefetch_desc(&tma_v);
        // Q^T operand: 16 rows (heads of this kv group; rows beyond G are ignored) x 128 dims, two 64-wide panels
        mbar_expect_tx(q_full, 2 * NPAD * 128);
        tma_load_2d(smem + DecSmem::Q_OFF, &tma_q, q_full, 0, b * p.Hq + kvh * G);
        tma_load_2d(smem + DecSmem::Q_OFF + NPAD * 128, &tma_q, q_full, 64, b * p.Hq + kvh * G);
        uint8_t* sk = smem + DecSmem::K_OFF;
        uint8_t* sv = smem + DecSmem::V_OFF;
        uint32_t phase = 0;
        for (int t = tile0; t < tile1; ++t, phase ^= 1) {
          const int page = p.block_table[(size_t)b * p.max_pages + t];
          if (!mbar_wait(k_empty, phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(k_full, KV_TILE_BYTES);
          tma_load_2d(sk, &tma_k, k_full, kvh * HD, page * PAGE);
          tma_load_2d(sk + PAGE * 128, &tma_k, k_full, kvh * HD + 64, page * PAGE);
          if (!mbar_wait(v_empty, phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
          mbar_expect_tx(v_full, KV_TILE_BYTES);
          tma_load_2d(sv, &tma_v, v_full, kvh * HD, page * PAGE);
          tma_load_2d(sv + PAGE * 128, &tma_v, v_full, kvh * HD + 64, page * PAGE);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc_s = make_idesc_bf16(128, NPAD, false, false);
        constexpr uint32_t idesc_o = make_idesc_bf16(128, NPAD, true, false);
        const uint32_t sq = smem_u32(smem + DecSmem::Q_OFF);
        const uint32_t sk = smem_u32(smem + DecSmem::K_OFF);
        const uint32_t sv = smem_u32(smem + DecSmem::V_OFF);
        bool ok = mbar_wait(q_full, 0, p.status, ERR_TIMEOUT_FULL);
        // S^T(j) = K(j) * Q^T into S buffer j&1 : K-steps over hd (8 x 16); panel = k/4, 32 B per step in a panel
        auto issue_s = [&](int j) -> bool {
          if (!mbar_wait(k_full, j & 1, p.status, ERR_TIMEOUT_FULL)) return false;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sk + (k >> 2) * (PAGE * 128) + (k & 3) * 32, 16, 1024);
            const uint64_t bd = make_smem_desc_sw128(sq + (k >> 2) * (NPAD * 128) + (k & 3) * 32, 16, 1024);
            umma_bf16(tmem_s + (j & 1) * NPAD, ad, bd, idesc_s, k > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[j & 1]);
          umma_commit(k_empty);          // the K buffer may be refilled as soon as these MMAs have read it
          return true;
        };
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
          if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
          if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(v_full, j & 1, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sp = smem_u32(smem + DecSmem::P_OFF + (j & 1) * 4096);
          // O^T += V^T * P^T : K-steps over kv (8 x 16 rows of 128 B); M chunks of 64 dims are 16 KB apart
#pragma unroll
          for (int k = 0; k < PAGE / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(sv + k * (16 * 128), PAGE * 128, 1024);
            const uint64_t bd = make_smem_desc_sw128(sp + (k >> 2) * (NPAD * 128) + (k & 3) * 32, 16, 1024);
            umma_bf16(tmem_o, ad, bd, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(v_empty);
          umma_commit(pv_done);
          if (j == n_tiles - 1) umma_commit(o_full);
        }
      }
    } else {
      // ---------------------------------------------------------------- softmax / correction / epilogue
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;  // kv token inside the tile (S^T) and head-dim index (O^T)
      const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
      float m_ref[NPAD], l_part[NPAD];      // reference maximum (log2 domain) and this thread's share of the row sum
#pragma unroll
      for (int h = 0; h < NPAD; ++h) { m_ref[h] = -INFINITY; l_part[h] = 0.f; }
      bool ok = true;
      for (int i = 0; i < n_tiles && ok; ++i) {
        if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        uint32_t sr[NPAD];
        tmem_ld_32x32b_x16(tmem_s + (i & 1) * NPAD + lane_addr, sr);
        tmem_ld_wait();
        const bool valid = (tile0 + i) * PAGE + row < len;
        float s[NPAD];
        float* redp = red + (i & 1) * 64;
#pragma unroll
        for (int h = 0; h < NPAD; ++h) {
          if (h < G) {
            s[h] = valid ? __uint_as_float(sr[h]) * p.scale_log2 : -INFINITY;
            const float tm = warp_max(s[h]);
            if (lane == 0) redp[quarter * NPAD + h] = tm;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // every thread sees the same tile maxima, so the decision to move the reference maximum is block-uniform
        float alpha[NPAD];
        bool move = false;
#pragma unroll
        for (int h = 0; h < NPAD; ++h) {
          alpha[h] = 1.f;
          if (h < G) {
            const float mt = fmaxf(fmaxf(redp[h], redp[NPAD + h]), fmaxf(redp[2 * NPAD + h], redp[3 * NPAD + h]));
            if (mt > m_ref[h] + 8.f || m_ref[h] == -INFINITY) {
              const float mn = fmaxf(mt, m_ref[h]);
              alpha[h] = exp2f(m_ref[h] - mn);      // 0 on the first tile
              m_ref[h] = mn;
              move = true;
            }
          }
        }
        if (move) {
#pragma unroll
          for (int h = 0; h < NPAD; ++h) l_part[h] *= alpha[h];
          if (i > 0) {
            // the running output is being accumulated by P*V(i-1): wait for it, then rescale columns (= heads)
            if (!mbar_wait(pv_done, (i - 1) & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
            tc_fence_after();
            uint32_t orr[NPAD];
            tmem_ld_32x32b_x16(tmem_o + lane_addr, orr);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < NPAD; ++h) orr[h] = __float_as_uint(__uint_as_float(orr[h]) * alpha[h]);
            tmem_st_32x32b_x8(tmem_o + lane_addr, orr);
            tmem_st_32x32b_x8(tmem_o + lane_addr + 8, orr + 8);
            tmem_st_wait();
          }
        }
        // P^T[h][token] as the K-major B operand: panel = token/64, row h of 128 B, 16-byte chunks swizzled by (h & 7)
        {
          uint8_t* pbase = smem + DecSmem::P_OFF + (i & 1) * 4096 + (row >> 6) * (NPAD * 128);
          const int tk = row & 63;
#pragma unroll
          for (int h = 0; h < NPAD; ++h) {
            if (h < G) {
              const float pv = exp2f(s[h] - m_ref[h]);
              l_part[h] += pv;
              const int off = h * 128 + ((((tk >> 3) ^ (h & 7)) << 4) | ((tk & 7) << 1));
              *reinterpret_cast<__nv_bfloat16*>(pbase + off) = __float2bfloat16_rn(pv);
            }
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[i & 1]);
      }
      if (ok && mbar_wait(o_full, 0, p.status, ERR_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
        // row sums: one block-wide reduction at the end instead of one per tile
        float* lred = red;   // reuse: [4][16]
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int h = 0; h < NPAD; ++h) {
          if (h < G) {
            const float t = warp_sum(l_part[h]);
            if (lane == 0) lred[quarter * NPAD + h] = t;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t orr[NPAD];
        tmem_ld_32x32b_x16(tmem_o + lane_addr, orr);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < NPAD; ++h) {
          if (h < G) {
            const float l = lred[h] + lred[NPAD + h] + lred[2 * NPAD + h] + lred[3 * NPAD + h];
            const float o = __uint_as_float(orr[h]) / l;
            if (p.splits == 1) {
              p.out[((size_t)b * p.Hq + kvh * G + h) * HD + row] = __float2bfloat16_rn(o);
            } else {
              const size_t idx = ((size_t)b * p.Hq + kvh * G + h) * p.splits + split;
              p.part_o[idx * HD + row] = o;
              if (row == 0) {
                p.part_ml[idx * 2] = m_ref[h];
                p.part_ml[idx * 2 + 1] = l;
              }
            }
          }
        }
      }
    }
  } else if (p.splits > 1 && warp >= 2) {
    // empty split: contribute nothing (m = -inf, l = 0)
    const int row = (warp & 3) * 32 + lane;
    for (int h = 0; h < G; ++h) {
      const size_t idx = ((size_t)b * p.Hq + kvh * G + h) * p.splits + split;
      p.part_o[idx * HD + row] = 0.f;
      if (row == 0) {
        p.part_ml[idx * 2] = -INFINITY;
        p.part_ml[idx * 2 + 1] = 0.f;
      }
    }
  }

  __syncwarp();
  // a grid larger than one wave releases its successors only now, so that their CTAs do not take SMs away from the
  // CTAs of this grid that have not started yet
  if (!p.early_trigger) pdl_launch_dependents();
  if (p.status != nullptr && *(volatile int*)p.status != 0) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

// Merge split partials: out = sum_s w_s * o_s with w_s = l_s 2^(m_s - m) / sum(...)
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int rows /*B*Hq*/, int splits) {
  const int r = blockIdx.x;
  const int d = threadIdx.x;
  if (r >= rows) return;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[((size_t)r * splits + s) * 2]);
  float den = 0.f, acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[((size_t)r * splits + s) * 2], ls = part_ml[((size_t)r * splits + s) * 2 + 1];
    const float w = ls > 0.f ? ls * exp2f(ms - m) : 0.f;
    den += w;
    acc += w * part_o[((size_t)r * splits + s) * HD + d];
  }
  out[(size_t)r * HD + d] = __float2bfloat16_rn(acc / den);
}

// RoPE on q and k of freshly projected tokens + scatter of k, v into the paged cache + compact q output.
// qkv: [T, ld] rows = [q heads | k heads | v heads]; slot = page * PAGE + offset inside the page.
__global__ void rope_kvwrite_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ pos,
                                    const int* __restrict__ slots, const float2* __restrict__ cos_sin,
                                    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                    __nv_bfloat16* __restrict__ v_cache, int T, int Hq, int Hkv, int ld, int max_pos) {
  constexpr int HALF = HD / 2;
  const int heads = Hq + 2 * Hkv;
  const long long total = (long long)T * heads * (HALF / 2);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % (HALF / 2)) * 2;
    const int head = (int)((idx / (HALF / 2)) % heads);
    const int t = (int)(idx / ((long long)(HALF / 2) * heads));
    const __nv_bfloat16* src = qkv + (size_t)t * ld + head * HD;
    float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
    float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i + HALF));
    __nv_bfloat16* dst;
    if (head < Hq) {
      dst = q_out + ((size_t)t * Hq + head) * HD;
    } else {
      const int slot = slots[t];
      if (slot < 0) continue;
      if (head < Hq + Hkv) dst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * HD;
      else dst = v_cache + ((size_t)slot * Hkv + (head - Hq - Hkv)) * HD;
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

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

}  // namespace b200

using namespace b200;

// q: [B*Hq, 128] contiguous; k_cache / v_cache: [num_pages*128, Hkv*128]; block_table [B, max_pages]; seq_lens [B].
// part_o / part_ml are only touched when splits > 1 (sizes [B*Hq*splits*128] and [B*Hq*splits*2] floats).
extern "C" int b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                const int* seq_lens, void* out, float* part_o, float* part_ml, int B, int Hq, int Hkv,
                                int num_pages, int max_pages, int splits, float scale, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B <= 0) return 0;
  if (Hq % Hkv || Hq / Hkv > NPAD || splits < 1) return -10;
  if (splits > 1 && (part_o == nullptr || part_ml == nullptr)) return -11;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_bf16_2d(&tq, q, (uint64_t)B * Hq, HD, HD, NPAD, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tk, k_cache, (uint64_t)num_pages * PAGE, (uint64_t)Hkv * HD, (uint64_t)Hkv * HD, PAGE, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tv, v_cache, (uint64_t)num_pages * PAGE, (uint64_t)Hkv * HD, (uint64_t)Hkv * HD, PAGE, 64);
  if (r) return r;
  static std::atomic<unsigned long long> configured{0};      // one bit per device
  if (!set_max_smem_once(configured, attn_decode_kernel, DecSmem::TOTAL)) return -2;
  DecodeParams p;
  p.block_table = block_table; p.seq_lens = seq_lens; p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml; p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.max_pages = max_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  dim3 grid(Hkv, B, splits);
  p.early_trigger = (long long)Hkv * B * splits <= 2LL * 148 ? 1 : 0;      // two resident CTAs on each of 148 SMs
  if (launch_pdl(attn_decode_kernel, grid, dim3(192), (size_t)DecSmem::TOTAL, stream, tq, tk, tv, p) != cudaSuccess) return -3;
  if (splits > 1) {
    attn_decode_merge_kernel<<<B * Hq, HD, 0, stream>>>(part_o, part_ml, reinterpret_cast<__nv_bfloat16*>(out), B * Hq,
                                                        splits);
    if (cudaGetLastError() != cudaSuccess) return -3;
  }
  return 0;
}

extern "C" int b200_rope_kvwrite(const void* qkv, const int* pos, const int* slots, const void* cos_sin, void* q_out,
                                 void* k_cache, void* v_cache, int T, int Hq, int Hkv, int ld, int max_pos,
                                 void* stream_) {
  if (T <= 0) return 0;
  long long work = (long long)T * (Hq + 2 * Hkv) * (HD / 4);
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  rope_kvwrite_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)qkv, pos, slots, (const float2*)cos_sin, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
      (__nv_bfloat16*)v_cache, T, Hq, Hkv, ld, max_pos);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ------------------------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in no_alloc.h). The split-KV partials go to a fixed array of this translation
// unit instead of a caller workspace. In host code the array's name is only a handle for the runtime, not a device
// address, so its address is resolved once per device with cudaGetSymbolAddress and then passed to the kernel.
#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_MAX_PARTIAL_ROWS * (HD + 2)];

static float* noalloc_scratch_for_current_device(int* err) {
  constexpr int MAX_DEV = 64;
  static std::atomic<float*> ptrs[MAX_DEV];      // zero-initialised; written once per device, readable from any thread
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) { *err = -21; return nullptr; }
  float* cached = ptrs[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) { *err = -21; return nullptr; }
    cached = static_cast<float*>(p);
    ptrs[dev].store(cached, std::memory_order_release);   // two threads racing here store the same address
  }
  *err = 0;
  return cached;
}

extern "C" int b200_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                        const int* block_table, const int* seq_lens, void* out, int B, int Hq, int Hkv,
                                        int num_pages, int max_pages, int splits, float scale, int* status,
                                        void* stream_) {
  if (B <= 0) return 0;
  if (splits < 1) return -10;
  const long long rows = (long long)B * Hq * splits;
  if (rows > B200_NOALLOC_MAX_PARTIAL_ROWS) return -20;
  int err = 0;
  float* scratch = noalloc_scratch_for_current_device(&err);
  if (scratch == nullptr) return err;
  float* part_o = scratch;                                              // [rows, HD]
  float* part_ml = scratch + (size_t)B200_NOALLOC_MAX_PARTIAL_ROWS * HD;  // [rows, 2]
  return b200_attn_decode(q, k_cache, v_cache, block_table, seq_lens, out, part_o, part_ml, B, Hq, Hkv, num_pages,
                          max_pages, splits, scale, status, stream_);
}
