// Causal attention forward over a packed (varlen) token stream on tcgen05: used for training / log-prob forwards and
// for rollout prefill. GQA, head_dim 128, one CTA per (128-row query tile of one sequence, query head).
//
//   S[128q,128kv] = Q K^T     (A = Q tile,  K-major;  B = K tile, K-major)   accumulator in TMEM columns [0,128)
//   O[128q,128d] += P V       (A = P (smem), K-major; B = V tile, MN-major)  accumulator in TMEM columns [128,256)
//
// warp 0: TMA producer (Q once, then K/V tiles through a 2-stage ring); warp 1: MMA issuer; warps 2-5: softmax, one
// query row per thread, online max/sum in the log2 domain with a lazily updated reference maximum (O is rescaled in
// TMEM only when the running maximum grew by more than 2^8), P written back to shared memory in the 128-byte-swizzled
// K-major layout the second MMA reads. Outputs: O (bf16) and the log-sum-exp per (head, token) for the backward pass.
// Takes the place of flash-attn 2's varlen forward that the reference reaches through HF Transformers
// (openrlhf/models/actor.py:152 sets attn_implementation="flash_attention_2").
#include "ptx.cuh"

namespace b200 {

constexpr int AT_BM = 128;   // query rows per tile
constexpr int AT_BN = 128;   // kv rows per tile
constexpr int AT_HD = 128;
constexpr int AT_STAGES = 2;
constexpr int AT_TILE_BYTES = 128 * 128 * 2;  // 32 KB: Q, K, V and P tiles all have this size

struct AttnFwdParams {
  const int* cu_seqlens;   // [B+1]
  const int* tile_seq;     // [n_tiles] sequence of each query tile (>= B: padding entry)
  const int* tile_q0;      // [n_tiles] first query row of the tile inside its sequence
  __nv_bfloat16* out;      // [T, ldo]
  float* lse;              // [Hq, T] natural-log LSE
  int n_seqs, T, Hq, Hkv, ldo;
  int q_col0, k_col0, v_col0;   // column of head 0 inside the q / k / v matrices the tensor maps describe
  float scale_log2;
  int* status;
};

struct AtSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int P_OFF = AT_TILE_BYTES;
  static constexpr int KV_OFF = 2 * AT_TILE_BYTES;
  static constexpr int BAR_OFF = KV_OFF + AT_STAGES * 2 * AT_TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const AttnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AtSmem::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + AT_STAGES;
  uint64_t* q_full = bars + 2 * AT_STAGES;
  uint64_t* s_full = q_full + 1;
  uint64_t* p_full = q_full + 2;
  uint64_t* o_full = q_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.tile_seq[blockIdx.x];
  if (seq < 0 || seq >= p.n_seqs) return;          // padding tile: whole CTA leaves before touching TMEM
  const int head = blockIdx.y;
  const int kvh = head / (p.Hq / p.Hkv);
  const int row_base = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - row_base;
  const int q0 = p.tile_q0[blockIdx.x];
  const int kv_end = min(len, q0 + AT_BM);          // causal: keys up to the last query row of the tile
  const int n_tiles = (kv_end + AT_BN - 1) / AT_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_expect_tx(q_full, AT_TILE_BYTES);
      tma_load_2d(smem + AtSmem::Q_OFF, &tma_q, q_full, p.q_col0 + head * AT_HD, row_base + q0);
      tma_load_2d(smem + AtSmem::Q_OFF + 16384, &tma_q, q_full, p.q_col0 + head * AT_HD + 64, row_base + q0);
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait(&kv_empty[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
        uint8_t* sk = smem + AtSmem::KV_OFF + stage * 2 * AT_TILE_BYTES;
        uint8_t* sv = sk + AT_TILE_BYTES;
        const int r = row_base + j * AT_BN;
        mbar_expect_tx(&kv_full[stage], 2 * AT_TILE_BYTES);
        tma_load_2d(sk, &tma_k, &kv_full[stage], p.k_col0 + kvh * AT_HD, r);
        tma_load_2d(sk + 16384, &tma_k, &kv_full[stage], p.k_col0 + kvh * AT_HD + 64, r);
        tma_load_2d(sv, &tma_v, &kv_full[stage], p.v_col0 + kvh * AT_HD, r);
        tma_load_2d(sv + 16384, &tma_v, &kv_full[stage], p.v_col0 + kvh * AT_HD + 64, r);
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + AtSmem::Q_OFF);
      const uint32_t sp = smem_u32(smem + AtSmem::P_OFF);
      bool ok = mbar_wait(q_full, 0, p.status, ERR_TIMEOUT_FULL);
      int stage = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!mbar_wait(&kv_full[stage], phase, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + AtSmem::KV_OFF + stage * 2 * AT_TILE_BYTES);
        const uint32_t sv = sk + AT_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(sq + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sk + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_s, ad, bd, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, j & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < AT_BN / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(sp + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sv + k * 2048, 16384, 1024);
          umma_bf16(tmem_o, ad, bd, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[stage]);
        if (j == n_tiles - 1) umma_commit(o_full);
        if (++stage == AT_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;              // query row inside the tile
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int q_pos = q0 + r;
    float m_ref = -INFINITY;                        // reference maximum used in the exponent (log2 domain)
    float l_run = 0.f;
    uint8_t* prow = smem + AtSmem::P_OFF + r * 128;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(s_full, j & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * AT_BN;
      const bool need_mask = (kv0 + AT_BN - 1 > q0) || (kv0 + AT_BN > len);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + c * 32 + i;
          const bool valid = !need_mask || (kv <= q_pos && kv < len);
          if (valid) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      mx *= p.scale_log2;
      // lazily move the reference maximum: only when it grew by more than 8 (factor 256), warp-uniform decision
      float m_new = m_ref;
      const bool grow = mx > m_ref + 8.f || m_ref == -INFINITY;
      if (grow) m_new = fmaxf(mx, m_ref);
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);   // m_ref=-inf -> 0
      if (__any_sync(0xffffffffu, grow) && j > 0) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
#pragma unroll
          for (int i = 0; i < 32; i += 8) tmem_st_32x32b_x8(tmem_o + lane_addr + c * 32 + i, v + i);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      m_ref = m_new;
      // pass 2: p = 2^(s*scale - m_ref), row sum, bf16 P tile into swizzled shared memory
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c * 32, v);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + c * 32 + i;
          const bool valid = !need_mask || (kv <= q_pos && kv < len);
          const float e = valid ? exp2f(__uint_as_float(v[i]) * p.scale_log2 - m_ref) : 0.f;
          pv[i] = e;
          lsum += e;
        }
        // columns c*32 .. c*32+31 -> panel (c >> 1), 16-byte chunks (c & 1) * 4 + q, swizzled by (r & 7)
        uint8_t* pp = prow + (c >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 o;
          o.x = pack_bf16x2(pv[q * 8 + 0], pv[q * 8 + 1]);
          o.y = pack_bf16x2(pv[q * 8 + 2], pv[q * 8 + 3]);
          o.z = pack_bf16x2(pv[q * 8 + 4], pv[q * 8 + 5]);
          o.w = pack_bf16x2(pv[q * 8 + 6], pv[q * 8 + 7]);
          const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(pp + chunk * 16) = o;
        }
      }
      l_run += lsum;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(o_full, 0, p.status, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool row_ok = q_pos < len;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + (size_t)(row_base + q_pos) * p.ldo + head * AT_HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]) * inv_l, __uint_as_float(v[q * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]) * inv_l, __uint_as_float(v[q * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]) * inv_l, __uint_as_float(v[q * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]) * inv_l, __uint_as_float(v[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(size_t)head * p.T + row_base + q_pos] = (m_ref + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  __syncwarp();
  if (p.status != nullptr && *(volatile int*)p.status != 0) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

}  // namespace b200

using namespace b200;

// q / k / v: row-major matrices with T rows; *_cols = number of columns the tensor map may address, *_ld = row stride,
// *_col0 = column where head 0 starts (so q, k, v may be three views of one fused qkv buffer, or separate tensors).
extern "C" int b200_attn_fwd(const void* q, const void* k, const void* v, int q_ld, int k_ld, int v_ld, int q_col0,
                             int k_col0, int v_col0, const int* cu_seqlens, const int* tile_seq, const int* tile_q0,
                             int n_tiles, void* out, int ldo, float* lse, int n_seqs, int T, int Hq, int Hkv,
                             float scale, int* status, void* stream_) {
  if (n_tiles <= 0 || T <= 0) return 0;
  if (Hq % Hkv || (q_ld % 8) || (k_ld % 8) || (v_ld % 8) || (ldo % 8) || (q_col0 % 8) || (k_col0 % 8) || (v_col0 % 8))
    return -10;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_bf16_2d(&tq, q, T, q_ld, q_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tk, k, T, k_ld, k_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tv, v, T, v_ld, v_ld, 128, 64);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AtSmem::TOTAL) != cudaSuccess)
      return -2;
    configured = true;
  }
  AttnFwdParams p;
  p.cu_seqlens = cu_seqlens; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.n_seqs = n_seqs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.ldo = ldo; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  dim3 grid(n_tiles, Hq);
  attn_fwd_kernel<<<grid, 192, AtSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
