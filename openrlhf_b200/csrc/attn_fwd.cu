// Causal attention forward over a packed (varlen) token stream on tcgen05: used for training / log-prob forwards and
// for rollout prefill. GQA, head_dim 128.
//
// One CTA works on TWO query streams that share the same K/V tiles, so that the tensor core runs one stream's MMAs
// while the other stream's softmax is in flight:
//   * pair_heads = 1 (even GQA group): heads 2x and 2x+1 of one kv-head on the same 128 query rows;
//   * pair_heads = 0: one head on the query rows q0..q0+127 and q0+128..q0+255 of one sequence.
//
//   S_s[128q,128kv] = Q_s K^T   (A = Q tile, smem K-major; B = K tile, smem K-major)  TMEM columns [128 s, 128 s + 128)
//   P_s (bf16) overwrites columns [128 s, 128 s + 64) of its own S tile (two values per 32-bit column)
//   O_s[128q,128d] += P_s V     (A = P in TMEM; B = V tile, smem MN-major)            TMEM columns [256 + 128 s, +128)
//
// warp 0: TMA producer (Q tiles once, K and V through separate 2-stage rings); warp 1: MMA issuer, order
// PV_0(j), S_0(j+1), PV_1(j), S_1(j+1); warps 2-5 / 6-9: softmax of stream 0 / 1, one query row per thread, online
// softmax in the log2 domain with a lazily moved reference maximum (O is rescaled in TMEM only when the running
// maximum grew by more than 2^8). Outputs: O (bf16) and the log-sum-exp per (head, token) for the backward pass.
// Takes the place of flash-attn 2's varlen forward that the reference reaches through HF Transformers
// (openrlhf/models/actor.py:152 sets attn_implementation="flash_attention_2").
#include <cstring>

#include "ptx.cuh"

namespace b200 {

constexpr int AT_HD = 128;
constexpr int AT_TILE_BYTES = 128 * 128 * 2;  // 32 KB: Q, K and V tiles all have this size

struct AttnFwdParams {
  const int* cu_seqlens;   // [B+1]
  const int* tile_seq;     // [n_tiles] sequence of each query tile (>= B: padding entry)
  const int* tile_q0;      // [n_tiles] first query row of the tile inside its sequence
  __nv_bfloat16* out;      // [T, ldo]
  float* lse;              // [Hq, T] natural-log LSE
  int n_seqs, T, Hq, Hkv, ldo;
  int q_col0, k_col0, v_col0;   // column of head 0 inside the q / k / v matrices the tensor maps describe
  int n_tiles, pair_heads;
  int q_row_off, q_rows;   // context parallel: q / out / lse hold the rows [q_row_off, q_row_off + q_rows) of the
                           // packed stream that cu_seqlens and the K/V tensor maps index globally (0, T otherwise)
  const int* kv_flags;     // context parallel: kv_flags[row / 128] == kv_epoch once that K/V tile has been gathered
  int kv_epoch;
  float scale_log2;
  int* status;
};

// Context-parallel gather role: the first n_copy_y rows of the grid copy the K/V rows [tile_lo*128, tile_hi*128) of
// the packed stream from their owners' fused qkv buffers (peer memory, plain loads) into this GPU's gathered K/V
// buffer and publish one flag per 128-row tile, so that every remote byte crosses NVLink once and the attention CTAs
// of the same launch start on a tile as soon as it has landed.
struct CpGather {
  const __nv_bfloat16* peer_qkv[8];   // each rank's [rows_per_rank, src_ld] buffer
  __nv_bfloat16* kv_g;                // [T_total, kv_cols]
  int* flags;
  int n_copy_y, tile_lo, tile_hi, rows_per_rank, src_ld, src_col0, kv_cols, epoch;
};

struct AtSmem {
  static constexpr int Q_OFF = 0;                          // 2 query tiles
  static constexpr int K_OFF = 2 * AT_TILE_BYTES;          // 2 stages
  static constexpr int V_OFF = 4 * AT_TILE_BYTES;          // 2 stages
  static constexpr int BAR_OFF = 6 * AT_TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const AttnFwdParams p, const CpGather cp) {
  if ((int)blockIdx.y < cp.n_copy_y) {
    // ------------------------------------------------------------ gather CTAs (lowest block indices: scheduled first)
    const int n_cta = cp.n_copy_y * gridDim.x;
    const int vec_per_row = cp.kv_cols >> 3;
    for (int tile = cp.tile_lo + blockIdx.y * gridDim.x + blockIdx.x; tile < cp.tile_hi; tile += n_cta) {
      const int row0 = tile * 128;
      const int owner = row0 / cp.rows_per_rank;
      const __nv_bfloat16* src = cp.peer_qkv[owner] + (size_t)(row0 - owner * cp.rows_per_rank) * cp.src_ld + cp.src_col0;
      __nv_bfloat16* dst = cp.kv_g + (size_t)row0 * cp.kv_cols;
      for (int i = threadIdx.x; i < 128 * vec_per_row; i += blockDim.x) {
        const int r = i / vec_per_row, c = i % vec_per_row;
        reinterpret_cast<uint4*>(dst + (size_t)r * cp.kv_cols)[c] =
            reinterpret_cast<const uint4*>(src + (size_t)r * cp.src_ld)[c];
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        asm volatile("fence.proxy.async.global;" ::: "memory");   // the tile is read back by TMA (async proxy)
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(cp.flags + tile), "r"(cp.epoch) : "memory");
      }
    }
    return;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AtSmem::BAR_OFF);
  uint64_t* k_full = bars;          // [2]
  uint64_t* k_empty = bars + 2;     // [2]
  uint64_t* v_full = bars + 4;      // [2]
  uint64_t* v_empty = bars + 6;     // [2]
  uint64_t* q_full = bars + 8;
  uint64_t* s_full = bars + 9;      // [2] per stream
  uint64_t* p_full = bars + 11;     // [2] per stream
  uint64_t* o_full = bars + 13;     // [2] per stream
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = p.n_tiles - 1 - ((int)blockIdx.y - cp.n_copy_y);   // later (longer) tiles of a sequence start first
  const int seq = p.tile_seq[t];
  if (seq < 0 || seq >= p.n_seqs) return;           // padding tile: whole CTA leaves before touching TMEM
  const int row_base = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - row_base;
  const int tq0 = p.tile_q0[t];
  const int head0 = p.pair_heads ? 2 * (int)blockIdx.x : (int)blockIdx.x;
  const int head1 = p.pair_heads ? head0 + 1 : head0;
  const int q0_0 = tq0, q0_1 = p.pair_heads ? tq0 : tq0 + 128;
  const int kvh = head0 / (p.Hq / p.Hkv);
  // causal: keys up to the last query row of the stream's tile
  const int lr0 = row_base + q0_0 - p.q_row_off, lr1 = row_base + q0_1 - p.q_row_off;   // rows inside q / out / lse
  const int nt0 = (q0_0 < len && lr0 >= 0 && lr0 < p.q_rows) ? (min(len, q0_0 + 128) + 127) / 128 : 0;
  const int nt1 = (q0_1 < len && lr1 >= 0 && lr1 < p.q_rows) ? (min(len, q0_1 + 128) + 127) / 128 : 0;
  const int n = max(nt0, nt1);
  if (n == 0) return;                               // context parallel: neither stream belongs to this rank

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
      mbar_init(&o_full[s], 1);
    }
    mbar_init(q_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      mbar_expect_tx(q_full, ((nt0 > 0) + (nt1 > 0)) * AT_TILE_BYTES);
      if (nt0 > 0) {
        tma_load_2d(smem + AtSmem::Q_OFF, &tma_q, q_full, p.q_col0 + head0 * AT_HD, lr0);
        tma_load_2d(smem + AtSmem::Q_OFF + 16384, &tma_q, q_full, p.q_col0 + head0 * AT_HD + 64, lr0);
      }
      if (nt1 > 0) {
        uint8_t* sq1 = smem + AtSmem::Q_OFF + AT_TILE_BYTES;
        tma_load_2d(sq1, &tma_q, q_full, p.q_col0 + head1 * AT_HD, lr1);
        tma_load_2d(sq1 + 16384, &tma_q, q_full, p.q_col0 + head1 * AT_HD + 64, lr1);
      }
      for (int j = 0; j < n; ++j) {
        const int stage = j & 1;
        const uint32_t phase = (j >> 1) & 1;
        const int r = row_base + j * 128;
        uint8_t* sk = smem + AtSmem::K_OFF + stage * AT_TILE_BYTES;
        uint8_t* sv = smem + AtSmem::V_OFF + stage * AT_TILE_BYTES;
        if (!mbar_wait(&k_empty[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
        if (p.kv_flags != nullptr) {                // context parallel: wait (bounded) until the tile was gathered
          const int* f = p.kv_flags + (r >> 7);
          const uint64_t t0 = globaltimer_ns();
          int seen;
          bool landed = true;
          while (true) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if (seen == p.kv_epoch) break;
            if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { landed = false; break; }
            __nanosleep(200);
          }
          if (!landed) {
            if (p.status != nullptr) atomicCAS(p.status, 0, ERR_TIMEOUT_FULL);
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        mbar_expect_tx(&k_full[stage], AT_TILE_BYTES);
        tma_load_2d(sk, &tma_k, &k_full[stage], p.k_col0 + kvh * AT_HD, r);
        tma_load_2d(sk + 16384, &tma_k, &k_full[stage], p.k_col0 + kvh * AT_HD + 64, r);
        if (!mbar_wait(&v_empty[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&v_full[stage], AT_TILE_BYTES);
        tma_load_2d(sv, &tma_v, &v_full[stage], p.v_col0 + kvh * AT_HD, r);
        tma_load_2d(sv + 16384, &tma_v, &v_full[stage], p.v_col0 + kvh * AT_HD + 64, r);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + AtSmem::Q_OFF);
      const uint32_t sk0 = smem_u32(smem + AtSmem::K_OFF);
      const uint32_t sv0 = smem_u32(smem + AtSmem::V_OFF);
      bool ok = mbar_wait(q_full, 0, p.status, ERR_TIMEOUT_FULL);
      auto issue_s = [&](int s, int j) {
        const uint32_t sk = sk0 + (j & 1) * AT_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < AT_HD / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(sq + s * AT_TILE_BYTES + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sk + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem_base + s * 128, ad, bd, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      };
      auto issue_pv = [&](int s, int j) -> bool {
        if (!mbar_wait(&p_full[s], j & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sv = sv0 + (j & 1) * AT_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < 128 / 16; ++k) {
          const uint64_t bd = make_smem_desc_sw128(sv + k * 2048, 16384, 1024);
          umma_bf16_ts(tmem_base + 256 + s * 128, tmem_base + s * 128 + k * 8, bd, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        return true;
      };
      if (ok && n > 0) ok = mbar_wait(&k_full[0], 0, p.status, ERR_TIMEOUT_FULL);
      if (ok && n > 0) {
        tc_fence_after();
        if (nt0 > 0) issue_s(0, 0);
        if (nt1 > 0) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n && ok; ++j) {
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        if (j < nt0) {
          if (!issue_pv(0, j)) { ok = false; break; }
          if (j == nt0 - 1) umma_commit(&o_full[0]);
        }
        if (j + 1 < n) {
          if (!mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
        }
        if (j + 1 < nt0) issue_s(0, j + 1);
        if (j < nt1) {
          if (!issue_pv(1, j)) { ok = false; break; }
          if (j == nt1 - 1) umma_commit(&o_full[1]);
        }
        umma_commit(&v_empty[j & 1]);
        if (j + 1 < nt1) issue_s(1, j + 1);
        if (j + 1 < n) umma_commit(&k_empty[(j + 1) & 1]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax of stream s, one query row per thread
    const int s = (warp - 2) >> 2;
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;              // query row inside the tile
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int nts = s ? nt1 : nt0;
    const int q0s = s ? q0_1 : q0_0;
    const int head = s ? head1 : head0;
    const int q_pos = q0s + r;
    const uint32_t tm_s = tmem_base + s * 128 + lane_addr;
    const uint32_t tm_o = tmem_base + 256 + s * 128 + lane_addr;
    float m_ref = -INFINITY;                        // reference maximum used in the exponent (log2 domain)
    float l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nts && ok; ++j) {
      // S(j) complete also means PV(j-1) of this stream is complete: MMAs finish in issue order
      if (!mbar_wait(&s_full[s], j & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[128];
      tmem_ld_32x32b_x32(tm_s, v);
      tmem_ld_32x32b_x32(tm_s + 32, v + 32);
      tmem_ld_32x32b_x32(tm_s + 64, v + 64);
      tmem_ld_32x32b_x32(tm_s + 96, v + 96);
      tmem_ld_wait();
      const int kv0 = j * 128;
      if (kv0 + 127 > q0s) {                        // diagonal tile: causal mask (keys past the sequence end are
#pragma unroll                                      // above every valid row's diagonal, so this covers them too)
        for (int i = 0; i < 128; ++i)
          if (kv0 + i > q_pos) v[i] = 0xff800000u;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
      mx *= p.scale_log2;
      // lazily move the reference maximum: only when it grew by more than 8 (factor 256)
      const bool grow = mx > m_ref + 8.f || m_ref == -INFINITY;
      const float m_new = grow ? fmaxf(mx, m_ref) : m_ref;
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_ref - m_new);   // m_ref = -inf -> 0
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tm_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x16(tm_o + c * 32, o);
          tmem_st_32x32b_x16(tm_o + c * 32 + 16, o + 16);
        }
      }
      l_run *= alpha;
      m_ref = m_new;
      // p = 2^(s*scale - m_ref); bf16 pairs go back into the first 64 columns of this stream's S tile
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float e0 = exp2f(fmaf(__uint_as_float(v[c * 32 + 2 * i]), p.scale_log2, -m_ref));
          const float e1 = exp2f(fmaf(__uint_as_float(v[c * 32 + 2 * i + 1]), p.scale_log2, -m_ref));
          lsum += e0 + e1;
          pk[i] = pack_bf16x2(e0, e1);
        }
        tmem_st_32x32b_x16(tm_s + c * 16, pk);
      }
      l_run += lsum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    if (ok && nts > 0 && mbar_wait(&o_full[s], 0, p.status, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool row_ok = q_pos < len;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      const int lrow = row_base + q_pos - p.q_row_off;
      __nv_bfloat16* orow = p.out + (size_t)lrow * p.ldo + head * AT_HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tm_o + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(o[q * 8 + 0]) * inv_l, __uint_as_float(o[q * 8 + 1]) * inv_l);
            w.y = pack_bf16x2(__uint_as_float(o[q * 8 + 2]) * inv_l, __uint_as_float(o[q * 8 + 3]) * inv_l);
            w.z = pack_bf16x2(__uint_as_float(o[q * 8 + 4]) * inv_l, __uint_as_float(o[q * 8 + 5]) * inv_l);
            w.w = pack_bf16x2(__uint_as_float(o[q * 8 + 6]) * inv_l, __uint_as_float(o[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = w;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(size_t)head * p.q_rows + lrow] = (m_ref + log2f(l_run)) * 0.6931471805599453f;
    }
  }

  __syncwarp();
  if (p.status != nullptr && *(volatile int*)p.status != 0) {
    // a wait gave up somewhere: give copies in flight time to land before the shared memory is released
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

}  // namespace b200

using namespace b200;

static int launch_attn_fwd(const void* q, int q_rows, const void* k, const void* v, int kv_rows, int q_ld, int k_ld,
                           int v_ld, int q_col0, int k_col0, int v_col0, const int* cu_seqlens, const int* tile_seq,
                           const int* tile_q0, int n_tiles, int tile_rows, void* out, int ldo, float* lse, int n_seqs,
                           int Hq, int Hkv, float scale, int q_row_off, const CpGather& cp, int* status,
                           void* stream_) {
  if (n_tiles <= 0 || q_rows <= 0) return 0;
  if (Hq % Hkv || (q_ld % 8) || (k_ld % 8) || (v_ld % 8) || (ldo % 8) || (q_col0 % 8) || (k_col0 % 8) || (v_col0 % 8))
    return -10;
  const int pair_heads = ((Hq / Hkv) % 2 == 0) ? 1 : 0;
  if (tile_rows != (pair_heads ? 128 : 256) || n_tiles + cp.n_copy_y > 65535) return -10;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_bf16_2d(&tq, q, q_rows, q_ld, q_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tk, k, kv_rows, k_ld, k_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tv, v, kv_rows, v_ld, v_ld, 128, 64);
  if (r) return r;
  static std::atomic<unsigned long long> configured{0};      // one bit per device
  if (!set_max_smem_once(configured, attn_fwd_kernel, AtSmem::TOTAL)) return -2;
  AttnFwdParams p;
  p.cu_seqlens = cu_seqlens; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.n_seqs = n_seqs; p.T = q_rows; p.Hq = Hq; p.Hkv = Hkv;
  p.ldo = ldo; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0; p.n_tiles = n_tiles; p.pair_heads = pair_heads;
  p.q_row_off = q_row_off; p.q_rows = q_rows; p.kv_flags = cp.n_copy_y > 0 ? cp.flags : nullptr; p.kv_epoch = cp.epoch;
  p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  dim3 grid(pair_heads ? Hq / 2 : Hq, n_tiles + cp.n_copy_y);
  attn_fwd_kernel<<<grid, 320, AtSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(tq, tk, tv, p, cp);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// q / k / v: row-major matrices with T rows; *_ld = row stride, *_col0 = column where head 0 starts (so q, k, v may be
// three views of one fused qkv buffer, or separate tensors). tile_seq / tile_q0 list query tiles of `tile_rows` rows:
// 128 when the GQA group is even (two heads per CTA), 256 otherwise (two 128-row halves of one head per CTA).
extern "C" int b200_attn_fwd(const void* q, const void* k, const void* v, int q_ld, int k_ld, int v_ld, int q_col0,
                             int k_col0, int v_col0, const int* cu_seqlens, const int* tile_seq, const int* tile_q0,
                             int n_tiles, int tile_rows, void* out, int ldo, float* lse, int n_seqs, int T, int Hq,
                             int Hkv, float scale, int* status, void* stream_) {
  CpGather cp;
  memset(&cp, 0, sizeof(cp));
  return launch_attn_fwd(q, T, k, v, T, q_ld, k_ld, v_ld, q_col0, k_col0, v_col0, cu_seqlens, tile_seq, tile_q0, n_tiles,
                         tile_rows, out, ldo, lse, n_seqs, Hq, Hkv, scale, 0, cp, status, stream_);
}

// Context-parallel forward. This rank holds rows [rank*T_loc, (rank+1)*T_loc) of the packed stream in qkv_local
// [T_loc, W] (fused layout q | k | v, already rotated; every rank's buffer is reachable through peer_qkv). Documents
// start on multiples of 128 rows, so no K/V tile straddles two ranks. The launch gathers the K/V rows
// [kv_tile_lo*128, (rank+1)*T_loc) into kv_g [T_total, 2*Hkv*128] with n_copy_y rows of gather CTAs and runs the
// attention of the local query rows against it; cu_seqlens and the tile list index the global stream. All ranks must
// have passed a barrier after writing their qkv buffers, and must pass another before those buffers are rewritten.
extern "C" int b200_attn_fwd_cp(const void* qkv_local, const void* const* peer_qkv, int world, int rank, int T_loc,
                                void* kv_g, int* flags, int epoch, int kv_tile_lo, int n_copy_y, const int* cu_seqlens,
                                const int* tile_seq, const int* tile_q0, int n_tiles, int tile_rows, void* out,
                                float* lse, int n_seqs, int Hq, int Hkv, float scale, int* status, void* stream_) {
  if (world < 1 || world > 8 || T_loc % 128 || n_copy_y < 1) return -10;
  const int W = (Hq + 2 * Hkv) * 128, kv_cols = 2 * Hkv * 128;
  CpGather cp;
  memset(&cp, 0, sizeof(cp));
  for (int i = 0; i < world; ++i) cp.peer_qkv[i] = reinterpret_cast<const __nv_bfloat16*>(peer_qkv[i]);
  cp.kv_g = reinterpret_cast<__nv_bfloat16*>(kv_g); cp.flags = flags; cp.n_copy_y = n_copy_y; cp.tile_lo = kv_tile_lo;
  cp.tile_hi = (rank + 1) * T_loc / 128; cp.rows_per_rank = T_loc; cp.src_ld = W; cp.src_col0 = Hq * 128;
  cp.kv_cols = kv_cols; cp.epoch = epoch;
  const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(kv_g);
  return launch_attn_fwd(qkv_local, T_loc, kv, kv + Hkv * 128, world * T_loc, W, kv_cols, kv_cols, 0, 0, 0, cu_seqlens,
                         tile_seq, tile_q0, n_tiles, tile_rows, out, Hq * 128, lse, n_seqs, Hq, Hkv, scale,
                         rank * T_loc, cp, status, stream_);
}
