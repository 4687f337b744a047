// Causal varlen GQA attention backward on tcgen05 (head_dim 128). One CTA owns one 128-key tile j of one
// (sequence, query head) and walks the query tiles i >= j. Everything is computed transposed (keys on the TMEM lanes),
// so that P^T can stay in tensor memory as the A operand of the dV product:
//
//   S^T  = K  Q_i^T                   (A = K smem,  B = Q_i smem, both K-major)            TMEM [0,128)
//   P^T  = exp2(S^T * c - LSE_i)      bf16 pairs written over TMEM [0,64)
//   dP^T = V  dO_i^T                  (A = V smem,  B = dO_i smem)                         TMEM [128,256)
//   dS^T = P^T o (dP^T - D_i) * scale bf16 tile in shared memory, 128-byte swizzled, rows = keys
//   dV  += P^T dO_i                   (A = P^T in TMEM, B = dO_i smem MN-major)            TMEM [256,384)
//   dK  += dS^T Q_i                   (A = dS^T smem K-major, B = Q_i smem MN-major)       TMEM [384,512)
//   dQ_i = dS K                       (A = dS^T smem read MN-major, B = K smem MN-major)   TMEM [128,256) after dP^T
//
// dQ_i is added into an fp32 accumulator in global memory with 16-byte vector reductions (one CTA per key tile
// contributes);
// dK / dV leave the CTA once, also as fp32 reductions (the query heads of a GQA group share them).
// warp 0: TMA producer (K, V once; Q_i, dO_i through a 2-stage ring); warp 1: MMA issuer; warps 2-5: softmax /
// dS (thread = key row); warps 6-9: LSE / D staging and the dQ read-out (thread = query row).
// Takes the place of flash-attn 2's varlen backward, which the reference reaches through HF Transformers
// (openrlhf/models/actor.py:152).
#include <algorithm>

#include "ptx.cuh"

namespace b200 {

constexpr int AB_TILE = 128 * 128 * 2;   // 32 KB

struct AttnBwdParams {
  const int* cu_seqlens;
  const int* tile_seq;      // [n_tiles] sequence of each key tile (>= n_seqs: padding entry)
  const int* tile_k0;       // [n_tiles] first key row of the tile inside its sequence
  const float* lse;         // [Hq, T] natural log
  const float* delta;       // [Hq, T] rowsum(dO o O)
  float* dq_acc;            // fp32, zero-initialised: row stride acc_ld, head h at column h*128
  float* dk_acc;            // same row stride, kv-head h at column h*128
  float* dv_acc;
  int acc_ld;               // row stride of dq_acc
  int dkv_ld;               // row stride of dk_acc / dv_acc
  int q_row_off, q_rows;    // context parallel: q / dO / lse / delta / dq_acc hold the rows [q_row_off, q_row_off +
                            // q_rows) of the packed stream; K, V, dk_acc, dv_acc and cu_seqlens index it globally
  int n_seqs, T, Hq, Hkv;
  int q_col0, k_col0, v_col0;
  float scale, scale_log2;
  int* status;
};

struct AbSmem {
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = AB_TILE;
  static constexpr int Q_OFF = 2 * AB_TILE;        // 2 stages
  static constexpr int DO_OFF = 4 * AB_TILE;       // 2 stages
  static constexpr int DS_OFF = 6 * AB_TILE;
  static constexpr int STAT_OFF = 7 * AB_TILE;     // [2 stages][lse2 128 | delta 128] floats
  static constexpr int BAR_OFF = STAT_OFF + 2048;
  static constexpr int NEEDED = BAR_OFF + 256;
  static constexpr int TOTAL = 232448;             // everything an SM offers one CTA; base alignment is checked
};

constexpr int ERR_SMEM_ALIGN = 7;



__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_do,
                const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if ((smem - smem_raw) + AbSmem::NEEDED > AbSmem::TOTAL) {   // uniform: nothing allocated yet
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, ERR_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AbSmem::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* stat_full = bars + 5;   // [2]
  uint64_t* s_full = bars + 7;
  uint64_t* p_full = bars + 8;
  uint64_t* dp_full = bars + 9;
  uint64_t* ds_full = bars + 10;
  uint64_t* dq_full = bars + 11;
  uint64_t* dq_empty = bars + 12;
  uint64_t* dkv_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  float* stats = reinterpret_cast<float*>(smem + AbSmem::STAT_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.tile_seq[blockIdx.y];
  if (seq < 0 || seq >= p.n_seqs) return;
  const int head = blockIdx.x;
  const int kvh = head / (p.Hq / p.Hkv);
  const int row_base = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - row_base;
  const int k0 = p.tile_k0[blockIdx.y];
  if (k0 >= len) return;
  const int jt = k0 >> 7;
  // query tiles i = i_lo .. i_lo + n - 1: at or below the diagonal, and among the rows this rank holds
  const int i_lo = max(jt, (max(0, p.q_row_off - row_base) + 127) >> 7);
  const int i_hi = min((len + 127) >> 7, (p.q_row_off + p.q_rows - row_base + 127) >> 7);
  const int n = i_hi - i_lo;
  if (n <= 0) return;
  const int q_base = row_base - p.q_row_off;       // local row of the document's first token

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
      mbar_init(&stat_full[s], 4);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, 4);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 4);
    mbar_init(dkv_full, 1);
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
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_q);
      tma_prefetch_desc(&tma_k);
      tma_prefetch_desc(&tma_v);
      tma_prefetch_desc(&tma_do);
      mbar_expect_tx(kv_full, 2 * AB_TILE);
      tma_load_2d(smem + AbSmem::K_OFF, &tma_k, kv_full, p.k_col0 + kvh * 128, row_base + k0);
      tma_load_2d(smem + AbSmem::K_OFF + 16384, &tma_k, kv_full, p.k_col0 + kvh * 128 + 64, row_base + k0);
      tma_load_2d(smem + AbSmem::V_OFF, &tma_v, kv_full, p.v_col0 + kvh * 128, row_base + k0);
      tma_load_2d(smem + AbSmem::V_OFF + 16384, &tma_v, kv_full, p.v_col0 + kvh * 128 + 64, row_base + k0);
      for (int it = 0; it < n; ++it) {
        const int st = it & 1;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1, p.status, ERR_TIMEOUT_EMPTY)) break;
        const int r = q_base + (i_lo + it) * 128;
        uint8_t* sq = smem + AbSmem::Q_OFF + st * AB_TILE;
        uint8_t* sdo = smem + AbSmem::DO_OFF + st * AB_TILE;
        mbar_expect_tx(&qdo_full[st], 2 * AB_TILE);
        tma_load_2d(sq, &tma_q, &qdo_full[st], p.q_col0 + head * 128, r);
        tma_load_2d(sq + 16384, &tma_q, &qdo_full[st], p.q_col0 + head * 128 + 64, r);
        tma_load_2d(sdo, &tma_do, &qdo_full[st], head * 128, r);
        tma_load_2d(sdo + 16384, &tma_do, &qdo_full[st], head * 128 + 64, r);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_kk = make_idesc_bf16(128, 128, false, false);   // both operands K-major
      constexpr uint32_t id_kn = make_idesc_bf16(128, 128, false, true);    // B read MN-major
      constexpr uint32_t id_nn = make_idesc_bf16(128, 128, true, true);     // A and B read MN-major
      const uint32_t sk = smem_u32(smem + AbSmem::K_OFF), sv = smem_u32(smem + AbSmem::V_OFF);
      const uint32_t sq0 = smem_u32(smem + AbSmem::Q_OFF), sdo0 = smem_u32(smem + AbSmem::DO_OFF);
      const uint32_t sds = smem_u32(smem + AbSmem::DS_OFF);
      auto kmaj = [](uint32_t base, int k) { return make_smem_desc_sw128(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024); };
      auto mnmaj = [](uint32_t base, int k) { return make_smem_desc_sw128(base + k * 2048, 16384, 1024); };
      auto issue_s = [&](int it) {      // S^T = K Q^T
        const uint32_t sq = sq0 + (it & 1) * AB_TILE;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tm_s, kmaj(sk, k), kmaj(sq, k), id_kk, k > 0 ? 1u : 0u);
        umma_commit(s_full);
      };
      auto issue_dp = [&](int it) {     // dP^T = V dO^T
        const uint32_t sdo = sdo0 + (it & 1) * AB_TILE;
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tm_dp, kmaj(sv, k), kmaj(sdo, k), id_kk, k > 0 ? 1u : 0u);
        umma_commit(dp_full);
      };
      bool ok = mbar_wait(kv_full, 0, p.status, ERR_TIMEOUT_FULL) &&
                mbar_wait(&qdo_full[0], 0, p.status, ERR_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int it = 0; it < n && ok; ++it) {
        const uint32_t sq = sq0 + (it & 1) * AB_TILE, sdo = sdo0 + (it & 1) * AB_TILE;
        // dV += P^T dO
        if (!mbar_wait(p_full, it & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16_ts(tm_dv, tm_s + k * 8, mnmaj(sdo, k), id_kn, (it > 0 || k > 0) ? 1u : 0u);
        // S^T of the next query tile may overwrite P^T as soon as the dV product above has read it (issue order)
        if (it + 1 < n) {
          if (!mbar_wait(&qdo_full[(it + 1) & 1], ((it + 1) >> 1) & 1, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_s(it + 1);
        }
        // dK += dS^T Q ; dQ = dS K
        if (!mbar_wait(ds_full, it & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tm_dk, kmaj(sds, k), mnmaj(sq, k), id_kn, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_bf16(tm_dp, mnmaj(sds, k), mnmaj(sk, k), id_nn, k > 0 ? 1u : 0u);
        umma_commit(dq_full);
        umma_commit(&qdo_empty[it & 1]);
        if (it + 1 < n) {
          if (!mbar_wait(dq_empty, it & 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          issue_dp(it + 1);
        } else {
          umma_commit(dkv_full);
        }
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- softmax / dS: one key row per thread
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    uint8_t* ds_row = smem + AbSmem::DS_OFF + r * 128;
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int st = it & 1;
      const float* lse2 = stats + st * 256;      // log2-domain LSE of the 128 query rows (+inf past the sequence end)
      const float* dlt = lse2 + 128;
      if (!mbar_wait(&stat_full[st], (it >> 1) & 1, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
      if (!mbar_wait(s_full, it & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (i_lo + it == jt);       // query tile == key tile: keep q >= k only
      uint32_t pk[64];                           // P^T row as bf16 pairs
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_s + lane_addr + c4 * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int c = c4 * 32 + 2 * i;
          float e0 = exp2f(fmaf(__uint_as_float(v[2 * i]), p.scale_log2, -lse2[c]));
          float e1 = exp2f(fmaf(__uint_as_float(v[2 * i + 1]), p.scale_log2, -lse2[c + 1]));
          if (diag) {
            if (c < r) e0 = 0.f;
            if (c + 1 < r) e1 = 0.f;
          }
          pk[c4 * 16 + i] = pack_bf16x2(e0, e1);
        }
      }
      tmem_st_32x32b_x16(tm_s + lane_addr, pk);
      tmem_st_32x32b_x16(tm_s + lane_addr + 16, pk + 16);
      tmem_st_32x32b_x16(tm_s + lane_addr + 32, pk + 32);
      tmem_st_32x32b_x16(tm_s + lane_addr + 48, pk + 48);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);

      if (!mbar_wait(dp_full, it & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_dp + lane_addr + c4 * 32, v);
        tmem_ld_wait();
        uint32_t ds[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int c = c4 * 32 + 2 * i;
          const __nv_bfloat162 pp = *reinterpret_cast<const __nv_bfloat162*>(&pk[c4 * 16 + i]);
          const float d0 = __bfloat162float(pp.x) * (__uint_as_float(v[2 * i]) - dlt[c]) * p.scale;
          const float d1 = __bfloat162float(pp.y) * (__uint_as_float(v[2 * i + 1]) - dlt[c + 1]) * p.scale;
          ds[i] = pack_bf16x2(d0, d1);
        }
        // columns c4*32 .. +31 -> panel (c4 >> 1), 16-byte chunks (c4 & 1) * 4 + q, swizzled by (r & 7)
        uint8_t* pp = ds_row + (c4 >> 1) * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c4 & 1) * 4 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(pp + chunk * 16) = make_uint4(ds[q * 4], ds[q * 4 + 1], ds[q * 4 + 2], ds[q * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // dV leaves through this warp group (lanes = key rows)
    if (ok && mbar_wait(dkv_full, 0, p.status, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const int kv = k0 + r;
      float* dst = p.dv_acc + (size_t)(row_base + kv) * p.dkv_ld + kvh * 128;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_dv + lane_addr + c4 * 32, v);
        tmem_ld_wait();
        if (kv < len) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            red_add_v4(dst + c4 * 32 + i * 4, __uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- LSE / D staging and dQ read-out (thread = query row)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    auto stage_stats = [&](int it) {
      const int q_pos = (i_lo + it) * 128 + r;
      float l2 = INFINITY, d = 0.f;              // past the sequence end: P becomes exp2(-inf) = 0
      if (q_pos < len) {
        const size_t idx = (size_t)head * p.q_rows + q_base + q_pos;
        l2 = p.lse[idx] * 1.4426950408889634f;
        d = p.delta[idx];
      }
      float* dst = stats + (it & 1) * 256;
      dst[r] = l2;
      dst[128 + r] = d;
      __syncwarp();
      if (lane == 0) mbar_arrive(&stat_full[it & 1]);
    };
    stage_stats(0);
    if (n > 1) stage_stats(1);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      if (!mbar_wait(dq_full, it & 1, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // lane = query row; 16-byte vector reductions (measured faster than scalar reductions that a warp issues over
      // 128 contiguous bytes: the L2 reduction rate follows the instruction count, not the sector count)
      const int q_pos = (i_lo + it) * 128 + r;
      float* dst = p.dq_acc + (size_t)(q_base + q_pos) * p.acc_ld + head * 128;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t v[64];
        tmem_ld_32x32b_x32(tm_dp + lane_addr + half * 64, v);
        tmem_ld_32x32b_x32(tm_dp + lane_addr + half * 64 + 32, v + 32);
        tmem_ld_wait();
        if (half == 1) {                         // everything is in registers: the dP^T / dQ columns are free again
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_empty);
        }
        if (q_pos < len) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            red_add_v4(dst + half * 64 + i * 4, __uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        }
      }
      // the softmax warps finished with stage (it & 1) before ds_full(it), which precedes dq_full(it)
      if (it + 2 < n) stage_stats(it + 2);
    }
    // dK leaves through this warp group
    if (ok && mbar_wait(dkv_full, 0, p.status, ERR_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const int kv = k0 + r;
      float* dst = p.dk_acc + (size_t)(row_base + kv) * p.dkv_ld + kvh * 128;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tm_dk + lane_addr + c4 * 32, v);
        tmem_ld_wait();
        if (kv < len) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            red_add_v4(dst + c4 * 32 + i * 4, __uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
        }
      }
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

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]: one warp per (token, head)
__global__ void __launch_bounds__(256)
attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                      float* __restrict__ delta, int T, int Hq, int ldo, int lddo) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)T * Hq;
  for (long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 5) {
    const int t = (int)(w / Hq), h = (int)(w % Hq);
    const uint2 a = *reinterpret_cast<const uint2*>(out + (size_t)t * ldo + h * 128 + lane * 4);
    const uint2 b = *reinterpret_cast<const uint2*>(dout + (size_t)t * lddo + h * 128 + lane * 4);
    const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
    const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
    const float s = warp_sum(a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y);
    if (lane == 0) delta[(size_t)h * T + t] = s;
  }
}

// fp32 accumulators -> bf16 gradient, with the transpose of the rotary embedding applied to the first n_rope heads of
// each row (rotate-half layout, head_dim 128; cos_sin [max_pos, 64] float2). n_rope = 0: a plain cast.
__global__ void __launch_bounds__(256)
attn_bwd_finalize_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, const int* __restrict__ pos,
                         const float2* __restrict__ cos_sin, int T, int n_heads, int n_rope, int max_pos) {
  const long long total = (long long)T * n_heads * 16;     // one thread: 4 dims of the low half and their partners
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx & 15) * 4;
    const int head = (int)((idx >> 4) % n_heads);
    const int t = (int)((idx >> 4) / n_heads);
    const size_t off = ((size_t)t * n_heads + head) * 128 + i;
    const float4 lo = *reinterpret_cast<const float4*>(acc + off);
    const float4 hi = *reinterpret_cast<const float4*>(acc + off + 64);
    float l[4] = {lo.x, lo.y, lo.z, lo.w}, h[4] = {hi.x, hi.y, hi.z, hi.w};
    if (head < n_rope) {
      int ps = pos[t];
      ps = ps < 0 ? 0 : (ps >= max_pos ? max_pos - 1 : ps);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 cs = cos_sin[(size_t)ps * 64 + i + k];
        const float a = l[k], b = h[k];
        l[k] = a * cs.x + b * cs.y;     // rotation by the negative angle
        h[k] = b * cs.x - a * cs.y;
      }
    }
    uint2 wl, wh;
    wl.x = pack_bf16x2(l[0], l[1]); wl.y = pack_bf16x2(l[2], l[3]);
    wh.x = pack_bf16x2(h[0], h[1]); wh.y = pack_bf16x2(h[2], h[3]);
    *reinterpret_cast<uint2*>(out + off) = wl;
    *reinterpret_cast<uint2*>(out + off + 64) = wh;
  }
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

}  // namespace b200

using namespace b200;

static int launch_delta(const void* out, int ldo, const void* dout, int lddo, float* delta, int rows, int Hq,
                        cudaStream_t stream) {
  const long long warps = (long long)rows * Hq;
  const int blocks = (int)std::min<long long>((warps * 32 + 255) / 256, 148 * 16);
  attn_bwd_delta_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                    reinterpret_cast<const __nv_bfloat16*>(dout), delta, rows, Hq, ldo,
                                                    lddo);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static int launch_finalize(const float* acc, void* dqkv, const int* pos, const void* cos_sin, int max_pos, int rows,
                           int Hq, int Hkv, cudaStream_t stream) {
  const long long work = (long long)rows * (Hq + 2 * Hkv) * 16;
  const int blocks = (int)std::min<long long>((work + 255) / 256, 148 * 16);
  attn_bwd_finalize_kernel<<<blocks, 256, 0, stream>>>(acc, reinterpret_cast<__nv_bfloat16*>(dqkv), pos,
                                                       reinterpret_cast<const float2*>(cos_sin), rows, Hq + 2 * Hkv,
                                                       (pos != nullptr && cos_sin != nullptr) ? Hq + Hkv : 0, max_pos);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static int launch_main(const void* q, int q_rows, const void* k, const void* v, int kv_rows, int q_ld, int k_ld, int v_ld,
                       int q_col0, int k_col0, int v_col0, const void* dout, int lddo, const float* lse,
                       const float* delta, const int* cu_seqlens, const int* tile_seq, const int* tile_k0, int n_tiles,
                       float* dq_acc, int dq_ld, float* dk_acc, float* dv_acc, int dkv_ld, int q_row_off, int n_seqs,
                       int Hq, int Hkv, float scale, int* status, cudaStream_t stream) {
  if (Hq % Hkv || (q_ld % 8) || (k_ld % 8) || (v_ld % 8) || (lddo % 8) || (q_col0 % 8) || (k_col0 % 8) || (v_col0 % 8) ||
      n_tiles > 65535)
    return -10;
  CUtensorMap tq, tk, tv, tdo;
  int r = make_tmap_bf16_2d(&tq, q, q_rows, q_ld, q_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tk, k, kv_rows, k_ld, k_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tv, v, kv_rows, v_ld, v_ld, 128, 64);
  if (r) return r;
  r = make_tmap_bf16_2d(&tdo, dout, q_rows, lddo, lddo, 128, 64);
  if (r) return r;
  static std::atomic<unsigned long long> configured{0};      // one bit per device
  if (!set_max_smem_once(configured, attn_bwd_kernel, AbSmem::TOTAL)) return -2;
  AttnBwdParams p;
  p.cu_seqlens = cu_seqlens; p.tile_seq = tile_seq; p.tile_k0 = tile_k0; p.lse = lse; p.delta = delta;
  p.dq_acc = dq_acc; p.dk_acc = dk_acc; p.dv_acc = dv_acc; p.acc_ld = dq_ld; p.dkv_ld = dkv_ld;
  p.q_row_off = q_row_off; p.q_rows = q_rows;
  p.n_seqs = n_seqs; p.T = q_rows; p.Hq = Hq; p.Hkv = Hkv; p.q_col0 = q_col0; p.k_col0 = k_col0; p.v_col0 = v_col0;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  attn_bwd_kernel<<<dim3(Hq, n_tiles), 320, AbSmem::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Backward of b200_attn_fwd. q / k / v as there (already rotated); out / dout [T, Hq*128] with row strides ldo / lddo;
// lse [Hq, T]. Workspaces: delta fp32 [Hq, T]; acc fp32 [T, (Hq + 2 Hkv) * 128] (zeroed here). Result: dqkv bf16
// [T, (Hq + 2 Hkv) * 128] = [dq heads | dk heads | dv heads]; with pos / cos_sin given, dq and dk are rotated back so
// that the result is the gradient of the un-rotated fused qkv projection output.
extern "C" int b200_attn_bwd(const void* q, const void* k, const void* v, int q_ld, int k_ld, int v_ld, int q_col0,
                             int k_col0, int v_col0, const void* out, int ldo, const void* dout, int lddo,
                             const float* lse, const int* cu_seqlens, const int* tile_seq, const int* tile_k0,
                             int n_tiles, float* delta, float* acc, void* dqkv, const int* pos, const void* cos_sin,
                             int max_pos, int n_seqs, int T, int Hq, int Hkv, float scale, int* status, void* stream_) {
  if (n_tiles <= 0 || T <= 0) return 0;
  if ((ldo % 8) || (lddo % 8)) return -10;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int W = (Hq + 2 * Hkv) * 128;
  if (cudaMemsetAsync(acc, 0, (size_t)T * W * sizeof(float), stream) != cudaSuccess) return -3;
  int r = launch_delta(out, ldo, dout, lddo, delta, T, Hq, stream);
  if (r) return r;
  r = launch_main(q, T, k, v, T, q_ld, k_ld, v_ld, q_col0, k_col0, v_col0, dout, lddo, lse, delta, cu_seqlens, tile_seq,
                  tile_k0, n_tiles, acc, W, acc + Hq * 128, acc + (Hq + Hkv) * 128, W, 0, n_seqs, Hq, Hkv, scale, status,
                  stream);
  if (r) return r;
  return launch_finalize(acc, dqkv, pos, cos_sin, max_pos, T, Hq, Hkv, stream);
}

// Context-parallel backward, first half: this rank's query rows against the gathered K/V (kv_g, as left by
// b200_attn_fwd_cp). dq goes into acc_local [T_loc, W] (columns of the q heads; the whole buffer is zeroed here); dk /
// dv partial sums go into this rank's dkv_g [T_total, 2*Hkv*128] fp32 at global rows (rows [0, (rank+1)*T_loc) are
// zeroed here). After a barrier, b200_cp_dkv_reduce sums the peers' partials for the local rows
// into acc_local's k / v columns and b200_attn_bwd_finalize produces the bf16 dqkv.
extern "C" int b200_attn_bwd_cp(const void* qkv_local, const void* kv_g, int world, int rank, int T_loc, int kv_tile_lo,
                                const void* out, const void* dout, int lddo, const float* lse, const int* cu_seqlens,
                                const int* tile_seq, const int* tile_k0, int n_tiles, float* delta, float* acc_local,
                                float* dkv_g, int n_seqs, int Hq, int Hkv, float scale, int* status, void* stream_) {
  if (n_tiles <= 0 || T_loc <= 0) return 0;
  if (T_loc % 128 || (lddo % 8)) return -10;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int W = (Hq + 2 * Hkv) * 128, kv_cols = 2 * Hkv * 128;
  if (cudaMemsetAsync(acc_local, 0, (size_t)T_loc * W * sizeof(float), stream) != cudaSuccess) return -3;
  (void)kv_tile_lo;   // every row a peer may read back has to be defined, not only the rows this rank adds to
  const size_t row_lo = 0, row_hi = (size_t)(rank + 1) * T_loc;
  if (cudaMemsetAsync(dkv_g + row_lo * kv_cols, 0, (row_hi - row_lo) * kv_cols * sizeof(float), stream) != cudaSuccess)
    return -3;
  int r = launch_delta(out, Hq * 128, dout, lddo, delta, T_loc, Hq, stream);
  if (r) return r;
  const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(kv_g);
  return launch_main(qkv_local, T_loc, kv, kv + Hkv * 128, world * T_loc, W, kv_cols, kv_cols, 0, 0, 0, dout, lddo, lse,
                     delta, cu_seqlens, tile_seq, tile_k0, n_tiles, acc_local, W, dkv_g, dkv_g + Hkv * 128, kv_cols,
                     rank * T_loc, n_seqs, Hq, Hkv, scale, status, stream);
}

extern "C" int b200_attn_bwd_finalize(const float* acc, void* dqkv, const int* pos, const void* cos_sin, int max_pos,
                                      int rows, int Hq, int Hkv, void* stream_) {
  if (rows <= 0) return 0;
  return launch_finalize(acc, dqkv, pos, cos_sin, max_pos, rows, Hq, Hkv, reinterpret_cast<cudaStream_t>(stream_));
}
