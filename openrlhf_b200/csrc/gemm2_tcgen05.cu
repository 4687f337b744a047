// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 (one MMA instruction drives the tensor cores of two SMs).
//
//   C[M,N] (+)= alpha * op(A)[M,K] * op(B)[K,N]  (+ bias[N]) (+ residual[M,N])
//
// A cluster of two CTAs owns one 256 x BN output tile. CTA r of the pair loads rows [128 r, 128 r + 128) of the A
// tile and columns [BN/2 r, BN/2 r + BN/2) of the B tile into its own shared memory (plain TMA loads: each CTA loads
// only what lives in its own shared memory, nothing is multicast), and holds the 128 x BN fp32 accumulator of its rows
// in its own tensor memory. One thread of the even CTA issues the MMAs for the pair; the instruction reads both CTAs'
// shared memory and writes both CTAs' tensor memory. Compared with the single-CTA kernel (gemm_tcgen05.cu) every
// CTA streams half of the B tile per k-block, i.e. 32 KB instead of 48 KB per 128 x 256 x 64 step, which leaves the
// shared-memory pipe and the TMA queue with headroom and allows a six-stage ring.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (both CTAs), warp 1 = TMEM owner (both CTAs) and MMA issuer
// (even CTA only), warps 2..5 = epilogue (both CTAs, each for its own 128 rows). Barriers:
//   full[s]        in the even CTA; its producer arrives with the byte count of BOTH CTAs' loads, both CTAs' TMA loads
//                  complete their bytes on it (the odd CTA addresses it through the cluster window)
//   empty[s]       in each CTA; the MMA thread's tcgen05.commit arrives on both CTAs' copies at once
//   tmem_full[a]   in each CTA; same commit form once a tile's MMAs are issued
//   tmem_empty[a]  in the even CTA; the four epilogue warps of both CTAs arrive on it (8 arrivals)
// Every wait is bounded (ptx.cuh); the two CTAs meet in a cluster barrier before tensor memory is released.
// The same layouts as the single-CTA kernel are supported (K-major / MN-major A and B: forward, dgrad, wgrad), with
// bf16 output (+ bias, + residual) or fp32 output (plain, or accumulated with 16-byte red.add for weight gradients).
#include <cstring>

#include "ptx.cuh"

namespace b200 {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int G2_BM = 128;       // rows per CTA (256 per pair)
constexpr int G2_BK = 64;
constexpr int G2_UMMA_K = 16;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;   // clears the bit that distinguishes the two CTAs of a pair in the
                                              // shared::cluster window: the address of the even CTA's copy

struct Gemm2Params {
  void* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int M, N, K, ldc;
  int out_f32, accumulate, k_splits;
  float alpha;
  int* status;
  // SwiGLU epilogue (K-major B = [gate rows | up rows], N = 2 * sw_half): the even CTA loads BN/2 gate rows, the odd
  // CTA the BN/2 up rows of the same output columns, so accumulator columns [0, BN/2) are gate and [BN/2, BN) are up
  // products; the epilogue writes silu(gate) * up to C[M, sw_half]; C2 (optional, [M, ldc2]) receives the bf16
  // gate / up values for the backward pass.
  int swiglu, sw_half;
  __nv_bfloat16* C2;
  int ldc2;
  // LM-head backward recomputation: C receives d logits = g / T * (onehot(label) - exp(z / T - lse)) as bf16
  // (z = the product, one row per token); see GemmParams::lp_mode in gemm_tcgen05.cu.
  int lp_mode;
  const long long* lp_labels;
  float lp_inv_t;
  const float* lp_lse;
  const float* lp_dlogp;
};

template <int BN>
struct Smem2 {
  static constexpr int A_BYTES = G2_BM * G2_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * G2_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 6 : 8;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 1024;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load whose completion bytes are counted on the EVEN CTA's barrier (same offset as `bar` in this CTA).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & PEER_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrive on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  asm volatile(
      "{\n"
      " .reg .b16 m;\n"
      " mov.b16 m, 3;\n"
      " tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n"
      "}\n" ::"r"(smem_u32(bar))
      : "memory");
}
// Arrive on the EVEN CTA's copy of `bar` (from either CTA).
__device__ __forceinline__ void mbar_arrive_even(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const Gemm2Params p) {
  using L = Smem2<BN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0: even CTA (issues the MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int m_pairs = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int n_blocks = p.swiglu ? (p.sw_half + BN / 2 - 1) / (BN / 2) : (p.N + BN - 1) / BN;
  const int kb_total = (p.K + G2_BK - 1) / G2_BK;
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int num_tiles = m_pairs * n_blocks * splits;
  constexpr int GROUP_M = 8;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);                // four epilogue warps of each CTA
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 2 * BN);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                              // both CTAs' barriers and tensor memory exist before any remote use
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](int tile, int& mp, int& n_blk, int& kb0, int& kb1) {
    const int split = tile % splits;
    const int t = tile / splits;
    const int per_group = GROUP_M * n_blocks;
    const int g = t / per_group;
    const int first = g * GROUP_M;
    const int gsz = min(m_pairs - first, GROUP_M);
    const int r = t % per_group;
    mp = first + r % gsz;
    n_blk = r / gsz;
    kb0 = split * kb_per_split;
    kb1 = min(kb_total, kb0 + kb_per_split);
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, each for its own halves)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int mp, n_blk, kb0, kb1;
        tile_coords(tile, mp, n_blk, kb0, kb1);
        const int row0 = mp * 2 * G2_BM + (int)cta * G2_BM;
        const int col0 = p.swiglu ? (int)cta * p.sw_half + n_blk * (BN / 2) : n_blk * BN + (int)cta * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, &full_bar[stage], kb * G2_BK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c)
              tma_load_2d_pair(sa + c * (G2_BK * 128), &tma_a, &full_bar[stage], row0 + c * 64, kb * G2_BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tma_b, &full_bar[stage], kb * G2_BK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 128; ++c)
              tma_load_2d_pair(sb + c * (G2_BK * 128), &tma_b, &full_bar[stage], col0 + c * 64, kb * G2_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * G2_BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
        int mp, n_blk, kb0, kb1;
        tile_coords(tile, mp, n_blk, kb0, kb1);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < G2_BK / G2_UMMA_K; ++k) {
            uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + k * (G2_UMMA_K * 128), G2_BK * 128, 1024)
                                  : make_smem_desc_sw128(sa + k * (G2_UMMA_K * 2), 16, 1024);
            uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + k * (G2_UMMA_K * 128), G2_BK * 128, 1024)
                                  : make_smem_desc_sw128(sb + k * (G2_UMMA_K * 2), 16, 1024);
            umma2_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty_bar[stage]);    // frees this stage in both CTAs once the MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma2_commit_both(&tmem_full[acc]);        // both CTAs' epilogues may read their halves of the accumulator
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps per CTA, 32 TMEM lanes each)
    const int quarter = warp & 3;
    const bool wide_c = !p.out_f32 && (p.ldc % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 31) == 0);
    const bool v4_ok = p.out_f32 && (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool wide_c2 = p.C2 != nullptr && (p.ldc2 % 16 == 0) && (p.sw_half % 16 == 0) &&
                         ((reinterpret_cast<uintptr_t>(p.C2) & 31) == 0);
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
      int mp, n_blk, kb0, kb1;
      tile_coords(tile, mp, n_blk, kb0, kb1);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = mp * 2 * G2_BM + (int)cta * G2_BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      const bool has_work = kb1 > kb0;
      const float alpha = p.alpha;
      if (p.swiglu) {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(taddr + c * 32, g);
          tmem_ld_32x32b_x32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          const int col0 = n_blk * (BN / 2) + c * 32;
          if (row_ok && has_work && col0 < p.sw_half) {
            __nv_bfloat16* yrow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 16) {
              // sw_half is a multiple of BN / 2 >= 64: a 32-column chunk is never ragged
              uint4 o[2], og[2], ou[2];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const int jj = j + 8 * hh;
                float y[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float gv = __uint_as_float(g[jj + q]);
                  y[q] = gv / (1.f + __expf(-gv)) * __uint_as_float(u[jj + q]);
                }
                o[hh].x = pack_bf16x2(y[0], y[1]);
                o[hh].y = pack_bf16x2(y[2], y[3]);
                o[hh].z = pack_bf16x2(y[4], y[5]);
                o[hh].w = pack_bf16x2(y[6], y[7]);
                og[hh].x = pack_bf16x2(__uint_as_float(g[jj]), __uint_as_float(g[jj + 1]));
                og[hh].y = pack_bf16x2(__uint_as_float(g[jj + 2]), __uint_as_float(g[jj + 3]));
                og[hh].z = pack_bf16x2(__uint_as_float(g[jj + 4]), __uint_as_float(g[jj + 5]));
                og[hh].w = pack_bf16x2(__uint_as_float(g[jj + 6]), __uint_as_float(g[jj + 7]));
                ou[hh].x = pack_bf16x2(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]));
                ou[hh].y = pack_bf16x2(__uint_as_float(u[jj + 2]), __uint_as_float(u[jj + 3]));
                ou[hh].z = pack_bf16x2(__uint_as_float(u[jj + 4]), __uint_as_float(u[jj + 5]));
                ou[hh].w = pack_bf16x2(__uint_as_float(u[jj + 6]), __uint_as_float(u[jj + 7]));
              }
              if (wide_c) {
                st_global_256(yrow + j, o[0], o[1]);
              } else {
                *reinterpret_cast<uint4*>(yrow + j) = o[0];
                *reinterpret_cast<uint4*>(yrow + j + 8) = o[1];
              }
              if (p.C2 != nullptr) {
                __nv_bfloat16* grow = p.C2 + (size_t)row * p.ldc2 + col0 + j;
                if (wide_c2) {
                  st_global_256(grow, og[0], og[1]);
                  st_global_256(grow + p.sw_half, ou[0], ou[1]);
                } else {
                  *reinterpret_cast<uint4*>(grow) = og[0];
                  *reinterpret_cast<uint4*>(grow + 8) = og[1];
                  *reinterpret_cast<uint4*>(grow + p.sw_half) = ou[0];
                  *reinterpret_cast<uint4*>(grow + p.sw_half + 8) = ou[1];
                }
              }
            }
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row_ok && has_work && col0 < p.N) {
          if (p.out_f32) {
            float* crow = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                const float4 v = make_float4(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha,
                                             __uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
                if (p.accumulate) {
                  if (v4_ok) red_add_v4(crow + j, v.x, v.y, v.z, v.w);
                  else { atomicAdd(crow + j, v.x); atomicAdd(crow + j + 1, v.y); atomicAdd(crow + j + 2, v.z); atomicAdd(crow + j + 3, v.w); }
                } else {
                  *reinterpret_cast<float4*>(crow + j) = v;
                }
              }
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 16) {
              uint4 o[2];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const int jj = j + 8 * hh;
                if (col0 + jj < p.N) {
                  float v[8];
#pragma unroll
                  for (int q = 0; q < 8; ++q) v[q] = __uint_as_float(r[jj + q]) * alpha;
                  if (p.lp_mode == 2) {
                    const float g = p.lp_dlogp[row] * p.lp_inv_t, lse = p.lp_lse[row];
                    const long long label = p.lp_labels[row];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                      const float o_ = -g * __expf(v[q] * p.lp_inv_t - lse);
                      v[q] = ((long long)(col0 + jj + q) == label) ? o_ + g : o_;
                    }
                  }
                  if (p.bias != nullptr) {
                    uint4 bb = *reinterpret_cast<const uint4*>(p.bias + col0 + jj);
                    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      float2 f = __bfloat1622float2(b2[q]);
                      v[2 * q] += f.x;
                      v[2 * q + 1] += f.y;
                    }
                  }
                  if (p.residual != nullptr) {
                    uint4 rr = *reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ldc + col0 + jj);
                    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      float2 f = __bfloat1622float2(r2[q]);
                      v[2 * q] += f.x;
                      v[2 * q + 1] += f.y;
                    }
                  }
                  o[hh].x = pack_bf16x2(v[0], v[1]);
                  o[hh].y = pack_bf16x2(v[2], v[3]);
                  o[hh].z = pack_bf16x2(v[4], v[5]);
                  o[hh].w = pack_bf16x2(v[6], v[7]);
                }
              }
              if (wide_c && col0 + j + 16 <= p.N) {
                st_global_256(crow + j, o[0], o[1]);
              } else {
                if (col0 + j < p.N) *reinterpret_cast<uint4*>(crow + j) = o[0];
                if (col0 + j + 8 < p.N) *reinterpret_cast<uint4*>(crow + j + 8) = o[1];
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_even(&tmem_empty[acc]);
    }
  }

  // Teardown. After an error some TMA copies may still be in flight towards this CTA's shared memory: give them a
  // bounded grace period. Both CTAs then meet (neither may retire while the other can still signal its barriers or
  // read its shared memory) before the pair's tensor memory is released.
  __syncwarp();
  if (p.status != nullptr && *(volatile int*)p.status != 0) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 2 * BN);
  }
}

}  // namespace b200

using namespace b200;

template <int BN, bool A_MN, bool B_MN>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const Gemm2Params& p, int sms, cudaStream_t stream) {
  using L = Smem2<BN>;
  static std::atomic<unsigned long long> configured{0};      // one bit per device (per template instance)
  auto kern = gemm2_bf16_kernel<BN, A_MN, B_MN>;
  if (!set_max_smem_once(configured, kern, L::TOTAL)) return -2;
  const int m_pairs = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int n_blocks = p.swiglu ? (p.sw_half + BN / 2 - 1) / (BN / 2) : (p.N + BN - 1) / BN;
  const int tiles = m_pairs * n_blocks * (p.k_splits > 1 ? p.k_splits : 1);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<dim3(2 * pairs), dim3(192), L::TOTAL, stream>>>(ta, tb, p);      // cluster size is a kernel attribute
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static int g2_sm_count = 0;

// Same contract as b200_gemm_bf16 (bf16 operands, bf16 or fp32 output) without split-K slabs, on CTA pairs.
// bn: 128 or 256 (0: 256).
extern "C" int b200_gemm2_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                               int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate,
                               int k_splits, float alpha, int bn, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_f32 ? 4 : 8)) || (N % (out_f32 ? 4 : 8))) return -10;
  if (k_splits > 1 && !(out_f32 && accumulate)) return -11;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -12;
  if (g2_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g2_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 128 && bn != 256) bn = 256;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_bf16_2d(&ta, A, M, K, lda, G2_BM, G2_BK);
  else r = make_tmap_bf16_2d(&ta, A, K, M, lda, G2_BK, 64);
  if (r) return r;
  if (!b_mn) r = make_tmap_bf16_2d(&tb, B, N, K, ldb, bn / 2, G2_BK);
  else r = make_tmap_bf16_2d(&tb, B, K, N, ldb, G2_BK, 64);
  if (r) return r;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.C = C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.out_f32 = out_f32; p.accumulate = accumulate; p.k_splits = k_splits;
  p.alpha = alpha; p.status = status;
#define B200_DISPATCH2(BN_)                                                                \
  if (!a_mn && !b_mn) return launch2<BN_, false, false>(ta, tb, p, g2_sm_count, stream);   \
  if (!a_mn && b_mn) return launch2<BN_, false, true>(ta, tb, p, g2_sm_count, stream);     \
  if (a_mn && !b_mn) return launch2<BN_, true, false>(ta, tb, p, g2_sm_count, stream);     \
  return launch2<BN_, true, true>(ta, tb, p, g2_sm_count, stream);
  if (bn == 256) { B200_DISPATCH2(256) }
  B200_DISPATCH2(128)
#undef B200_DISPATCH2
}


// Y[M, I] = silu(A W_gate^T) * (A W_up^T) with W = [gate rows | up rows] ([2I, K], K-major) on CTA pairs; GU (optional,
// [M, ldgu]) receives the bf16 gate / up products for the backward pass. I must be a multiple of bn / 2.
extern "C" int b200_gemm2_bf16_swiglu(const void* A, const void* W, void* Y, void* GU, int M, int I, int K, int lda,
                                      int ldb, int ldy, int ldgu, int bn, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if (bn != 128 && bn != 256) bn = 256;
  if ((lda % 8) || (ldb % 8) || (ldy % 8) || (I % (bn / 2)) || (GU != nullptr && (ldgu % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(GU)) & 15) return -12;
  if (g2_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g2_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, A, M, K, lda, G2_BM, G2_BK);
  if (r) return r;
  r = make_tmap_bf16_2d(&tb, W, 2 * I, K, ldb, bn / 2, G2_BK);
  if (r) return r;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.C = Y;
  p.M = M; p.N = 2 * I; p.K = K; p.ldc = ldy; p.k_splits = 1; p.alpha = 1.f; p.status = status;
  p.swiglu = 1; p.sw_half = I;
  p.C2 = reinterpret_cast<__nv_bfloat16*>(GU); p.ldc2 = ldgu;
  if (bn == 256) return launch2<256, false, false>(ta, tb, p, g2_sm_count, stream);
  return launch2<128, false, false>(ta, tb, p, g2_sm_count, stream);
}


// LM-head backward recomputation on CTA pairs: dlogits (bf16 [T, ldc]) = g / T * (onehot(label) - softmax(H W^T / T)).
extern "C" int b200_lmhead2_dlogits(const void* H, const void* W, void* dlogits, const long long* labels,
                                    const float* lse, const float* dlogp, float inv_t, int T, int V, int K, int ldh,
                                    int ldw, int ldc, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (T <= 0 || V <= 0 || K <= 0) return 0;
  if ((ldh % 8) || (ldw % 8) || (ldc % 8) || (V % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(H) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(dlogits)) & 15)
    return -12;
  if (g2_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g2_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, H, T, K, ldh, G2_BM, G2_BK);
  if (r) return r;
  r = make_tmap_bf16_2d(&tb, W, V, K, ldw, 128, G2_BK);
  if (r) return r;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.C = dlogits;
  p.M = T; p.N = V; p.K = K; p.ldc = ldc; p.k_splits = 1; p.alpha = 1.f; p.status = status;
  p.lp_mode = 2; p.lp_labels = labels; p.lp_inv_t = inv_t; p.lp_lse = lse; p.lp_dlogp = dlogp;
  return launch2<256, false, false>(ta, tb, p, g2_sm_count, stream);
}
