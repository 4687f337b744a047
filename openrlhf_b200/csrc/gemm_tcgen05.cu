// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands staged by TMA).
//
//   C[M,N] (+)= alpha * op(A)[M,K] * op(B)[K,N]  (+ bias[N]) (+ residual[M,N])
//
// Persistent, warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM), warps 2..5 = epilogue.
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
// Operand layouts (all row-major tensors in global memory):
//   A_MN = false: A is [M,K] (K contiguous)     A_MN = true: A is [K,M] (M contiguous, i.e. A^T is used)
//   B_MN = false: B is [N,K] (K contiguous)     B_MN = true: B is [K,N] (N contiguous)
// which covers forward (Y = X W^T), dgrad (dX = dY W) and wgrad (dW = dY^T X) of a linear layer without
// materialising a transpose. Replaces the cuBLAS calls behind nn.Linear in the reference
// (openrlhf/models/actor.py:149-157 instantiates HF models whose projections are nn.Linear).
#include <cstring>

#include "ptx.cuh"

namespace b200 {

constexpr int BM = 128;
constexpr int BK = 64;   // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;

struct GemmParams {
  void* C;               // bf16 or fp32, row-major, leading dimension ldc (elements)
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldc] or null (bf16 outputs only)
  int M, N, K;
  int ldc;
  int out_f32;     // 1: C is fp32
  int accumulate;  // 1: C += result (fp32 outputs only; uses red.add so split-K tiles may overlap)
  int k_splits;    // >1 requires out_f32, and either accumulate or a per-split output slab (split_stride)
  long long split_stride;  // elements between the fp32 output slabs of consecutive K splits (0: all splits share C)
  float alpha;
  int* status;     // device status word (0 = ok)
  // tensor-parallel extensions (all zero / null for a plain GEMM)
  float* peer_c[8];     // fp32 accumulation buffers of the TP peers: the epilogue adds its tile into every one of
  int n_peer_c;         //   them with red.add over NVLink (row-parallel linear: GEMM + all-reduce in one kernel)
  int ag_world;         // >0: A is row-sharded over ag_world ranks (all-gather fused into the A-tile loads)
  int ag_rows;          //   rows held by each rank (multiple of 128)
  int rs_rows;          // >0 with peer_c: reduce-scatter epilogue, rank r owns output rows [r*rs_rows, (r+1)*rs_rows)
  // grouped (mixture-of-experts) extensions
  int group_mode;            // 0 plain; 1: every 128-row M tile belongs to one group and multiplies that group's B
                             // (rows of A / C sorted by group, each group padded to a multiple of 128 rows);
                             // 2: one output matrix per group, K runs over that group's rows (weight gradients)
  const int* tile_group;     // mode 1: [m tiles] group of each tile, < 0 = unused padding tile
  int group_b_rows;          // mode 1: rows of the stacked B matrix per group (N if B is [G*N, K], K if B is [G*K, N])
  const int* group_offsets;  // mode 2: [G+1] first row of each group in the K dimension (multiples of 64)
  int n_groups;              // mode 2
  long long group_c_stride;  // mode 2: elements between consecutive groups' outputs
  // fp8 (e4m3) operands, both K-major: a k-block is 128 elements (still 128 bytes per row), MMA kind::f8f6f4
  int fp8;
  const float* alpha_dev;    // optional device scalar multiplied into alpha (product of the two quantisation scales)
  // SwiGLU epilogue (K-major B = [gate rows | up rows], N = 2 * sw_half): a tile multiplies BN/2 gate rows and the
  // BN/2 up rows of the same columns (two TMA boxes per stage), and the epilogue writes silu(gate) * up to
  // C[M, sw_half]; C2 (optional, [M, ldc2]) receives the bf16 gate / up values for the backward pass
  int swiglu;
  int sw_half;
  __nv_bfloat16* C2;
  int ldc2;
  // LM-head epilogues (K-LMHEAD): the product is logits[tokens, vocabulary], never written as such.
  //   lp_mode 1 (forward): every tile reduces its BN columns to per-row softmax partials
  //       lp_partial[(n_blk * M + row) * 8 + {0: max z, 1: sum exp((z - max) / T), 2: sum exp(z - max),
  //                   3: sum exp(z - max) (z - max), 4: label logit, 5: 1 if the label's column is in this tile}]
  //       (a merge kernel folds the n_blocks partials of a row into log-prob, log-sum-exp and entropy);
  //   lp_mode 2 (backward recomputation): C receives d logits = g / T * (onehot(label) - exp(z / T - lse)) as bf16.
  int lp_mode;
  const long long* lp_labels;   // [M] label token of each row (outside [0, N): no one-hot term, vocabulary shards)
  float lp_inv_t;               // 1 / temperature
  float* lp_partial;            // mode 1
  const float* lp_lse;          // mode 2: [M] log-sum-exp of z / T
  const float* lp_dlogp;        // mode 2: [M] upstream gradient of the log-prob
  int lp_entropy;               // mode 1: also accumulate the entropy terms (slots 2, 3)
  // B is a weight matrix that no kernel in flight writes (decode chain under programmatic dependent launch): the
  // producer fetches the first B tiles of its ring before it waits for the previous kernel, so the weights stream
  // while the predecessor is still running; A and everything written come after the wait.
  int b_static;
};

// Tensor maps of the A shards of all ranks (each CTA loads its remote tile itself; plain tiled TMA, peer memory).
struct PeerMaps {
  CUtensorMap m[8];
};

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int BAR_BYTES = 1024;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024 alignment slack
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ PeerMaps peer_a, const GemmParams p) {
  using L = SmemLayout<BN>;
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
  const int m_blocks = (p.M + BM - 1) / BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int bke = p.fp8 ? 2 * BK : BK;              // elements per k-block (one 128-byte swizzle row)
  const int kb_total = (p.K + bke - 1) / bke;
  const int splits = p.k_splits > 1 ? p.k_splits : 1;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int num_tiles = m_blocks * n_blocks * splits * (p.group_mode == 2 ? p.n_groups : 1);
  constexpr int GROUP_M = 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();    // the next kernel may run its prologue (and fetch its weights) while this one works
  // operands and C may be produced / still read by the previous kernel in the stream; with static weights the
  // producer thread waits only after it has issued its first B tiles (below)
  const bool early_b = p.b_static && !A_MN && !B_MN && p.ag_world == 0 && p.group_mode == 0;
  if (!(early_b && threadIdx.x == 0)) pdl_wait();

  auto tile_coords = [&](int tile, int& m_blk, int& n_blk, int& kb0, int& kb1, int& grp) {
    grp = 0;
    if (p.group_mode == 2) {             // one output per group; K range = that group's rows
      const int per = m_blocks * n_blocks;
      grp = tile / per;
      const int t = tile % per;
      m_blk = t % m_blocks;
      n_blk = t / m_blocks;
      kb0 = p.group_offsets[grp] / BK;
      kb1 = p.group_offsets[grp + 1] / BK;
      return;
    }
    int split = tile % splits;
    int t = tile / splits;
    int per_group = GROUP_M * n_blocks;
    int g = t / per_group;
    int first_m = g * GROUP_M;
    int gsz = min(m_blocks - first_m, GROUP_M);
    int r = t % per_group;
    m_blk = first_m + r % gsz;
    n_blk = r / gsz;
    kb0 = split * kb_per_split;
    kb1 = min(kb_total, kb0 + kb_per_split);
    if (p.group_mode == 1) {
      grp = p.tile_group[m_blk];
      if (grp < 0) kb1 = kb0;            // padding tile: no work for any role
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int prefetched = 0;      // stages of the first tile whose B boxes are already in flight
      if (early_b) {
        if ((int)blockIdx.x < num_tiles) {
          int m_blk, n_blk, kb0, kb1, grp;
          tile_coords(blockIdx.x, m_blk, n_blk, kb0, kb1, grp);
          for (int kb = kb0; kb < kb1 && prefetched < STAGES; ++kb, ++prefetched) {
            uint8_t* sb = smem + prefetched * L::STAGE_BYTES + L::A_BYTES;     // fresh ring: every stage is empty
            mbar_expect_tx(&full_bar[prefetched], L::STAGE_BYTES);
            if (p.swiglu) {
              tma_load_2d(sb, &tma_b, &full_bar[prefetched], kb * bke, n_blk * (BN / 2));
              tma_load_2d(sb + (BN / 2) * 128, &tma_b, &full_bar[prefetched], kb * bke, p.sw_half + n_blk * (BN / 2));
            } else {
              tma_load_2d(sb, &tma_b, &full_bar[prefetched], kb * bke, n_blk * BN);
            }
          }
        }
        pdl_wait();
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk, kb0, kb1, grp;
        tile_coords(tile, m_blk, n_blk, kb0, kb1, grp);
        for (int kb = kb0; kb < kb1; ++kb) {
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (prefetched > 0) {
            // first pass over the ring: the stage was armed and its B boxes issued before the dependency wait
            --prefetched;
            tma_load_2d(sa, &tma_a, &full_bar[stage], kb * bke, m_blk * BM);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          if (!A_MN) {
            if (p.ag_world > 0) {
              const int row0 = m_blk * BM;
              const int owner = row0 / p.ag_rows;
              tma_load_2d(sa, &peer_a.m[owner], &full_bar[stage], kb * BK, row0 - owner * p.ag_rows);
            } else {
              tma_load_2d(sa, &tma_a, &full_bar[stage], kb * bke, m_blk * BM);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (BK * 128), &tma_a, &full_bar[stage], m_blk * BM + c * 64, kb * BK);
          }
          const int brow = p.group_mode == 1 ? grp * p.group_b_rows : 0;   // this group's block of the stacked B
          if (!B_MN) {
            if (p.swiglu) {
              tma_load_2d(sb, &tma_b, &full_bar[stage], kb * bke, n_blk * (BN / 2));
              tma_load_2d(sb + (BN / 2) * 128, &tma_b, &full_bar[stage], kb * bke, p.sw_half + n_blk * (BN / 2));
            } else {
              tma_load_2d(sb, &tma_b, &full_bar[stage], kb * bke, brow + n_blk * BN);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), &tma_b, &full_bar[stage], n_blk * BN + c * 64, brow + kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        int m_blk, n_blk, kb0, kb1, grp;
        tile_coords(tile, m_blk, n_blk, kb0, kb1, grp);
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
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: advance 32 B inside the 128 B swizzle row. MN-major: advance 16 k-rows of 128 B.
            uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                  : make_smem_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                  : make_smem_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            if (p.fp8) umma_e4m3(d_tmem, adesc, bdesc, make_idesc_e4m3(BM, BN), (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 32 TMEM lanes each)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may read
    // 32-byte stores need 32-byte aligned rows: base pointer and leading dimension (bf16 elements) both allow it
    const bool wide_c = !p.out_f32 && (p.ldc % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 31) == 0);
    // fp32 outputs: rows and slabs 32-byte aligned (8 floats)
    const bool wide_f = p.out_f32 && (p.ldc % 8 == 0) && (p.split_stride % 8 == 0) && (p.group_c_stride % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.C) & 31) == 0);
    // 16-byte vector reductions (wgrad accumulation, tensor-parallel pushes): rows, slabs and bases 16-byte aligned
    const bool v4_ok = p.out_f32 && (p.ldc % 4 == 0) && (p.split_stride % 4 == 0) && (p.group_c_stride % 4 == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool wide_c2 = p.C2 != nullptr && (p.ldc2 % 16 == 0) && (p.sw_half % 16 == 0) &&
                         ((reinterpret_cast<uintptr_t>(p.C2) & 31) == 0);
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int m_blk, n_blk, kb0, kb1, grp;
      tile_coords(tile, m_blk, n_blk, kb0, kb1, grp);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      const bool has_work = kb1 > kb0;
      const float alpha = p.alpha_dev != nullptr ? p.alpha * *p.alpha_dev : p.alpha;
      if (p.lp_mode == 1) {
        // ---- fused LM head, forward: softmax partials of this tile's columns; thread = token row
        const long long label = row_ok ? p.lp_labels[row] : -1;
        const int colbase = n_blk * BN;
        constexpr float LOG2E = 1.4426950408889634f;
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {                  // pass 1: row maximum over the tile
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = colbase + c * 32;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) mx = fmaxf(mx, __uint_as_float(r[j]) * alpha);
        }
        float s = 0.f, s1 = 0.f, sz = 0.f, lab = 0.f, has = 0.f;
        const float kt = p.lp_inv_t * LOG2E;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {                  // pass 2: sums relative to the tile maximum
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col0 = colbase + c * 32;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < p.N) {
              const float d = __uint_as_float(r[j]) * alpha - mx;
              s += exp2f(d * kt);
              if (p.lp_entropy) {
                const float e = exp2f(d * LOG2E);
                s1 += e;
                sz += e * d;
              }
              if ((long long)(col0 + j) == label) { lab = d + mx; has = 1.f; }
            }
          }
        }
        if (row_ok && has_work) {
          float4* dst = reinterpret_cast<float4*>(p.lp_partial + ((size_t)n_blk * p.M + row) * 8);
          dst[0] = make_float4(mx, s, s1, sz);
          dst[1] = make_float4(lab, has, 0.f, 0.f);
        }
      } else if (p.swiglu) {
        // TMEM columns [0, BN/2) hold the gate products, [BN/2, BN) the up products of the same output columns
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
            float* crow = reinterpret_cast<float*>(p.C) +
                          (p.group_mode == 2 ? (size_t)grp * p.group_c_stride : (size_t)(tile % splits) * p.split_stride) +
                          (size_t)row * p.ldc + col0;
            if (wide_f && p.n_peer_c == 0 && !p.accumulate && col0 + 32 <= p.N) {
              // plain fp32 tile (split-K slabs of the decode path): 32-byte stores, whole sectors per thread
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 lo, hi;
                lo.x = __float_as_uint(__uint_as_float(r[j]) * alpha);
                lo.y = __float_as_uint(__uint_as_float(r[j + 1]) * alpha);
                lo.z = __float_as_uint(__uint_as_float(r[j + 2]) * alpha);
                lo.w = __float_as_uint(__uint_as_float(r[j + 3]) * alpha);
                hi.x = __float_as_uint(__uint_as_float(r[j + 4]) * alpha);
                hi.y = __float_as_uint(__uint_as_float(r[j + 5]) * alpha);
                hi.z = __float_as_uint(__uint_as_float(r[j + 6]) * alpha);
                hi.w = __float_as_uint(__uint_as_float(r[j + 7]) * alpha);
                st_global_256(crow + j, lo, hi);
              }
            } else
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]) * alpha, __uint_as_float(r[j + 1]) * alpha,
                                       __uint_as_float(r[j + 2]) * alpha, __uint_as_float(r[j + 3]) * alpha);
                if (p.n_peer_c > 0) {
                  if (p.rs_rows > 0) {
                    // reduce-scatter: rank r owns rows [r * rs_rows, (r + 1) * rs_rows) of the output; a tile goes
                    // only to the owner of its rows, at the row's index inside the owner's [rs_rows, ldc] buffer, as
                    // one 16-byte reduction per four columns. (tp - 1) / tp of the tiles cross NVLink, once.
                    const int owner = row / p.rs_rows;
                    float* dst = p.peer_c[owner] + (size_t)(row - owner * p.rs_rows) * p.ldc + col0 + j;
                    if (v4_ok) red_add_v4(dst, v.x, v.y, v.z, v.w);
                    else { atomicAdd(dst, v.x); atomicAdd(dst + 1, v.y); atomicAdd(dst + 2, v.z); atomicAdd(dst + 3, v.w); }
                  } else {
                    const size_t off = (size_t)row * p.ldc + col0 + j;
                    for (int pr = 0; pr < p.n_peer_c; ++pr) {      // all-reduce by push: every peer gets the tile
                      float* dst = p.peer_c[pr] + off;
                      if (v4_ok) red_add_v4(dst, v.x, v.y, v.z, v.w);
                      else { atomicAdd(dst, v.x); atomicAdd(dst + 1, v.y); atomicAdd(dst + 2, v.z); atomicAdd(dst + 3, v.w); }
                    }
                  }
                } else if (p.accumulate) {
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
                    // d logits of the log-prob: g / T * (onehot - softmax(z / T)), from the recomputed logits
                    const float g = p.lp_dlogp[row] * p.lp_inv_t, lse = p.lp_lse[row];
                    const long long label = p.lp_labels[row];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                      const float o = -g * __expf(v[q] * p.lp_inv_t - lse);
                      v[q] = ((long long)(col0 + jj + q) == label) ? o + g : o;
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
                st_global_256(crow + j, o[0], o[1]);          // one full 32-byte sector per thread
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
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // Teardown. After an error some TMA copies may still be in flight towards this CTA's shared memory:
  // give them a bounded grace period before the CTA retires.
  __syncwarp();
  if (p.status != nullptr && *(volatile int*)p.status != 0) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with `ld` elements between rows; box = [box_rows, 64].
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

// 2-D 8-bit tensor map over a row-major [rows, cols] matrix with `ld` bytes between rows; box = [box_rows, 128].
static int make_tmap_u8_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                           uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const PeerMaps& pa, const GemmParams& p, int sms,
                  cudaStream_t stream) {
  using L = SmemLayout<BN>;
  static std::atomic<unsigned long long> configured{0};      // one bit per device (per template instance)
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!set_max_smem_once(configured, kern, L::TOTAL)) return -2;
  int m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  int tiles = m_blocks * n_blocks * (p.k_splits > 1 ? p.k_splits : 1) * (p.group_mode == 2 ? p.n_groups : 1);
  int grid = tiles < sms ? tiles : sms;
  return launch_pdl(kern, dim3(grid), dim3(192), (size_t)L::TOTAL, stream, ta, tb, pa, p) == cudaSuccess ? 0 : -3;
}

// out[m, n] = bf16(sum_s ws[s, m, n] + bias[n] + residual[m, n]); ws holds the fp32 partial products of a split-K GEMM.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int splits, long long slab, const __nv_bfloat16* __restrict__ bias,
                     const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int M, int N, int ldc) {
  pdl_launch_dependents();
  pdl_wait();
  const int nvec = N >> 2;
  const long long total = (long long)M * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(idx / nvec), v = (int)(idx % nvec);
    float4 acc = reinterpret_cast<const float4*>(ws + (size_t)m * N)[v];
    for (int s = 1; s < splits; ++s) {
      const float4 t = reinterpret_cast<const float4*>(ws + (size_t)s * slab + (size_t)m * N)[v];
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    if (bias != nullptr) {
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(bias + v * 4);
      float2 a = __bfloat1622float2(b2[0]), b = __bfloat1622float2(b2[1]);
      acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
    }
    if (residual != nullptr) {
      const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(residual + (size_t)m * ldc + v * 4);
      float2 a = __bfloat1622float2(r2[0]), b = __bfloat1622float2(r2[1]);
      acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + (size_t)m * ldc + v * 4) = o;
  }
}

}  // namespace b200

using namespace b200;

static int g_sm_count = 0;

// Second half of a split-K bf16 GEMM: reduce the fp32 slabs in `ws` ([splits, M, N]) and apply bias / residual.
extern "C" int b200_splitk_reduce(const float* ws, int splits, const void* bias, const void* residual, void* out, int M,
                                  int N, int ldc, void* stream_) {
  if (M <= 0 || N <= 0) return 0;
  if (N % 4 || ldc % 4) return -10;
  long long work = (long long)M * (N / 4);
  long long blocks = (work + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch_pdl(splitk_reduce_kernel, dim3((int)blocks), dim3(256), (size_t)0, reinterpret_cast<cudaStream_t>(stream_),
                    ws, splits, (long long)M * N, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual,
                    (__nv_bfloat16*)out, M, N, ldc) == cudaSuccess ? 0 : -3;
}

// Declares (on != 0) or ends the decode chain for the calling process: kernels launched meanwhile carry the
// programmatic-dependent-launch attribute and GEMMs treat their B operand as static weights. Returns the old mode.
extern "C" int b200_set_pdl(int on) { return b200::g_pdl_mode.exchange(on ? 1 : 0); }

// C-callable entry point. a_mn / b_mn select the operand layouts documented at the top of this file.
// lda / ldb are the row strides (elements) of the tensors as they sit in memory. Returns 0 on a successful launch.
extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                              int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                              int accumulate, int k_splits, long long split_stride, float alpha, int bn, int* status,
                              void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_f32 ? 4 : 8)) || (N % (out_f32 ? 4 : 8))) return -10;
  if (k_splits > 1 && !(out_f32 && (accumulate || split_stride > 0))) return -11;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -12;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 64 && bn != 128 && bn != 256) bn = (N >= 2048 || (long long)M * N >= (long long)128 * 256 * 148) ? 256 : (N >= 512 ? 128 : 64);
  CUtensorMap ta, tb;
  int r;
  // K-major operands: box = 64 (K) x tile rows. MN-major operands: box = 64 (M/N) x 64 (K) per chunk.
  if (!a_mn) r = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
  else r = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, 64);
  if (r) return r;
  if (!b_mn) r = make_tmap_bf16_2d(&tb, B, N, K, ldb, bn, BK);
  else r = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, 64);
  if (r) return r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.out_f32 = out_f32; p.accumulate = accumulate; p.k_splits = k_splits; p.split_stride = split_stride; p.alpha = alpha; p.status = status;
  p.n_peer_c = 0; p.ag_world = 0; p.ag_rows = 0;
  p.b_static = pdl_static_weights() ? 1 : 0;
  for (int i = 0; i < 8; ++i) p.peer_c[i] = nullptr;
  static PeerMaps no_peers;
#define B200_DISPATCH(BN_)                                                                            \
  if (!a_mn && !b_mn) return launch<BN_, false, false>(ta, tb, no_peers, p, g_sm_count, stream);     \
  if (!a_mn && b_mn) return launch<BN_, false, true>(ta, tb, no_peers, p, g_sm_count, stream);       \
  if (a_mn && !b_mn) return launch<BN_, true, false>(ta, tb, no_peers, p, g_sm_count, stream);       \
  return launch<BN_, true, true>(ta, tb, no_peers, p, g_sm_count, stream);
  if (bn == 256) { B200_DISPATCH(256) }
  if (bn == 128) { B200_DISPATCH(128) }
  B200_DISPATCH(64)
#undef B200_DISPATCH
}


// ------------------------------------------------------------------------------------------------------------------
// Fused LM head (K-LMHEAD). Forward: logits = H W^T are reduced tile by tile to softmax partials inside the GEMM
// epilogue (lp_mode 1) and a merge kernel folds a row's partials into log p(label), log-sum-exp and entropy; the
// [tokens, vocabulary] logits are never written. Backward: the logits are recomputed and the epilogue writes
// d logits directly (lp_mode 2), ready to be the operand of the dH and dW GEMMs.
// Stands in for lm_head -> logits.float() -> log_softmax -> gather (+ entropy) of the reference
// (openrlhf/models/actor.py:265-296, openrlhf/models/utils.py:139-186).
constexpr int LMHEAD_BN = 256;

extern "C" int b200_lmhead_num_blocks(int V) { return (V + LMHEAD_BN - 1) / LMHEAD_BN; }

static int lmhead_launch(const void* H, const void* W, int T, int V, int K, int ldh, int ldw, GemmParams& p,
                         cudaStream_t stream) {
  if (T <= 0 || V <= 0 || K <= 0) return 0;
  if ((ldh % 8) || (ldw % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(H) | reinterpret_cast<uintptr_t>(W)) & 15) return -12;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, H, T, K, ldh, BM, BK);
  if (r) return r;
  r = make_tmap_bf16_2d(&tb, W, V, K, ldw, LMHEAD_BN, BK);
  if (r) return r;
  p.M = T; p.N = V; p.K = K; p.k_splits = 1; p.alpha = 1.f;
  static PeerMaps no_peers;
  return launch<LMHEAD_BN, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
}

// partial: fp32 [b200_lmhead_num_blocks(V), T, 8]
extern "C" int b200_lmhead_partials(const void* H, const void* W, const long long* labels, float inv_t, int want_entropy,
                                    float* partial, int T, int V, int K, int ldh, int ldw, int* status, void* stream_) {
  if ((reinterpret_cast<uintptr_t>(partial) & 15) != 0) return -12;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.status = status; p.ldc = 8; p.out_f32 = 1;
  p.lp_mode = 1; p.lp_labels = labels; p.lp_inv_t = inv_t; p.lp_partial = partial; p.lp_entropy = want_entropy;
  return lmhead_launch(H, W, T, V, K, ldh, ldw, p, reinterpret_cast<cudaStream_t>(stream_));
}

// dlogits: bf16 [T, ldc] (ldc >= V, multiple of 8)
extern "C" int b200_lmhead_dlogits(const void* H, const void* W, void* dlogits, const long long* labels, const float* lse,
                                   const float* dlogp, float inv_t, int T, int V, int K, int ldh, int ldw, int ldc,
                                   int* status, void* stream_) {
  if ((ldc % 8) || (V % 8) || (reinterpret_cast<uintptr_t>(dlogits) & 15)) return -10;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.status = status; p.C = dlogits; p.ldc = ldc; p.out_f32 = 0;
  p.lp_mode = 2; p.lp_labels = labels; p.lp_inv_t = inv_t; p.lp_lse = lse; p.lp_dlogp = dlogp;
  return lmhead_launch(H, W, T, V, K, ldh, ldw, p, reinterpret_cast<cudaStream_t>(stream_));
}

namespace b200 {
// One thread per token row: fold the row's n_blocks tile partials (see GemmParams::lp_mode) into
//   logp = z_label / T - logsumexp(z / T),  lse = logsumexp(z / T),  entropy = H(softmax(z)) (untempered).
__global__ void __launch_bounds__(256)
lmhead_merge_kernel(const float* __restrict__ partial, int n_blocks, int T, float inv_t, float* __restrict__ out_logp,
                    float* __restrict__ out_entropy, float* __restrict__ out_lse) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= T) return;
  float M = -INFINITY;
  for (int b = 0; b < n_blocks; ++b) M = fmaxf(M, partial[((size_t)b * T + row) * 8]);
  float S = 0.f, S1 = 0.f, SZ = 0.f, lab = 0.f, has = 0.f;
  for (int b = 0; b < n_blocks; ++b) {
    const float4 a = *reinterpret_cast<const float4*>(partial + ((size_t)b * T + row) * 8);
    const float4 c = *reinterpret_cast<const float4*>(partial + ((size_t)b * T + row) * 8 + 4);
    const float d = a.x - M;                       // <= 0
    S += a.y * __expf(d * inv_t);
    if (out_entropy != nullptr) {
      const float e = __expf(d);
      S1 += a.z * e;
      SZ += (a.w + a.z * d) * e;                   // sum e^{z-M} (z-M) = e^{m-M} (sum e^{z-m} (z-m) + (m-M) sum e^{z-m})
    }
    if (c.y > 0.5f) { lab = c.x; has = 1.f; }
  }
  const float logS = __logf(S);
  if (out_lse != nullptr) out_lse[row] = M * inv_t + logS;
  if (out_logp != nullptr) out_logp[row] = has > 0.5f ? (lab - M) * inv_t - logS : -(M * inv_t + logS);
  if (out_entropy != nullptr) out_entropy[row] = __logf(S1) - SZ / S1;
}
}  // namespace b200

extern "C" int b200_lmhead_merge(const float* partial, int n_blocks, int T, float inv_t, float* out_logp,
                                 float* out_entropy, float* out_lse, void* stream_) {
  if (T <= 0) return 0;
  b200::lmhead_merge_kernel<<<(T + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      partial, n_blocks, T, inv_t, out_logp, out_entropy, out_lse);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}


// Y[M, I] = silu(A W_gate^T) * (A W_up^T) with W = [gate rows | up rows] ([2I, K], K-major); GU (optional, [M, ldgu])
// receives the bf16 gate / up products for the backward pass. I must be a multiple of bn / 2.
extern "C" int b200_gemm_bf16_swiglu(const void* A, const void* W, void* Y, void* GU, int M, int I, int K, int lda,
                                     int ldb, int ldy, int ldgu, int bn, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if (bn != 128 && bn != 256) bn = ((long long)M * 2 * I >= (long long)128 * 256 * 148) ? 256 : 128;
  if ((lda % 8) || (ldb % 8) || (ldy % 8) || (I % (bn / 2)) || (GU != nullptr && (ldgu % 8))) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(GU)) & 15) return -12;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
  if (r) return r;
  r = make_tmap_bf16_2d(&tb, W, 2 * I, K, ldb, bn / 2, BK);      // two boxes of bn/2 rows per stage
  if (r) return r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = Y;
  p.M = M; p.N = 2 * I; p.K = K; p.ldc = ldy;
  p.k_splits = 1; p.alpha = 1.f; p.status = status;
  p.swiglu = 1; p.sw_half = I;
  p.C2 = reinterpret_cast<__nv_bfloat16*>(GU); p.ldc2 = ldgu;
  p.b_static = pdl_static_weights() ? 1 : 0;
  static PeerMaps no_peers;
  if (bn == 256) return launch<256, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
  return launch<128, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
}


// Tensor-parallel linear layers of the rollout engine as single kernels (plain tiled TMA on peer memory for loads,
// red.add over NVLink for the reduction; no collective launch in between).
//  * row-parallel (o_proj / down_proj): C_partial = A[M, K/tp] * B[N, K/tp]^T is added, tile by tile from the epilogue,
//    into the fp32 buffer `peer_c[r]` of every TP rank r: afterwards each rank holds the all-reduced sum. Mode 2 is
//    the reduce-scatter form: rank r owns output rows [r*rows_per_rank, (r+1)*rows_per_rank) and every tile goes only
//    to the owner of its rows ((tp-1)/tp of the output crosses NVLink once; the gather-A GEMM that follows reads the
//    row shards from their owners).
//  * column-parallel with sequence-parallel input (qkv / gate_up): A is row-sharded over the TP ranks
//    (`a_shards[r]` = rank r's [rows_per_rank, K] block); the A-tile loads fetch the rows from their owner, i.e. the
//    all-gather is fused into the operand loads. Output is bf16 C[M_total, N_local] (+ bias).
extern "C" int b200_gemm_bf16_tp(const void* A, const void* const* a_shards, const void* B, void* C,
                                 const void* const* peer_c, const void* bias, int M, int N, int K, int lda, int ldb,
                                 int ldc, int tp, int rows_per_rank,
                                 int mode /*0: push all-reduce, 1: gather-A, 2: reduce-scatter by rows*/, int bn,
                                 int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tp < 1 || tp > 8 || (lda % 8) || (ldb % 8)) return -10;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 64 && bn != 128 && bn != 256) bn = N >= 2048 ? 256 : (N >= 512 ? 128 : 64);
  CUtensorMap ta, tb;
  PeerMaps pm = {};
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.k_splits = 1; p.split_stride = 0; p.alpha = 1.f; p.status = status;
  p.n_peer_c = 0; p.ag_world = 0; p.ag_rows = 0;
  for (int i = 0; i < 8; ++i) p.peer_c[i] = nullptr;
  int r;
  if (mode == 0 || mode == 2) {
    if (ldc % 4 || N % 4) return -10;
    if (mode == 2) {
      if (rows_per_rank <= 0 || rows_per_rank * tp < M) return -10;
      p.rs_rows = rows_per_rank;
    }
    r = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
    if (r) return r;
    p.C = const_cast<void*>(peer_c[0]);
    p.out_f32 = 1; p.accumulate = 1; p.n_peer_c = tp;
    for (int i = 0; i < tp; ++i) p.peer_c[i] = reinterpret_cast<float*>(const_cast<void*>(peer_c[i]));
  } else {
    if (rows_per_rank % BM || M != rows_per_rank * tp || ldc % 8 || N % 8) return -10;
    for (int i = 0; i < tp; ++i) {
      r = make_tmap_bf16_2d(&pm.m[i], a_shards[i], rows_per_rank, K, lda, BM, BK);
      if (r) return r;
    }
    ta = pm.m[0];
    p.C = C; p.out_f32 = 0; p.accumulate = 0; p.ag_world = tp; p.ag_rows = rows_per_rank;
  }
  r = make_tmap_bf16_2d(&tb, B, N, K, ldb, bn, BK);
  if (r) return r;
  if (bn == 256) return launch<256, false, false>(ta, tb, pm, p, g_sm_count, stream);
  if (bn == 128) return launch<128, false, false>(ta, tb, pm, p, g_sm_count, stream);
  return launch<64, false, false>(ta, tb, pm, p, g_sm_count, stream);
}


// Grouped GEMMs for mixture-of-experts layers (rows sorted by expert, every expert padded to a multiple of 128 rows).
//   mode 1: C[P, N] = A[P, K] * B_g^T, g = tile_group[row / 128]; B is the experts' weights stacked along rows:
//           b_mn = 0: [G*N, K] (forward), b_mn = 1: [G*K, N] (input gradient; here "K" is the weight's output dim).
//   mode 2: C_g[M, N] (+)= A[rows of g, M]^T * B[rows of g, N] (weight gradients; fp32 output, one matrix per group,
//           group_offsets[G+1] = padded row offsets, multiples of 128).
extern "C" int b200_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                      int ldc, int b_mn, int mode, const int* tile_group, int group_b_rows,
                                      const int* group_offsets, int n_groups, long long group_c_stride, int accumulate,
                                      int bn, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || n_groups <= 0) return 0;
  if (mode != 1 && mode != 2) return -10;
  const int out_f32 = mode == 2;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_f32 ? 4 : 8)) || (N % (out_f32 ? 4 : 8))) return -10;
  if (mode == 1 && (M % 128)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -12;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 64 && bn != 128 && bn != 256) bn = N >= 1024 ? 256 : (N >= 512 ? 128 : 64);
  CUtensorMap ta, tb;
  int r;
  const int a_mn = mode == 2;
  if (mode == 2) b_mn = 1;
  if (!a_mn) r = make_tmap_bf16_2d(&ta, A, M, K, lda, BM, BK);
  else r = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, 64);
  if (r) return r;
  if (mode == 1) {
    if (!b_mn) r = make_tmap_bf16_2d(&tb, B, (uint64_t)n_groups * group_b_rows, K, ldb, bn, BK);
    else r = make_tmap_bf16_2d(&tb, B, (uint64_t)n_groups * group_b_rows, N, ldb, BK, 64);
  } else {
    r = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, 64);
  }
  if (r) return r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.out_f32 = out_f32; p.accumulate = out_f32 ? accumulate : 0;
  p.k_splits = 1; p.alpha = 1.f; p.status = status;
  p.group_mode = mode; p.tile_group = tile_group; p.group_b_rows = group_b_rows; p.group_offsets = group_offsets;
  p.n_groups = n_groups; p.group_c_stride = group_c_stride;
  static PeerMaps no_peers;
#define B200_DISPATCH(BN_)                                                                            \
  if (!a_mn && !b_mn) return launch<BN_, false, false>(ta, tb, no_peers, p, g_sm_count, stream);     \
  if (!a_mn && b_mn) return launch<BN_, false, true>(ta, tb, no_peers, p, g_sm_count, stream);       \
  return launch<BN_, true, true>(ta, tb, no_peers, p, g_sm_count, stream);
  if (bn == 256) { B200_DISPATCH(256) }
  if (bn == 128) { B200_DISPATCH(128) }
  B200_DISPATCH(64)
#undef B200_DISPATCH
}


// fp8 GEMM: C[M,N] (bf16) = alpha * (*alpha_dev) * A[M,K] (e4m3) @ B[N,K]^T (e4m3) (+ bias)(+ residual), fp32
// accumulation in tensor memory. alpha_dev (optional, device) carries the product of the per-tensor quantisation
// scales so that no host read is needed. lda / ldb in elements (= bytes), multiples of 16.
extern "C" int b200_gemm_e4m3(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                              int N, int K, int lda, int ldb, int ldc, float alpha, const float* alpha_dev, int bn,
                              int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (ldc % 8) || (N % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -12;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (bn != 64 && bn != 128 && bn != 256) bn = (N >= 2048 || (long long)M * N >= (long long)128 * 256 * 148) ? 256 : (N >= 512 ? 128 : 64);
  CUtensorMap ta, tb;
  int r = make_tmap_u8_2d(&ta, A, M, K, lda, BM);
  if (r) return r;
  r = make_tmap_u8_2d(&tb, B, N, K, ldb, bn);
  if (r) return r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.k_splits = 1; p.alpha = alpha; p.alpha_dev = alpha_dev; p.status = status;
  p.fp8 = 1;
  static PeerMaps no_peers;
  if (bn == 256) return launch<256, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
  if (bn == 128) return launch<128, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
  return launch<64, false, false>(ta, tb, no_peers, p, g_sm_count, stream);
}
