// Fused dk + dv kernel: one reverse-time sweep that reads q, k, v, do once and writes dk and dv.
//
//   dk_t = sum_{j>=t} lambda^(j-t) (v_t . do_j) q_j        dv_t = sum_{j>=t} lambda^(j-t) (k_t . q_j) do_j
//
// These are the two reverse-time instances of the generic product in la_kernels.cuh, (A, Bm, C) = (v, do, q) and
// (k, q, do). Run separately they read six tensors; here each 128-token block goes through the same TMEM buffers
// twice (sub-iteration u = 0 for dk, u = 1 for dv) with the q and do tiles shared, and both use ONE running state,
// dKV = sum_t lambda^t q_t^T do_t (d x e, lightning_attn2.py:392-395): the dk term reads its bf16 copy as a K-major
// operand (v . dKV^T), the dv term as an MN-major operand (k . dKV), so no transpose is needed.
//
// Roles, barriers and data layout follow la_pipe_kernel.cuh: warp 0 TMA producer (+ TMA stores), warp 1 MMA issuer,
// warps 2-5 mask group, warps 6-13 state/output group. q and do are double-buffered; k and v are single-buffered and,
// once S and X of their sub-iteration are done, double as staging buffers for the dv / dk output tiles.
#pragma once
#include <type_traits>

#include "la_pipe_kernel.cuh"

namespace lab200 {

struct LaDkdvParams {
  const float* slopes;     // [h] decay rates or nullptr
  const float* state_in;   // [bh][state_slots][d][e] fp32 reverse-time state entering the (chunk of the) sequence, or nullptr
  float* state_out;        // same indexing, or nullptr
  int* status;
  int n, h, d, e;
  int nblocks, blocks_per_chunk, chunk0, state_slots;
  long long wait_budget;
  long long* trace;        // optional clock stamps (see lab200_la_debug_trace), LA_TRACE_SLOTS per block
  int trace_blocks;
};

// barrier slots; every slot has two instances indexed by block parity
enum : int {
  LDK_FULL_QG = 0, LDK_FULL_V, LDK_FULL_K,
  LDK_S_READY0, LDK_S_READY1, LDK_P_READY0, LDK_P_READY1, LDK_A_FREE0, LDK_A_FREE1, LDK_PC_DONE0, LDK_PC_DONE1,
  LDK_O_FREE0, LDK_O_FREE1, LDK_O_STAGED0, LDK_O_STAGED1,
  LDK_Q_SCALED, LDK_D_DONE, LDK_D_FREE, LDK_STATE_READY, LDK_NUM_BARS
};

template <int ND, int NE, int FMT>
__global__ void __launch_bounds__(LAP_THREADS, 1)
la_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
               const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, const LaDkdvParams p) {
  static_assert(ND <= 2 && NE <= 2, "d, e <= 128");
  constexpr int SLAB = LA_SLAB_BYTES;
  constexpr int DQ = 64 * ND, DE = 64 * NE;
  constexpr int SC = DE / 2;  // state columns per thread (state rows = d index, columns = e index)
  constexpr uint32_t T_S = 0, T_OI = 128, T_OX = 256, T_D = 384;
  constexpr uint32_t IDESC_S = umma_idesc(FMT, 128, 128, 0, 0);
  constexpr uint32_t IDESC_X0 = umma_idesc(FMT, 128, DQ, 0, 0);   // v . dKV^T : state copy as K-major B, N = d
  constexpr uint32_t IDESC_X1 = umma_idesc(FMT, 128, DE, 0, 1);   // k . dKV   : state copy as MN-major B, N = e
  constexpr uint32_t IDESC_PC0 = umma_idesc(FMT, 128, DQ, 0, 1);  // P0 . q
  constexpr uint32_t IDESC_PC1 = umma_idesc(FMT, 128, DE, 0, 1);  // P1 . do
  constexpr uint32_t IDESC_D = umma_idesc(FMT, 128, DE, 1, 1);    // (w q)^T . do

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sQ = base;                 // 2 stages x 2 slabs
  const uint32_t sG = sQ + 4 * SLAB;        // 2 stages x 2 slabs
  const uint32_t sK = sG + 4 * SLAB;        // 2 slabs (also staging for the dv tile)
  const uint32_t sV = sK + 2 * SLAB;        // 2 slabs (also staging for the dk tile)
  const uint32_t sS = sV + 2 * SLAB;        // bf16 copy of dKV: NE slabs of [128 rows (d)][64 columns (e)]
  const uint32_t sBar = sS + NE * SLAB;
  const uint32_t sMisc = sBar + 2 * LDK_NUM_BARS * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sMisc - raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (sMisc + 4 - raw));
  volatile int* fail_code = reinterpret_cast<volatile int*>(smem_raw + (sMisc + 8 - raw));
  volatile float* decay_tab = reinterpret_cast<volatile float*>(smem_raw + (sMisc + 16 - raw));
  auto bar = [&](int which, int it) -> uint32_t { return sBar + (which * 2 + (it & 1)) * 8; };
  auto par = [](int it) -> uint32_t { return static_cast<uint32_t>((it >> 1) & 1); };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int chunk = p.chunk0 + blockIdx.y;
  const int bh = blockIdx.z;
  const int blk_begin = chunk * p.blocks_per_chunk;
  const int blk_end = min(p.nblocks, blk_begin + p.blocks_per_chunk);
  const int nb = blk_end - blk_begin;
  const int nd16 = p.d >> 4, ne16 = p.e >> 4;
  const long long budget = p.wait_budget;
  const bool have_state_in = (p.state_in != nullptr);
  auto blk_of = [&](int i) { return blk_end - 1 - i; };  // reverse time

  const float s = p.slopes ? p.slopes[bh % p.h] : 0.f;
  const float s2 = -s * 1.4426950408889634f;

  if (tid == 0) {
    for (int i = 0; i < LDK_NUM_BARS; ++i) {
      uint32_t count = 1u;
      if (i == LDK_P_READY0 || i == LDK_P_READY1) count = LAP_MASK_THREADS;
      if (i == LDK_O_FREE0 || i == LDK_O_FREE1 || i == LDK_O_STAGED0 || i == LDK_O_STAGED1 || i == LDK_Q_SCALED ||
          i == LDK_D_FREE || i == LDK_STATE_READY)
        count = LAP_STATE_THREADS;
      mbar_init(sBar + (i * 2) * 8, count);
      mbar_init(sBar + (i * 2 + 1) * 8, count);
    }
    *abort_flag = 0;
    *fail_code = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmG); tma_prefetch_desc(&tmDK); tma_prefetch_desc(&tmDV);
  }
  if (tid < LA_BLOCK) decay_tab[tid] = ex2f(s2 * static_cast<float>(tid));
  if (warp == 0) {
    tmem_alloc(sMisc, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

#define LDK_FAIL(code) { if (*fail_code == 0) *fail_code = (code); }
#define LDK_TRACE(slot, it) if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && (it) < p.trace_blocks) \
    p.trace[(it) * LA_TRACE_SLOTS + (slot)] = clock64();
#define LDK_WAIT(which, it, code) if (!lap_wait(bar(which, it), par(it), abort_flag, budget)) { LDK_FAIL(code) break; }

  if (warp == 0) {
    // =========================================== TMA producer ===========================================
    if (lane == 0) {
      auto store_tile = [&](int i, int u) -> bool {  // output tile of block i, sub-iteration u (0: dk from sV, 1: dv from sK)
        if (!lap_wait(bar(u ? LDK_O_STAGED1 : LDK_O_STAGED0, i), par(i), abort_flag, budget)) return false;
        const int nslab = u ? NE : ND;
        for (int sl = 0; sl < nslab; ++sl)
          tma_store_3d(u ? static_cast<const void*>(&tmDV) : static_cast<const void*>(&tmDK), (u ? sK : sV) + sl * SLAB,
                       sl * 64, blk_of(i) * LA_BLOCK, bh);
        tma_store_commit();
        return true;
      };
      bool alive = true;
      for (int it = 0; it < nb; ++it) {
        const int blk = blk_of(it);
        const int st = it & 1;
        if (it >= 2) {  // q, do stage reuse: D of block it-2 was their last reader
          if (!lap_wait(bar(LDK_D_DONE, it - 2), par(it - 2), abort_flag, budget)) { LDK_FAIL(LA_ERR_WAIT_MMA2) alive = false; break; }
        }
        mbar_arrive_expect_tx(bar(LDK_FULL_QG, it), (2 + NE) * SLAB);
        for (int sl = 0; sl < 2; ++sl)  // q always as two slabs: it is the M = 128 side of the state MMA
          tma_load_3d(sQ + (st * 2 + sl) * SLAB, &tmQ, sl * 64, blk * LA_BLOCK, bh, bar(LDK_FULL_QG, it));
        for (int sl = 0; sl < NE; ++sl)
          tma_load_3d(sG + (st * 2 + sl) * SLAB, &tmG, sl * 64, blk * LA_BLOCK, bh, bar(LDK_FULL_QG, it));
        if (it >= 1) {  // the v buffer still holds the staged dk tile of block it-1
          if (!store_tile(it - 1, 0)) { LDK_FAIL(LA_ERR_WAIT_MMA2) alive = false; break; }
          tma_store_wait_read();
        }
        mbar_arrive_expect_tx(bar(LDK_FULL_V, it), NE * SLAB);
        for (int sl = 0; sl < NE; ++sl) tma_load_3d(sV + sl * SLAB, &tmV, sl * 64, blk * LA_BLOCK, bh, bar(LDK_FULL_V, it));
        if (it >= 1) {  // the k buffer still holds the staged dv tile of block it-1
          if (!store_tile(it - 1, 1)) { LDK_FAIL(LA_ERR_WAIT_MMA2) alive = false; break; }
          tma_store_wait_read();
        }
        mbar_arrive_expect_tx(bar(LDK_FULL_K, it), ND * SLAB);
        for (int sl = 0; sl < ND; ++sl) tma_load_3d(sK + sl * SLAB, &tmK, sl * 64, blk * LA_BLOCK, bh, bar(LDK_FULL_K, it));
      }
      if (alive && nb > 0 && *abort_flag == 0) {
        if (!store_tile(nb - 1, 0) || !store_tile(nb - 1, 1)) LDK_FAIL(LA_ERR_WAIT_MMA2)
      }
      tma_store_wait_all();
    }
  } else if (warp == 1) {
    // ============================================ MMA issuer ============================================
    if (lane == 0) {
      auto issue_S0 = [&](int i) -> bool {  // S0 = v do^T (contraction over e)
        if (!lap_wait(bar(LDK_FULL_V, i), par(i), abort_flag, budget)) return false;
        if (!lap_wait(bar(LDK_FULL_QG, i), par(i), abort_flag, budget)) return false;
        tc_fence_after_sync();
        const uint32_t g0 = sG + (i & 1) * 2 * SLAB;
        for (int kq = 0; kq < ne16; ++kq) {
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_S, smem_desc_sw128(sV + off, 16), smem_desc_sw128(g0 + off, 16), IDESC_S, kq > 0);
        }
        umma_commit(bar(LDK_S_READY0, i));
        return true;
      };
      bool alive = (nb > 0) ? issue_S0(0) : true;
      if (!alive) LDK_FAIL(LA_ERR_WAIT_INPUT)
      for (int it = 0; it < nb && alive; ++it) {
        const uint32_t sQs = sQ + (it & 1) * 2 * SLAB, sGs = sG + (it & 1) * 2 * SLAB;
        const bool have_state = have_state_in || (it > 0);
        LDK_TRACE(0, it)
        // ---- u = 0: X0 = v dKV^T, then PC0 = P0 q ------------------------------------------------------------
        if (have_state) {
          LDK_WAIT(LDK_STATE_READY, it, LA_ERR_WAIT_MMA2)
          if (it > 0) { LDK_WAIT(LDK_O_FREE1, it - 1, LA_ERR_WAIT_MMA2) }
          tc_fence_after_sync();
          for (int kq = 0; kq < ne16; ++kq) {
            const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
            umma_f16(tmem + T_OX, smem_desc_sw128(sV + off, 16), smem_desc_sw128(sS + off, 16), IDESC_X0, kq > 0);
          }
        }
        umma_commit(bar(LDK_A_FREE0, it));
        LDK_TRACE(1, it)
        LDK_WAIT(LDK_P_READY0, it, LA_ERR_WAIT_MMA2)
        LDK_TRACE(2, it)
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_OI, tmem + T_S + kk * 8, smem_desc_sw128(sQs + kk * 2048, SLAB), IDESC_PC0, kk > 0);
        umma_commit(bar(LDK_PC_DONE0, it));
        // ---- u = 1: S1 = k q^T, X1 = k dKV, PC1 = P1 do ---------------------------------------------------------
        LDK_WAIT(LDK_FULL_K, it, LA_ERR_WAIT_INPUT)
        tc_fence_after_sync();
        for (int kq = 0; kq < nd16; ++kq) {
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_S, smem_desc_sw128(sK + off, 16), smem_desc_sw128(sQs + off, 16), IDESC_S, kq > 0);
        }
        umma_commit(bar(LDK_S_READY1, it));
        LDK_TRACE(3, it)
        LDK_WAIT(LDK_O_FREE0, it, LA_ERR_WAIT_MMA2)  // the dk epilogue has read O_intra and O_inter
        LDK_TRACE(4, it)
        tc_fence_after_sync();
        if (have_state) {
          for (int kq = 0; kq < nd16; ++kq) {  // contraction over d: state rows
            const uint32_t offK = (kq >> 2) * SLAB + (kq & 3) * 32;
            umma_f16(tmem + T_OX, smem_desc_sw128(sK + offK, 16), smem_desc_sw128(sS + kq * 2048, SLAB), IDESC_X1, kq > 0);
          }
        }
        umma_commit(bar(LDK_A_FREE1, it));
        LDK_WAIT(LDK_P_READY1, it, LA_ERR_WAIT_MMA2)
        LDK_TRACE(5, it)
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_OI, tmem + T_S + kk * 8, smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_PC1, kk > 0);
        umma_commit(bar(LDK_PC_DONE1, it));
        // ---- S0 of the next block goes out before the state MMA so the mask group never waits for it ---------------
        if (it + 1 < nb) {
          if (!issue_S0(it + 1)) { LDK_FAIL(LA_ERR_WAIT_INPUT) break; }
        }
        LDK_TRACE(6, it)
        // ---- D = (w_state q)^T do ------------------------------------------------------------------------------
        LDK_WAIT(LDK_Q_SCALED, it, LA_ERR_WAIT_MMA2)
        if (it > 0) { LDK_WAIT(LDK_D_FREE, it - 1, LA_ERR_WAIT_MMA2) }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem + T_D, smem_desc_sw128(sQs + kk * 2048, SLAB), smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_D, kk > 0);
        umma_commit(bar(LDK_D_DONE, it));
        LDK_TRACE(7, it)
      }
    }
  } else if (warp < 6) {
    // ============================================ mask group ============================================
    // Reverse-time mask on both sub-iterations: keep c >= r with lambda^(c-r). Same tile scheme as la_pipe_kernel.
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
    float g[32];  // per-column part of the decay inside a live tile: lambda^i
#pragma unroll
    for (int i = 0; i < 32; ++i) g[i] = ex2f(s2 * static_cast<float>(i));
    // Diagonal tile: lambda^(i-lane) = g[i] * lambda^(-lane); the row factor is >= 1, at most lambda^-31, and the per-element
    // table is used instead for decay rates where it could leave the fp32 range (CTA-uniform choice).
    const bool diag_rank1 = s * 31.f < 60.f;
    const float rowd = diag_rank1 ? ex2f(-s2 * static_cast<float>(lane)) : 0.f;
    bool alive = true;
    for (int it = 0; it < nb && alive; ++it) {
#pragma unroll 1
      for (int u = 0; u < 2; ++u) {
        bool ok = lap_wait(bar(u ? LDK_S_READY1 : LDK_S_READY0, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LDK_FAIL(LA_ERR_WAIT_MMA1) alive = false; break; }
        if (q == 0 && lane == 0) { LDK_TRACE(8 + 2 * u, it) }
        tc_fence_after_sync();
#pragma unroll 1
        for (int t = 0; t < 4; ++t) {
          const int c0 = t * 32;
          const int kind = (t == q) ? 2 : ((t > q) ? 1 : 0);  // 0 dead, 1 live, 2 diagonal; warp-uniform
          uint32_t v[32];
          if (kind) {
            tmem_ld32(tmem + lanebase + T_S + c0, v);
            tmem_wait_ld();
          }
          uint32_t pk[16];
          if (kind == 1) {
            const float rowf = decay_tab[c0 - r];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              pk[i >> 1] = pack2<FMT>(__uint_as_float(v[i]) * (rowf * g[i]), __uint_as_float(v[i + 1]) * (rowf * g[i + 1]));
          } else if (kind == 2 && diag_rank1) {
            float rd = rowd;
            asm volatile("" : "+f"(rd));  // keeps the 32 products rd * g[i] from being hoisted out of the block loop into registers
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int d0 = i - lane, d1 = d0 + 1;
              const float f0 = (d0 >= 0) ? __uint_as_float(v[i]) * (rd * g[i]) : 0.f;
              const float f1 = (d1 >= 0) ? __uint_as_float(v[i + 1]) * (rd * g[i + 1]) : 0.f;
              pk[i >> 1] = pack2<FMT>(f0, f1);
            }
          } else if (kind == 2) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int d0 = i - lane, d1 = d0 + 1;
              const float m0 = decay_tab[max(d0, 0)], m1 = decay_tab[max(d1, 0)];
              const float f0 = (d0 >= 0) ? __uint_as_float(v[i]) * m0 : 0.f;
              const float f1 = (d1 >= 0) ? __uint_as_float(v[i + 1]) * m1 : 0.f;
              pk[i >> 1] = pack2<FMT>(f0, f1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = 0u;
          }
          tmem_st16(tmem + lanebase + T_S + t * 16, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar(u ? LDK_P_READY1 : LDK_P_READY0, it));
        if (q == 0 && lane == 0) { LDK_TRACE(9 + 2 * u, it) }
      }
    }
  } else {
    // ========================================= state / output group =====================================
    const int w8 = warp - 6;
    const int q = warp & 3, hf = w8 >> 2;
    const int r = q * 32 + lane;
    const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
    const float w_out = ex2f(s2 * static_cast<float>(LA_BLOCK - r));  // reverse time
    const float w_state = ex2f(s2 * static_cast<float>(r));
    const uint32_t w_state2 = pack2<FMT>(w_state, w_state);
    const float decay_blk = ex2f(s2 * static_cast<float>(LA_BLOCK));
    const bool st_row_valid = (r < p.d);

    float stt[SC];  // dKV[r][hf * SC ...]
#pragma unroll
    for (int i = 0; i < SC; ++i) stt[i] = 0.f;
    if (have_state_in && st_row_valid) {
      const float* src = p.state_in + ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.d + r) * p.e + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.e) {
          const float4 v4 = *reinterpret_cast<const float4*>(src + i);
          stt[i] = v4.x; stt[i + 1] = v4.y; stt[i + 2] = v4.z; stt[i + 3] = v4.w;
        }
      }
    }
    auto store_state_smem = [&]() {
#pragma unroll
      for (int i = 0; i < SC; i += 8) {
        const int col = hf * SC + i;
        const uint32_t addr = sS + (col >> 6) * SLAB + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4);
        st_shared_v4(addr, pack2<FMT>(stt[i], stt[i + 1]), pack2<FMT>(stt[i + 2], stt[i + 3]),
                     pack2<FMT>(stt[i + 4], stt[i + 5]), pack2<FMT>(stt[i + 6], stt[i + 7]));
      }
    };
    if (have_state_in) {
      store_state_smem();
      fence_proxy_async_smem();
    }
    mbar_arrive(bar(LDK_STATE_READY, 0));  // state entering block 0

    // epilogue of sub-iteration U: O_intra + w_out O_inter -> swizzled tile in the buffer the A operand came from
    auto epilogue = [&](auto u_tag, int it, bool have_state) -> bool {
      constexpr int U = decltype(u_tag)::value;
      constexpr int OC = (U == 0 ? DQ : DE) / 2;
      bool ok = lap_wait(bar(U ? LDK_PC_DONE1 : LDK_PC_DONE0, it), par(it), abort_flag, budget);
      ok = ok && lap_wait(bar(U ? LDK_A_FREE1 : LDK_A_FREE0, it), par(it), abort_flag, budget);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return false;
      tc_fence_after_sync();
      const uint32_t sOs = U ? sK : sV;
#pragma unroll
      for (int cc = 0; cc < OC; cc += 16) {
        uint32_t a[16], b[16];
        tmem_ld16(tmem + lanebase + T_OI + hf * OC + cc, a);
        if (have_state) tmem_ld16(tmem + lanebase + T_OX + hf * OC + cc, b);
        tmem_wait_ld();
        if (cc + 16 >= OC) {
          tc_fence_before_sync();
          mbar_arrive(bar(U ? LDK_O_FREE1 : LDK_O_FREE0, it));
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          uint32_t o4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float x0 = __uint_as_float(a[g * 8 + 2 * j]), x1 = __uint_as_float(a[g * 8 + 2 * j + 1]);
            if (have_state) {
              x0 = fmaf(w_out, __uint_as_float(b[g * 8 + 2 * j]), x0);
              x1 = fmaf(w_out, __uint_as_float(b[g * 8 + 2 * j + 1]), x1);
            }
            o4[j] = pack2<FMT>(x0, x1);
          }
          const int col = hf * OC + cc + g * 8;
          st_shared_v4(sOs + (col >> 6) * SLAB + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4), o4[0], o4[1], o4[2], o4[3]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(bar(U ? LDK_O_STAGED1 : LDK_O_STAGED0, it));
      return true;
    };

    for (int it = 0; it < nb; ++it) {
      const bool has_next = (it + 1 < nb);
      const bool have_state = have_state_in || (it > 0);
      const uint32_t sQs = sQ + (it & 1) * 2 * SLAB;
      // ---- dk tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 0>{}, it, have_state)) { LDK_FAIL(LA_ERR_WAIT_MMA2) break; }
      if (w8 == 0 && lane == 0) { LDK_TRACE(12, it) }
      // ---- q rows *= w_state(r), in place, for D: S1 (and PC0 before it) must be done with the unscaled tile ------
      {
        bool ok = lap_wait(bar(LDK_S_READY1, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LDK_FAIL(LA_ERR_WAIT_MMA1) break; }
        if (s != 0.f) {
          constexpr int NCH = ND * 4;  // 16-byte chunks per thread: this thread's half of row r
          uint32_t u[NCH][4];
          uint32_t addr[NCH];
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            const int gch = hf * NCH + c;
            const int ks = gch >> 3, p0 = gch & 7;
            const int pos = (NCH >= 8) ? ((p0 + r) & 7) : ((p0 & 4) | ((p0 + r) & 3));
            addr[c] = sQs + ks * SLAB + r * 128 + (pos << 4);
            ld_shared_v4(addr[c], u[c][0], u[c][1], u[c][2], u[c][3]);
          }
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
#pragma unroll
            for (int j = 0; j < 4; ++j) u[c][j] = mul2<FMT>(u[c][j], w_state2);
            st_shared_v4(addr[c], u[c][0], u[c][1], u[c][2], u[c][3]);
          }
          fence_proxy_async_smem();
        }
        mbar_arrive(bar(LDK_Q_SCALED, it));
        if (w8 == 0 && lane == 0) { LDK_TRACE(13, it) }
      }
      // ---- dv tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 1>{}, it, have_state)) { LDK_FAIL(LA_ERR_WAIT_MMA2) break; }
      if (w8 == 0 && lane == 0) { LDK_TRACE(14, it) }
      // ---- state recurrence: dKV = lambda^128 dKV + D ---------------------------------------------------------------
      {
        bool ok = lap_wait(bar(LDK_D_DONE, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LDK_FAIL(LA_ERR_WAIT_MMA2) break; }
      }
      tc_fence_after_sync();
#pragma unroll
      for (int cc = 0; cc < SC; cc += 32) {
        uint32_t dl[32];
        tmem_ld32(tmem + lanebase + T_D + hf * SC + cc, dl);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) stt[cc + i] = fmaf(decay_blk, stt[cc + i], __uint_as_float(dl[i]));
      }
      tc_fence_before_sync();
      mbar_arrive(bar(LDK_D_FREE, it));
      if (has_next) {  // X0 and X1 of this block are done with the old copy (A_FREE1 was awaited in the dv epilogue)
        store_state_smem();
        fence_proxy_async_smem();
        mbar_arrive(bar(LDK_STATE_READY, it + 1));
      }
      if (w8 == 0 && lane == 0) { LDK_TRACE(15, it) }
    }
    if (*abort_flag == 0 && p.state_out != nullptr && st_row_valid) {
      float* dst = p.state_out + ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.d + r) * p.e + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.e) *reinterpret_cast<float4*>(dst + i) = make_float4(stt[i], stt[i + 1], stt[i + 2], stt[i + 3]);
      }
    }
  }
#undef LDK_WAIT
#undef LDK_TRACE
#undef LDK_FAIL

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, *fail_code ? *fail_code : LA_ERR_WAIT_MMA2);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace lab200
