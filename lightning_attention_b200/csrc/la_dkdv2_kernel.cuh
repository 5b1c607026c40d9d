// Fused dk + dv kernel: one reverse-time sweep that reads q, k, v, do once and writes dk and dv.
//
//   dk_t = sum_{j>=t} lambda^(j-t) (v_t . do_j) q_j        dv_t = sum_{j>=t} lambda^(j-t) (k_t . q_j) do_j
//
// These are the two reverse-time instances of the generic product in la_kernels.cuh, (A, Bm, C) = (v, do, q) and
// (k, q, do) (lightning_attn2.py:156-162 in-block, :335-395 across blocks). Run separately they read six tensors;
// here the q and do tiles are shared and both halves use ONE running state, dKV = sum_t lambda^t q_t^T do_t
// (d x e, lightning_attn2.py:392-395): the dk term reads its bf16 copy as a K-major operand (v . dKV^T), the dv term
// as an MN-major operand (k . dKV), so no transpose is needed.
//
// Per 128-token block, with r = row in the block and w(r) = lambda^(128-r):
//   S0 = v do^T -> TMEM region SA        S1 = k q^T -> TMEM region SB               (two regions: the two mask passes and
//   P0 = mask(S0) -> SA[0,64)            P1 = mask(S1) -> SB[0,64)                   their MMAs overlap)
//   Vs = w v      -> SA[64,128)          Ks = w k      -> SB[64,128)                (bf16, written with tcgen05.st)
//   dk = [P0 | Vs] [q ; dKV^T]           dv = [P1 | Ks] [do ; dKV]                  (ONE accumulator each: the cross-block
//                                                                                    term is a second K range of the same
//                                                                                    tcgen05.mma chain, A read from TMEM)
//   D  = (lambda^r q)^T do ;  dKV <- lambda^128 dKV + D                             (fp32 registers + bf16 copy in smem)
// Shared memory: do double-buffered; q, k, v single-buffered (k and v are free as soon as their S product and scaled copy
// are done; q is free once D, issued right after the dk half, has read it); one 32 KB staging buffer through which the dk
// tile and then the dv tile of a block leave by TMA store (row-per-thread stores straight from registers to global
// memory were measured 1500 cycles per block slower: 32 distinct lines per warp instruction).
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer (one thread), warps 2-5 mask group (one per TMEM lane quadrant),
// warps 6-13 state/output group. Every wait is bounded and polls a CTA-wide abort flag.
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
  int layout;
  long long wait_budget;
  long long* trace;        // optional clock stamps (see lab200_la_debug_trace), LA_TRACE_SLOTS per block
  int trace_blocks;
};

// barrier slots; every slot has two instances indexed by block parity
enum : int {
  LD2_FULL_Q = 0, LD2_FULL_G, LD2_FULL_V, LD2_FULL_K,
  LD2_S0_READY, LD2_S1_READY, LD2_P0_READY, LD2_P1_READY, LD2_VS_READY, LD2_KS_READY,
  LD2_PC0_DONE, LD2_PC1_DONE, LD2_O_FREE0, LD2_O_FREE1, LD2_O_STAGED0, LD2_O_STAGED1, LD2_BUF_FREE0, LD2_BUF_FREE1,
  LD2_Q_SCALED, LD2_D_DONE, LD2_D_FREE, LD2_STATE_READY, LD2_NUM_BARS
};

template <int ND, int NE, int FMT>
__global__ void __launch_bounds__(LAP_THREADS, 1)
la_dkdv2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
                const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV, const LaDkdvParams p) {
  static_assert(ND <= 2 && NE <= 2, "d, e <= 128");
  constexpr int SLAB = LA_SLAB_BYTES;
  constexpr int DQ = 64 * ND, DE = 64 * NE;
  constexpr int SC = DE / 2;  // state columns per thread (state rows = d index, columns = e index)
  constexpr uint32_t T_SA = 0, T_SB = 128, T_O = 256, T_D = 384;
  constexpr uint32_t T_XA = 64;  // offset of the scaled A-operand copy inside an S region
  constexpr uint32_t IDESC_S = umma_idesc(FMT, 128, 128, 0, 0);
  constexpr uint32_t IDESC_X0 = umma_idesc(FMT, 128, DQ, 0, 0);   // Vs . dKV^T : state copy as K-major B, N = d
  constexpr uint32_t IDESC_X1 = umma_idesc(FMT, 128, DE, 0, 1);   // Ks . dKV   : state copy as MN-major B, N = e
  constexpr uint32_t IDESC_PC0 = umma_idesc(FMT, 128, DQ, 0, 1);  // P0 . q
  constexpr uint32_t IDESC_PC1 = umma_idesc(FMT, 128, DE, 0, 1);  // P1 . do
  constexpr uint32_t IDESC_D = umma_idesc(FMT, 128, DE, 1, 1);    // (w q)^T . do

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sQ = base;                 // 2 slabs
  const uint32_t sG = sQ + 2 * SLAB;        // 2 stages x 2 slabs
  const uint32_t sK = sG + 4 * SLAB;        // 2 slabs
  const uint32_t sV = sK + 2 * SLAB;        // 2 slabs
  const uint32_t sO = sV + 2 * SLAB;        // 2 slabs: staging of the dk tile, then of the dv tile
  const uint32_t sS = sO + 2 * SLAB;        // bf16 copy of dKV: NE slabs of [128 rows (d)][64 columns (e)]
  const uint32_t sBar = sS + NE * SLAB;
  const uint32_t sMisc = sBar + 2 * LD2_NUM_BARS * 8;
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
  const int zc = p.layout ? (bh / p.h) * p.n * p.h + (bh % p.h) : bh;  // third tensor-map coordinate of this pair
  auto blk_of = [&](int i) { return blk_end - 1 - i; };  // reverse time

  const float s = p.slopes ? p.slopes[bh % p.h] : 0.f;
  const float s2 = -s * 1.4426950408889634f;

  if (tid == 0) {
    for (int i = 0; i < LD2_NUM_BARS; ++i) {
      uint32_t count = 1u;
      if (i == LD2_P0_READY || i == LD2_P1_READY) count = LAP_MASK_THREADS;
      if (i == LD2_VS_READY || i == LD2_KS_READY || i == LD2_O_FREE0 || i == LD2_O_FREE1 || i == LD2_Q_SCALED ||
          i == LD2_D_FREE || i == LD2_STATE_READY || i == LD2_O_STAGED0 || i == LD2_O_STAGED1)
        count = LAP_STATE_THREADS;
      mbar_init(sBar + (i * 2) * 8, count);
      mbar_init(sBar + (i * 2 + 1) * 8, count);
    }
    *abort_flag = 0;
    *fail_code = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmG);
    tma_prefetch_desc(&tmDK); tma_prefetch_desc(&tmDV);
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

#define LD2_FAIL(code) { if (*fail_code == 0) *fail_code = (code); }
#define LD2_STAMP(slot, it) if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && (it) < p.trace_blocks) \
    p.trace[(it) * LA_TRACE_SLOTS + (slot)] = clock64();
#ifdef LD2_MASK_TRACE  // debugging build: only the MMA warp's block start (slot 0) and the fine stamps of one mask warp
#define LD2_TRACE(slot, it) if ((slot) == 0) { LD2_STAMP(slot, it) }
#define LD2_TRACE_M(slot, it) LD2_STAMP(slot, it)
#else
#define LD2_TRACE(slot, it) LD2_STAMP(slot, it)
#define LD2_TRACE_M(slot, it)
#endif
#define LD2_WAIT(which, it, code) if (!lap_wait(bar(which, it), par(it), abort_flag, budget)) { LD2_FAIL(code) break; }

  if (warp == 0) {
    // =========================================== TMA producer ===========================================
    // Loads of block it are issued as their buffers come free during block it-1; in between, the two staged output tiles of
    // block it-1 are stored. The order below is the order in which these events happen in a block.
    if (lane == 0) {
      auto store_tile = [&](int i, int u) -> bool {  // tile u (0: dk, 1: dv) of block i: staged -> global, then free the buffer
        if (!lap_wait(bar(u ? LD2_O_STAGED1 : LD2_O_STAGED0, i), par(i), abort_flag, budget)) return false;
        const int nslab = u ? NE : ND;
        for (int sl = 0; sl < nslab; ++sl)
          tma_store_3d(u ? static_cast<const void*>(&tmDV) : static_cast<const void*>(&tmDK), sO + sl * SLAB, sl * 64,
                       blk_of(i) * LA_BLOCK, zc);
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(bar(u ? LD2_BUF_FREE1 : LD2_BUF_FREE0, i));
        return true;
      };
      bool alive = true;
      for (int it = 0; it < nb; ++it) {
        const int blk = blk_of(it);
        const int st = it & 1;
        alive = false;
#if defined(LD2_PF)
        if (it + 1 < nb) {
          const int nblk = blk_of(it + 1);
          for (int sl = 0; sl < NE; ++sl) tma_prefetch_l2_3d(&tmV, sl * 64, nblk * LA_BLOCK, zc);
          for (int sl = 0; sl < ND; ++sl) tma_prefetch_l2_3d(&tmK, sl * 64, nblk * LA_BLOCK, zc);
#if LD2_PF >= 2
          for (int sl = 0; sl < 2; ++sl) tma_prefetch_l2_3d(&tmQ, sl * 64, nblk * LA_BLOCK, zc);
#endif
        }
#endif
        // do: P1 do of block it-2 was the last reader of this stage
        if (it >= 2) { LD2_WAIT(LD2_PC1_DONE, it - 2, LA_ERR_WAIT_MMA2) }
        mbar_arrive_expect_tx(bar(LD2_FULL_G, it), NE * SLAB);
        for (int sl = 0; sl < NE; ++sl)
          tma_load_3d(sG + (st * 2 + sl) * SLAB, &tmG, sl * 64, blk * LA_BLOCK, zc, bar(LD2_FULL_G, it));
        // v of the previous block: S0 has consumed it (P0 exists) and its scaled copy sits in TMEM
        if (it >= 1) { LD2_WAIT(LD2_VS_READY, it - 1, LA_ERR_WAIT_MMA1) }
        mbar_arrive_expect_tx(bar(LD2_FULL_V, it), NE * SLAB);
        for (int sl = 0; sl < NE; ++sl) tma_load_3d(sV + sl * SLAB, &tmV, sl * 64, blk * LA_BLOCK, zc, bar(LD2_FULL_V, it));
        if (it >= 1 && !store_tile(it - 1, 0)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
        // q of the previous block: D was its last reader
        if (it >= 1) { LD2_WAIT(LD2_D_DONE, it - 1, LA_ERR_WAIT_MMA2) }
        mbar_arrive_expect_tx(bar(LD2_FULL_Q, it), 2 * SLAB);
        for (int sl = 0; sl < 2; ++sl)  // q always as two slabs: it is the M = 128 side of the state MMA
          tma_load_3d(sQ + sl * SLAB, &tmQ, sl * 64, blk * LA_BLOCK, zc, bar(LD2_FULL_Q, it));
        if (it >= 1) { LD2_WAIT(LD2_KS_READY, it - 1, LA_ERR_WAIT_MMA1) }
        mbar_arrive_expect_tx(bar(LD2_FULL_K, it), ND * SLAB);
        for (int sl = 0; sl < ND; ++sl) tma_load_3d(sK + sl * SLAB, &tmK, sl * 64, blk * LA_BLOCK, zc, bar(LD2_FULL_K, it));
        if (it >= 1 && !store_tile(it - 1, 1)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
        alive = true;
      }
      if (alive && nb > 0 && *abort_flag == 0) {
        if (!store_tile(nb - 1, 0) || !store_tile(nb - 1, 1)) LD2_FAIL(LA_ERR_WAIT_MMA2)
      }
      tma_store_wait_all();
    }
  } else if (warp == 1) {
    // ============================================ MMA issuer ============================================
    // Issue order per block: [P0 q, Vs dKV^T] -> dk; S0 of the next block; D (the last reader of q, whose buffer is then
    // reloaded); [P1 do, Ks dKV] -> dv; S1 of the next block. The two S products of block it+1 are in TMEM before the mask
    // group gets to them.
    if (lane == 0) {
      auto issue_S0 = [&](int i) -> bool {  // S0 = v do^T (contraction over e)
        if (!lap_wait(bar(LD2_FULL_V, i), par(i), abort_flag, budget)) return false;
        if (!lap_wait(bar(LD2_FULL_G, i), par(i), abort_flag, budget)) return false;
        tc_fence_after_sync();
        const uint32_t g0 = sG + (i & 1) * 2 * SLAB;
        for (int kq = 0; kq < ne16; ++kq) {
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_SA, smem_desc_sw128(sV + off, 16), smem_desc_sw128(g0 + off, 16), IDESC_S, kq > 0);
        }
        umma_commit(bar(LD2_S0_READY, i));
        return true;
      };
      auto issue_S1 = [&](int i) -> bool {  // S1 = k q^T (contraction over d)
        if (!lap_wait(bar(LD2_FULL_K, i), par(i), abort_flag, budget)) return false;
        if (!lap_wait(bar(LD2_FULL_Q, i), par(i), abort_flag, budget)) return false;
        tc_fence_after_sync();
        const uint32_t q0 = sQ;
        for (int kq = 0; kq < nd16; ++kq) {
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_SB, smem_desc_sw128(sK + off, 16), smem_desc_sw128(q0 + off, 16), IDESC_S, kq > 0);
        }
        umma_commit(bar(LD2_S1_READY, i));
        return true;
      };
      bool alive = true;
      if (nb > 0) {
        alive = issue_S0(0) && issue_S1(0);
        if (!alive) LD2_FAIL(LA_ERR_WAIT_INPUT)
      }
      for (int it = 0; it < nb && alive; ++it) {
        const uint32_t sQs = sQ, sGs = sG + (it & 1) * 2 * SLAB;
        const bool have_state = have_state_in || (it > 0);
        LD2_TRACE(0, it)
        // ---- dk = P0 q + Vs dKV^T -------------------------------------------------------------------------------
        LD2_WAIT(LD2_P0_READY, it, LA_ERR_WAIT_MMA1)
        if (it > 0) { LD2_WAIT(LD2_O_FREE1, it - 1, LA_ERR_WAIT_MMA2) }  // the dv epilogue of the previous block has read O
        LD2_TRACE(1, it)
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_O, tmem + T_SA + kk * 8, smem_desc_sw128(sQs + kk * 2048, SLAB), IDESC_PC0, kk > 0);
        if (have_state) {
          LD2_WAIT(LD2_VS_READY, it, LA_ERR_WAIT_MMA2)
          LD2_WAIT(LD2_STATE_READY, it, LA_ERR_WAIT_MMA2)
          tc_fence_after_sync();
          for (int kq = 0; kq < ne16; ++kq) {  // contraction over e: state copy columns
            const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
            umma_f16_ts(tmem + T_O, tmem + T_SA + T_XA + kq * 8, smem_desc_sw128(sS + off, 16), IDESC_X0, 1);
          }
        }
        umma_commit(bar(LD2_PC0_DONE, it));
        LD2_TRACE(2, it)
        if (it + 1 < nb) {
          if (!issue_S0(it + 1)) { LD2_FAIL(LA_ERR_WAIT_INPUT) break; }
        }
        LD2_TRACE(3, it)
        // ---- D = (w_state q)^T do ------------------------------------------------------------------------------
        LD2_WAIT(LD2_Q_SCALED, it, LA_ERR_WAIT_MMA2)
        if (it > 0) { LD2_WAIT(LD2_D_FREE, it - 1, LA_ERR_WAIT_MMA2) }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem + T_D, smem_desc_sw128(sQs + kk * 2048, SLAB), smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_D, kk > 0);
        umma_commit(bar(LD2_D_DONE, it));
        LD2_TRACE(7, it)
        // ---- dv = P1 do + Ks dKV -----------------------------------------------------------------------------------
        LD2_WAIT(LD2_P1_READY, it, LA_ERR_WAIT_MMA1)
        LD2_WAIT(LD2_O_FREE0, it, LA_ERR_WAIT_MMA2)  // the dk epilogue has read O
        LD2_TRACE(4, it)
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_O, tmem + T_SB + kk * 8, smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_PC1, kk > 0);
        if (have_state) {
          LD2_WAIT(LD2_KS_READY, it, LA_ERR_WAIT_MMA2)
          tc_fence_after_sync();
          for (int kq = 0; kq < nd16; ++kq)  // contraction over d: state copy rows
            umma_f16_ts(tmem + T_O, tmem + T_SB + T_XA + kq * 8, smem_desc_sw128(sS + kq * 2048, SLAB), IDESC_X1, 1);
        }
        umma_commit(bar(LD2_PC1_DONE, it));
        LD2_TRACE(5, it)
        if (it + 1 < nb) {
          if (!issue_S1(it + 1)) { LD2_FAIL(LA_ERR_WAIT_INPUT) break; }
        }
        LD2_TRACE(6, it)
      }
    }
  } else if (warp < 6) {
    // ============================================ mask group ============================================
    // Reverse-time mask on both products: keep c >= r with lambda^(c-r). One warp per TMEM lane quadrant, four 32-column
    // tiles each, in column order; P tile t goes back over S columns [16 t, 16 t + 16), which the warp has read by then.
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
        const uint32_t T_S = u ? T_SB : T_SA;
        bool ok = lap_wait(bar(u ? LD2_S1_READY : LD2_S0_READY, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA1) alive = false; break; }
        if (q == 0 && lane == 0) { LD2_TRACE(8 + 2 * u, it) }
        if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(15, it) }
        tc_fence_after_sync();
#pragma unroll 1
        for (int t = 0; t < 4; ++t) {
          const int c0 = t * 32;
          const int kind = (t == q) ? 2 : ((t > q) ? 1 : 0);  // 0 dead, 1 live, 2 diagonal; warp-uniform
          uint32_t v[32];
          if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(t * 3 + 1, it) }
          if (kind) {
            tmem_ld32(tmem + lanebase + T_S + c0, v);
            tmem_wait_ld();
          }
          if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(t * 3 + 2, it) }
          uint32_t pk[16];
          if (kind == 1) {
            const float rowf = decay_tab[c0 - r];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              pk[i >> 1] = pack2<FMT>(__uint_as_float(v[i]) * (rowf * g[i]), __uint_as_float(v[i + 1]) * (rowf * g[i + 1]));
          } else if (kind == 2 && diag_rank1) {
            // Masked elements (column i < lane) are zeroed by AND-ing the value's bits with a sign mask, not by a select on
            // the product: the compiler turned 32 selects into 32 branches per tile, and the diagonal tile, ~150 instructions
            // otherwise, then took ~2,800 cycles (clock stamps), which made the mask passes the bound of the whole kernel.
            float rd = rowd;
            asm volatile("" : "+f"(rd));  // keeps the 32 products rd * g[i] from being hoisted out of the block loop into registers
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint32_t k0 = ~static_cast<uint32_t>((i - lane) >> 31), k1 = ~static_cast<uint32_t>((i + 1 - lane) >> 31);
              pk[i >> 1] = pack2<FMT>(__uint_as_float(v[i] & k0) * (rd * g[i]), __uint_as_float(v[i + 1] & k1) * (rd * g[i + 1]));
            }
          } else if (kind == 2) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int d0 = i - lane, d1 = d0 + 1;
              const uint32_t k0 = ~static_cast<uint32_t>(d0 >> 31), k1 = ~static_cast<uint32_t>(d1 >> 31);
              const float m0 = decay_tab[max(d0, 0)], m1 = decay_tab[max(d1, 0)];
              pk[i >> 1] = pack2<FMT>(__uint_as_float(v[i] & k0) * m0, __uint_as_float(v[i + 1] & k1) * m1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) pk[i] = 0u;
          }
          tmem_st16(tmem + lanebase + T_S + t * 16, pk);
          if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(t * 3 + 3, it) }
        }
        if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(13, it) }
        tmem_wait_st();
        if (q == 0 && lane == 0 && u == 1) { LD2_TRACE_M(14, it) }
        tc_fence_before_sync();
        mbar_arrive(bar(u ? LD2_P1_READY : LD2_P0_READY, it));
        if (q == 0 && lane == 0) { LD2_TRACE(9 + 2 * u, it) }
      }
    }
  } else {
    // ========================================= state / output group =====================================
    const int w8 = warp - 6;
    const int q = warp & 3, hf = w8 >> 2;
    const int r = q * 32 + lane;
    const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
    const float w_out = ex2f(s2 * static_cast<float>(LA_BLOCK - r));  // reverse time
    const uint32_t w_out2 = pack2<FMT>(w_out, w_out);
    const float w_state = ex2f(s2 * static_cast<float>(r));
    const uint32_t w_state2 = pack2<FMT>(w_state, w_state);
    const float decay_blk = ex2f(s2 * static_cast<float>(LA_BLOCK));
    const bool st_row_valid = (r < p.d);
    const bool tracer = (w8 == 0 && lane == 0);

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
    mbar_arrive(bar(LD2_STATE_READY, 0));  // state entering block 0

    // Row r of a [128][64 NS] shared-memory tile, scaled by w(r), as the A operand of a TMEM-sourced MMA: this thread's
    // half of the row's 16-byte chunks -> bf16 pairs -> TMEM columns [T + 4 * chunk, ...).
    auto scaled_copy_to_tmem = [&](auto ns_tag, uint32_t tile, uint32_t tcol) {
      constexpr int NS = decltype(ns_tag)::value;
      constexpr int NCH = NS * 4;  // chunks per thread
      uint32_t u[NCH][4];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int gch = hf * NCH + c;  // chunk index in the row, 0 .. NS*8-1
        ld_shared_v4(tile + (gch >> 3) * SLAB + r * 128 + ((((gch & 7) ^ (r & 7))) << 4), u[c][0], u[c][1], u[c][2], u[c][3]);
      }
#pragma unroll
      for (int c4 = 0; c4 < NCH; c4 += 4) {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int j = 0; j < 4; ++j) pk[c * 4 + j] = mul2<FMT>(u[c4 + c][j], w_out2);
        }
        tmem_st16(tmem + lanebase + tcol + (hf * NCH + c4) * 4, pk);
      }
      tmem_wait_st();
      tc_fence_before_sync();
    };

    // epilogue of half U: O -> registers -> swizzled tile in the staging buffer (dk for U = 0, dv for U = 1); the producer
    // warp stores it. The buffer is free once the previous tile (the other half) has been read by its TMA store.
    auto epilogue = [&](auto u_tag, int it) -> bool {
      constexpr int U = decltype(u_tag)::value;
      constexpr int OC = (U == 0 ? DQ : DE) / 2;
      bool ok = lap_wait(bar(U ? LD2_PC1_DONE : LD2_PC0_DONE, it), par(it), abort_flag, budget);
      if (U == 1) ok = ok && lap_wait(bar(LD2_BUF_FREE0, it), par(it), abort_flag, budget);
      if (U == 0 && it > 0) ok = ok && lap_wait(bar(LD2_BUF_FREE1, it - 1), par(it - 1), abort_flag, budget);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return false;
      tc_fence_after_sync();
#pragma unroll
      for (int cc = 0; cc < OC; cc += 16) {
        uint32_t a[16];
        tmem_ld16(tmem + lanebase + T_O + hf * OC + cc, a);
        tmem_wait_ld();
        if (cc + 16 >= OC) {
          tc_fence_before_sync();
          mbar_arrive(bar(U ? LD2_O_FREE1 : LD2_O_FREE0, it));
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int col = hf * OC + cc + g * 8;
          st_shared_v4(sO + (col >> 6) * SLAB + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4),
                       pack2<FMT>(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1])),
                       pack2<FMT>(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3])),
                       pack2<FMT>(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5])),
                       pack2<FMT>(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7])));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(bar(U ? LD2_O_STAGED1 : LD2_O_STAGED0, it));
      return true;
    };

    for (int it = 0; it < nb; ++it) {
      const bool has_next = (it + 1 < nb);
      // ---- Vs = w v into SA[64, 128): the mask group is done with S0 ----------------------------------------------
      {
        bool ok = lap_wait(bar(LD2_P0_READY, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA1) break; }
        tc_fence_after_sync();
        scaled_copy_to_tmem(std::integral_constant<int, NE>{}, sV, T_SA + T_XA);
        mbar_arrive(bar(LD2_VS_READY, it));
        if (tracer) { LD2_TRACE(12, it) }
      }
      // ---- dk tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 0>{}, it)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
      if (tracer) { LD2_TRACE(13, it) }
      // ---- q rows *= w_state(r), in place, for D: S1 and P0 q are done with the unscaled tile -------------------------
      {
        bool ok = lap_wait(bar(LD2_S1_READY, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA1) break; }
        if (s != 0.f) {
          constexpr int NCH = ND * 4;  // 16-byte chunks per thread: this thread's half of row r
          uint32_t u[NCH][4];
          uint32_t addr[NCH];
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            const int gch = hf * NCH + c;
            const int ks = gch >> 3, p0 = gch & 7;
            const int pos = (NCH >= 8) ? ((p0 + r) & 7) : ((p0 & 4) | ((p0 + r) & 3));
            addr[c] = sQ + ks * SLAB + r * 128 + (pos << 4);
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
        mbar_arrive(bar(LD2_Q_SCALED, it));
      }
      // ---- Ks = w k into SB[64, 128) ---------------------------------------------------------------------------------
      {
        bool ok = lap_wait(bar(LD2_P1_READY, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA1) break; }
        tc_fence_after_sync();
        scaled_copy_to_tmem(std::integral_constant<int, ND>{}, sK, T_SB + T_XA);
        mbar_arrive(bar(LD2_KS_READY, it));
        if (tracer) { LD2_TRACE(14, it) }
      }
      // ---- state recurrence: dKV = lambda^128 dKV + D (registers; the shared-memory copy follows the dv half) ---------
      {
        bool ok = lap_wait(bar(LD2_D_DONE, it), par(it), abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
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
      mbar_arrive(bar(LD2_D_FREE, it));
      // ---- dv tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 1>{}, it)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
      if (has_next) {  // PC1_DONE (awaited by the dv epilogue) covers both halves of this block: they are done with the old copy
        store_state_smem();
        fence_proxy_async_smem();
        mbar_arrive(bar(LD2_STATE_READY, it + 1));
      }
      if (tracer) { LD2_TRACE(15, it) }
    }
    if (*abort_flag == 0 && p.state_out != nullptr && st_row_valid) {
      float* dst = p.state_out + ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.d + r) * p.e + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.e) *reinterpret_cast<float4*>(dst + i) = make_float4(stt[i], stt[i + 1], stt[i + 2], stt[i + 3]);
      }
    }
  }
#undef LD2_WAIT
#undef LD2_TRACE
#undef LD2_TRACE_M
#undef LD2_STAMP
#undef LD2_FAIL

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, *fail_code ? *fail_code : LA_ERR_WAIT_MMA2);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace lab200
