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
// Shared memory: do double-buffered; q, k, v single-buffered; one 32 KB staging buffer through which the dk tile and then
// the dv tile of a block leave by TMA store (row-per-thread stores straight from registers to global memory were measured
// 1500 cycles per block slower: 32 distinct lines per warp instruction).
//
// Every single-buffered tile is released as early as its readers allow, and the chain from one load of it to the next holds
// nothing else (a tile load takes 2,200-3,000 cycles under full load):
//   q: load -> S1, P0 q (commit QP_DONE) -> rows scaled in place (state group) -> D (commit D_DONE) -> next load
//   k: load -> S1 -> mask pass 1 -> scaled copy Ks, by the same warps (PK1_READY) -> next load
//   v: load -> S0 (issued one block ahead) -> mask pass 0 -> scaled copy Vs (PV0_READY) -> next load
// Roles (480 threads): warp 0 issues the loads, in the order in which their buffers come free; warp 1 issues the MMAs (one
// elected thread), per block: P0 q | Vs dKV^T | S0 of the next block | D | P1 do + Ks dKV | S1 of the next block; warps 2-5
// are the mask group (one per TMEM lane quadrant), which also writes the scaled copies right behind its own mask passes;
// warps 6-13 are the state/output group (q scaling, the two output tiles, the state recurrence and its bf16 copy); warp 14
// stores the staged output tiles, so that waiting for a store to have read the staging buffer never delays a load.
// Every wait is bounded and polls a CTA-wide abort flag.
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

constexpr int LD2_THREADS = 480;  // 15 warps: 65536 / 480 still allows 128 registers per thread

// barrier slots; every slot has two instances indexed by block parity
enum : int {
  LD2_FULL_Q = 0, LD2_FULL_G, LD2_FULL_V, LD2_FULL_K,
  LD2_S0_READY, LD2_S1_READY,
  LD2_PV0_READY,  // P0 and the scaled copy Vs are in SA (mask group); v may be reloaded
  LD2_PK1_READY,  // P1 and the scaled copy Ks are in SB (mask group); k may be reloaded
  LD2_QP_DONE,    // S1 and P0 q have read the unscaled q tile
  LD2_PC0_DONE, LD2_PC1_DONE, LD2_O_FREE0, LD2_O_FREE1, LD2_O_STAGED0, LD2_O_STAGED1, LD2_BUF_FREE0, LD2_BUF_FREE1,
  LD2_Q_SCALED, LD2_D_DONE, LD2_D_FREE, LD2_STATE_READY, LD2_NUM_BARS
};

template <int ND, int NE, int FMT>
__global__ void __launch_bounds__(LD2_THREADS, 1)
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
      if (i == LD2_PV0_READY || i == LD2_PK1_READY) count = LAP_MASK_THREADS;
      if (i == LD2_O_FREE0 || i == LD2_O_FREE1 || i == LD2_Q_SCALED || i == LD2_D_FREE || i == LD2_STATE_READY ||
          i == LD2_O_STAGED0 || i == LD2_O_STAGED1)
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

#ifdef LD2_WAITACC
  // Debugging build (-DLD2_WAITACC), used with lab200_la_debug_trace: lane 0 of every warp of CTA (0, 0, 0) sums the cycles it
  // spends inside bounded waits, per barrier, and the clock at a few events per block, and writes the sums behind the per-block
  // stamps: trace[blocks * LA_TRACE_SLOTS + 16 + warp * LD2_NUM_BARS + barrier] and, after those 15 rows, [warp * 8 + event].
  // The trace buffer must have room for them. Dividing by the block count gives the average wait per block and, relative to
  // the MMA warp's event 0, the average time of each event inside a block.
  long long wait_acc = 0;
  long long wait_site[LD2_NUM_BARS];
  long long ev_sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define LD2_EV(site) ev_sum[site] += clock64();
  for (int i = 0; i < LD2_NUM_BARS; ++i) wait_site[i] = 0;
  auto lap_wait_timed = [&](uint32_t b, uint32_t pa, volatile int* af, long long bud) -> bool {
    const long long t0 = clock64();
    const bool ok = lab200::lap_wait(b, pa, af, bud);
    wait_acc += clock64() - t0;
    wait_site[(b - sBar) >> 4] += clock64() - t0;
    return ok;
  };
#define lap_wait lap_wait_timed
#endif
#ifndef LD2_EV
#define LD2_EV(site)
#endif
#define LD2_FAIL(code) { if (*fail_code == 0) *fail_code = (code); }
#define LD2_STAMP(slot, it) if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && (it) < p.trace_blocks) \
    p.trace[(it) * LA_TRACE_SLOTS + (slot)] = clock64();
#define LD2_TRACE(slot, it) LD2_STAMP(slot, it)
#define LD2_WAIT(which, it, code) if (!lap_wait(bar(which, it), par(it), abort_flag, budget)) { LD2_FAIL(code) break; }

  if (warp == 0) {
    // =========================================== TMA loads ==============================================
    // Prologue: everything block 0 needs, do of block 1, and (once Vs of block 0 exists) v of block 1. Then, per block it,
    // the reloads in the order in which their buffers come free: q (D has read it), k (Ks exists), do two blocks ahead
    // (P1 do has read the stage), v two blocks ahead (Vs of the next block exists).
    if (issuer_lane(lane)) {
      auto load_q = [&](int i) {
        mbar_arrive_expect_tx(bar(LD2_FULL_Q, i), 2 * SLAB);
        for (int sl = 0; sl < 2; ++sl)  // q always as two slabs: it is the M = 128 side of the state MMA
          tma_load_3d(sQ + sl * SLAB, &tmQ, sl * 64, blk_of(i) * LA_BLOCK, zc, bar(LD2_FULL_Q, i));
      };
      auto load_k = [&](int i) {
        mbar_arrive_expect_tx(bar(LD2_FULL_K, i), ND * SLAB);
        for (int sl = 0; sl < ND; ++sl) tma_load_3d(sK + sl * SLAB, &tmK, sl * 64, blk_of(i) * LA_BLOCK, zc, bar(LD2_FULL_K, i));
      };
      auto load_v = [&](int i) {
        mbar_arrive_expect_tx(bar(LD2_FULL_V, i), NE * SLAB);
        for (int sl = 0; sl < NE; ++sl) tma_load_3d(sV + sl * SLAB, &tmV, sl * 64, blk_of(i) * LA_BLOCK, zc, bar(LD2_FULL_V, i));
      };
      auto load_g = [&](int i) {
        mbar_arrive_expect_tx(bar(LD2_FULL_G, i), NE * SLAB);
        for (int sl = 0; sl < NE; ++sl)
          tma_load_3d(sG + ((i & 1) * 2 + sl) * SLAB, &tmG, sl * 64, blk_of(i) * LA_BLOCK, zc, bar(LD2_FULL_G, i));
      };
      if (nb > 0) {
        load_v(0); load_g(0); load_k(0); load_q(0);
        if (nb > 1) load_g(1);
      }
      do {
        if (nb > 1) {
          LD2_WAIT(LD2_PV0_READY, 0, LA_ERR_WAIT_MMA1)
          load_v(1);
        }
        for (int it = 0; it < nb; ++it) {
          if (it + 1 < nb) {
            // q and k of the next block go to L2 now, a block before their loads: those loads sit in the chains that bound
            // the block (D -> q -> S1, Ks -> k -> S1) and complete in ~1,300 cycles from L2 instead of ~2,800 from HBM.
            // (Prefetching v and do as well was measured slower.)
            for (int sl = 0; sl < 2; ++sl) tma_prefetch_l2_3d(&tmQ, sl * 64, blk_of(it + 1) * LA_BLOCK, zc);
            for (int sl = 0; sl < ND; ++sl) tma_prefetch_l2_3d(&tmK, sl * 64, blk_of(it + 1) * LA_BLOCK, zc);
          }
          if (it + 1 < nb) {
            LD2_WAIT(LD2_D_DONE, it, LA_ERR_WAIT_MMA2)
            load_q(it + 1);
            LD2_EV(0)
            LD2_WAIT(LD2_PK1_READY, it, LA_ERR_WAIT_MMA1)
            load_k(it + 1);
            LD2_EV(1)
          }
          if (it + 2 < nb) {
            LD2_WAIT(LD2_PC1_DONE, it, LA_ERR_WAIT_MMA2)
            load_g(it + 2);
            LD2_EV(2)
            LD2_WAIT(LD2_PV0_READY, it + 1, LA_ERR_WAIT_MMA1)
            load_v(it + 2);
            LD2_EV(3)
          }
        }
      } while (false);
    }
  } else if (warp == 14) {
    // =========================================== TMA stores =============================================
    // The two staged output tiles of a block leave in turn through the one staging buffer.
    if (issuer_lane(lane)) {
      for (int it = 0; it < nb; ++it) {
        bool ok = true;
#pragma unroll 1
        for (int u = 0; u < 2 && ok; ++u) {
          ok = lap_wait(bar(u ? LD2_O_STAGED1 : LD2_O_STAGED0, it), par(it), abort_flag, budget);
          if (!ok) break;
          const int nslab = u ? NE : ND;
          for (int sl = 0; sl < nslab; ++sl)
            tma_store_3d(u ? static_cast<const void*>(&tmDV) : static_cast<const void*>(&tmDK), sO + sl * SLAB, sl * 64,
                         blk_of(it) * LA_BLOCK, zc);
          tma_store_commit();
          tma_store_wait_read();
          mbar_arrive(bar(u ? LD2_BUF_FREE1 : LD2_BUF_FREE0, it));
          LD2_EV(u)
        }
        if (!ok) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
      }
      tma_store_wait_all();
    }
  } else if (warp == 1) {
    // ============================================ MMA issuer ============================================
    if (issuer_lane(lane)) {
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
        for (int kq = 0; kq < nd16; ++kq) {
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_SB, smem_desc_sw128(sK + off, 16), smem_desc_sw128(sQ + off, 16), IDESC_S, kq > 0);
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
        const uint32_t sGs = sG + (it & 1) * 2 * SLAB;
        const bool have_state = have_state_in || (it > 0);
        LD2_TRACE(0, it)
        LD2_EV(0)
        // ---- dk = P0 q + Vs dKV^T; the first half is the last reader of the unscaled q tile ----------------------------
        LD2_WAIT(LD2_PV0_READY, it, LA_ERR_WAIT_MMA1)
        if (it > 0) { LD2_WAIT(LD2_O_FREE1, it - 1, LA_ERR_WAIT_MMA2) }  // the dv epilogue of the previous block has read O
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_O, tmem + T_SA + kk * 8, smem_desc_sw128(sQ + kk * 2048, SLAB), IDESC_PC0, kk > 0);
        umma_commit(bar(LD2_QP_DONE, it));
        LD2_TRACE(1, it)
        LD2_EV(1)
        if (have_state) {
          LD2_WAIT(LD2_STATE_READY, it, LA_ERR_WAIT_MMA2)
          tc_fence_after_sync();
          for (int kq = 0; kq < ne16; ++kq) {  // contraction over e: state copy columns
            const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
            umma_f16_ts(tmem + T_O, tmem + T_SA + T_XA + kq * 8, smem_desc_sw128(sS + off, 16), IDESC_X0, 1);
          }
        }
        umma_commit(bar(LD2_PC0_DONE, it));
        LD2_TRACE(2, it)
        LD2_EV(2)
        if (it + 1 < nb) {
          if (!issue_S0(it + 1)) { LD2_FAIL(LA_ERR_WAIT_INPUT) break; }
        }
        LD2_TRACE(3, it)
        LD2_EV(3)
        // ---- D = (w_state q)^T do: the last reader of q ------------------------------------------------------------------
        LD2_WAIT(LD2_Q_SCALED, it, LA_ERR_WAIT_MMA2)
        if (it > 0) { LD2_WAIT(LD2_D_FREE, it - 1, LA_ERR_WAIT_MMA2) }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem + T_D, smem_desc_sw128(sQ + kk * 2048, SLAB), smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_D, kk > 0);
        umma_commit(bar(LD2_D_DONE, it));
        LD2_TRACE(7, it)
        LD2_EV(4)
        // ---- dv = P1 do + Ks dKV -----------------------------------------------------------------------------------
        LD2_WAIT(LD2_PK1_READY, it, LA_ERR_WAIT_MMA1)
        LD2_WAIT(LD2_O_FREE0, it, LA_ERR_WAIT_MMA2)  // the dk epilogue has read O
        LD2_TRACE(4, it)
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16_ts(tmem + T_O, tmem + T_SB + kk * 8, smem_desc_sw128(sGs + kk * 2048, SLAB), IDESC_PC1, kk > 0);
        if (have_state) {
          for (int kq = 0; kq < nd16; ++kq)  // contraction over d: state copy rows
            umma_f16_ts(tmem + T_O, tmem + T_SB + T_XA + kq * 8, smem_desc_sw128(sS + kq * 2048, SLAB), IDESC_X1, 1);
        }
        umma_commit(bar(LD2_PC1_DONE, it));
        LD2_TRACE(5, it)
        LD2_EV(5)
        if (it + 1 < nb) {
          if (!issue_S1(it + 1)) { LD2_FAIL(LA_ERR_WAIT_INPUT) break; }
        }
        LD2_TRACE(6, it)
        LD2_EV(6)
      }
    }
  } else if (warp < 6) {
    // ============================================ mask group ============================================
    // Reverse-time mask on both products: keep c >= r with lambda^(c-r). One warp per TMEM lane quadrant, four 32-column
    // tiles each, in column order; P tile t goes back over S columns [16 t, 16 t + 16), which the warp has read by then.
    // Behind each pass the same warp writes the scaled copy of its 32 rows of v (k) into columns [64, 128) of the region,
    // whose S values it has consumed: pass 1 and Ks of block it, then pass 0 and Vs of block it + 1.
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
    const float w_out = ex2f(s2 * static_cast<float>(LA_BLOCK - r));  // reverse time
    const uint32_t w_out2 = pack2<FMT>(w_out, w_out);

    // one mask pass over region T_S (S product of block i) followed by the scaled copy of `tile`; arrives on `ready`
    auto pass = [&](int u, int i) -> bool {
      const uint32_t T_S = u ? T_SB : T_SA;
      bool ok = lap_wait(bar(u ? LD2_S1_READY : LD2_S0_READY, i), par(i), abort_flag, budget);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return false;
      if (q == 0 && lane == 0) { LD2_TRACE(8 + 2 * u, i) }
      LD2_EV(2 * u)
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
          for (int i2 = 0; i2 < 32; i2 += 2)
            pk[i2 >> 1] = pack2<FMT>(__uint_as_float(v[i2]) * (rowf * g[i2]), __uint_as_float(v[i2 + 1]) * (rowf * g[i2 + 1]));
        } else if (kind == 2 && diag_rank1) {
          // Masked elements (column i < lane) are zeroed by AND-ing the value's bits with a sign mask, not by a select on
          // the product: the compiler turned 32 selects into 32 branches per tile, and the diagonal tile, ~150 instructions
          // otherwise, then took ~2,800 cycles (clock stamps), which made the mask passes the bound of the whole kernel.
          float rd = rowd;
          asm volatile("" : "+f"(rd));  // keeps the 32 products rd * g[i] from being hoisted out of the block loop into registers
#pragma unroll
          for (int i2 = 0; i2 < 32; i2 += 2) {
            const uint32_t k0 = ~static_cast<uint32_t>((i2 - lane) >> 31), k1 = ~static_cast<uint32_t>((i2 + 1 - lane) >> 31);
            pk[i2 >> 1] = pack2<FMT>(__uint_as_float(v[i2] & k0) * (rd * g[i2]), __uint_as_float(v[i2 + 1] & k1) * (rd * g[i2 + 1]));
          }
        } else if (kind == 2) {
#pragma unroll
          for (int i2 = 0; i2 < 32; i2 += 2) {
            const int d0 = i2 - lane, d1 = d0 + 1;
            const uint32_t k0 = ~static_cast<uint32_t>(d0 >> 31), k1 = ~static_cast<uint32_t>(d1 >> 31);
            const float m0 = decay_tab[max(d0, 0)], m1 = decay_tab[max(d1, 0)];
            pk[i2 >> 1] = pack2<FMT>(__uint_as_float(v[i2] & k0) * m0, __uint_as_float(v[i2 + 1] & k1) * m1);
          }
        } else {
#pragma unroll
          for (int i2 = 0; i2 < 16; ++i2) pk[i2] = 0u;
        }
        tmem_st16(tmem + lanebase + T_S + t * 16, pk);
      }
      // scaled copy: row r of the [128][64 NS] tile times w(r) -> bf16 pairs -> columns [T_S + 64, ...), 4 columns per 16-byte chunk
      const uint32_t tile = u ? sK : sV;
      const int nch = (u ? ND : NE) * 8;  // 16-byte chunks in the row
#pragma unroll 1
      for (int c8 = 0; c8 < nch; c8 += 8) {  // one 64-feature slab of the row per step: eight loads in flight
        uint32_t w[2][16];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          ld_shared_v4(tile + (c8 >> 3) * SLAB + r * 128 + (((c ^ (r & 7))) << 4), w[c >> 2][(c & 3) * 4], w[c >> 2][(c & 3) * 4 + 1],
                       w[c >> 2][(c & 3) * 4 + 2], w[c >> 2][(c & 3) * 4 + 3]);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int j = 0; j < 16; ++j) w[hh][j] = mul2<FMT>(w[hh][j], w_out2);
          tmem_st16(tmem + lanebase + T_S + T_XA + (c8 + hh * 4) * 4, w[hh]);
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(u ? LD2_PK1_READY : LD2_PV0_READY, i));
      if (q == 0 && lane == 0) { LD2_TRACE(9 + 2 * u, i) }
      LD2_EV(2 * u + 1)
      return true;
    };
    bool alive = (nb == 0) || pass(0, 0);
    if (!alive) LD2_FAIL(LA_ERR_WAIT_MMA1)
    for (int it = 0; it < nb && alive; ++it) {
      alive = pass(1, it);
      if (alive && it + 1 < nb) alive = pass(0, it + 1);
      if (!alive) LD2_FAIL(LA_ERR_WAIT_MMA1)
    }
  } else {
    // ========================================= state / output group =====================================
    const int w8 = warp - 6;
    const int q = warp & 3, hf = w8 >> 2;
    const int r = q * 32 + lane;
    const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
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

    // epilogue of half U: O -> registers -> swizzled tile in the staging buffer (dk for U = 0, dv for U = 1); the store
    // warp sends it off. The buffer is free once the previous tile (the other half) has been read by its TMA store.
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
      // ---- q rows *= w_state(r), in place, for D: S1 and P0 q are done with the unscaled tile; first in the block because
      //      the next load of q waits for D -----------------------------------------------------------------------------
      {
        bool ok = lap_wait(bar(LD2_QP_DONE, it), par(it), abort_flag, budget);
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
        if (tracer) { LD2_TRACE(12, it) }
        LD2_EV(0)
      }
      // ---- dk tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 0>{}, it)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
      if (tracer) { LD2_TRACE(13, it) }
      LD2_EV(1)
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
      if (tracer) { LD2_TRACE(14, it) }
      LD2_EV(2)
      // ---- dv tile ---------------------------------------------------------------------------------------------
      if (!epilogue(std::integral_constant<int, 1>{}, it)) { LD2_FAIL(LA_ERR_WAIT_MMA2) break; }
      LD2_EV(3)
      if (has_next) {  // PC1_DONE (awaited by the dv epilogue) covers both halves of this block: they are done with the old copy
        store_state_smem();
        fence_proxy_async_smem();
        mbar_arrive(bar(LD2_STATE_READY, it + 1));
      }
      if (tracer) { LD2_TRACE(15, it) }
      LD2_EV(4)
    }
    if (*abort_flag == 0 && p.state_out != nullptr && st_row_valid) {
      float* dst = p.state_out + ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.d + r) * p.e + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.e) *reinterpret_cast<float4*>(dst + i) = make_float4(stt[i], stt[i + 1], stt[i + 2], stt[i + 3]);
      }
    }
  }
#ifdef LD2_WAITACC
#undef lap_wait
  if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && lane == 0)
    p.trace[p.trace_blocks * LA_TRACE_SLOTS + warp] = wait_acc;
  if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && lane == 0)
    for (int i = 0; i < LD2_NUM_BARS; ++i) p.trace[p.trace_blocks * LA_TRACE_SLOTS + 16 + warp * LD2_NUM_BARS + i] = wait_site[i];
  if (p.trace != nullptr && bh == 0 && blockIdx.y == 0 && lane == 0)
    for (int i = 0; i < 8; ++i) p.trace[p.trace_blocks * LA_TRACE_SLOTS + 16 + 15 * LD2_NUM_BARS + warp * 8 + i] = ev_sum[i];
#undef LD2_EV
#endif
#undef LD2_WAIT
#undef LD2_TRACE
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
