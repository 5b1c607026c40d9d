// Warp-specialised, software-pipelined version of the Lightning Attention-2 block kernel (dk <= 128).
//
// Same mathematics, operands, shared-memory slab layout and state conventions as la_chunk_kernel in
// la_kernels.cuh; what changes is who does what and when. The serial kernel runs the phases of one
// 128-token block one after another behind CTA-wide barriers; here four roles work on different blocks
// at the same time and hand tiles to each other through mbarriers:
//
//   warp 0      TMA producer   loads A, Bm, C tiles of block i+1, i+2 into two shared-memory stages
//   warp 1      MMA issuer     X_i = A State_i, D_i = C^T (w Bm), PC_i = P_i C, S_{i+1} = A Bm^T, in this order (one thread)
//   warps 2-5   mask group     S_i (TMEM) -> decay mask -> P_i (bf16, back into TMEM over S)
//   warps 6-13  state/output   Bm_i rows *= w_state (for D_i); D_i -> StateT = lambda^128 StateT + D_i (fp32 registers)
//                              -> bf16 copy for X_{i+1}; O_i = PC_i + w_out X_i -> swizzled shared-memory tile -> TMA store
//
// P never touches shared memory: it is written to TMEM with tcgen05.st and consumed by tcgen05.mma as the
// A operand, which frees the 32 KB that double-buffering A needs. Every wait is bounded and checks a
// CTA-wide abort flag, so a protocol error ends with an error status instead of a hang.
#pragma once
#include "la_kernels.cuh"

namespace lab200 {

constexpr int LAP_THREADS = 448;
constexpr int LAP_MASK_THREADS = 128, LAP_STATE_THREADS = 256;


// barrier slots (each has two instances, indexed by block parity)
enum : int { LAP_FULL_AB = 0, LAP_FULL_C, LAP_S_READY, LAP_P_READY, LAP_PC_DONE, LAP_D_DONE, LAP_O_FREE, LAP_D_FREE,
             LAP_STATE_READY, LAP_O_STAGED, LAP_BM_SCALED, LAP_NUM_BARS };

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// TMA store of one [128 rows][64 columns] slab, shared -> global; rows/columns outside the tensor are dropped.
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Bounded, abortable wait. Returns false if the budget ran out here or another role gave up.
__device__ __forceinline__ bool lap_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > budget) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}

template <int NKS, int NVS, int MODE, int FMT>
__global__ void __launch_bounds__(LAP_THREADS, 1)
la_pipe_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmO, const LaParams p) {
  static_assert(NKS <= 2, "the pipelined kernel double-buffers all inputs; dk <= 128 only");
  constexpr int SLAB = LA_SLAB_BYTES;
  constexpr int DV = 64 * NVS;
  constexpr int DKP = 64 * NKS;
  constexpr int SC = DKP / 2;
  constexpr int OC = DV / 2;
  constexpr int NAS = NKS > NVS ? NKS : NVS;  // slabs per A stage: the stage also stages the block's output tile
  constexpr uint32_t T_S = 0, T_OI = 128, T_OX = 128 + DV, T_D = 128 + 2 * DV;
  static_assert(T_D + DKP <= 512, "TMEM budget");
  constexpr uint32_t IDESC_S = umma_idesc(FMT, 128, 128, 0, 0);
  constexpr uint32_t IDESC_X = umma_idesc(FMT, 128, DV, 0, 0);
  constexpr uint32_t IDESC_PC = umma_idesc(FMT, 128, DV, 0, 1);
  constexpr uint32_t IDESC_ST = umma_idesc(FMT, 128, DKP, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t sA = base;                                         // 2 stages x NAS slabs (MODE 0)
  const uint32_t sB = sA + (MODE == 0 ? 2 * NAS * SLAB : 0);        // 2 stages x NKS slabs
  const uint32_t sC = sB + 2 * NKS * SLAB;                          // 2 stages x 2 slabs
  const uint32_t sS = sC + 2 * 2 * SLAB;                            // bf16 state, NKS x [DV rows][128 B] (MODE 0)
  // Output tiles are staged in the C stage of their own block (free once P C is done) and leave by TMA store.
  const uint32_t sBar = sS + (MODE == 0 ? NKS * DV * 128 : 0);      // 2 x LAP_NUM_BARS mbarriers
  const uint32_t sMisc = sBar + 2 * LAP_NUM_BARS * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sMisc - raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (sMisc + 4 - raw));
  volatile int* fail_code = reinterpret_cast<volatile int*>(smem_raw + (sMisc + 8 - raw));
  volatile float* decay_tab = reinterpret_cast<volatile float*>(smem_raw + (sMisc + 16 - raw));
  auto bar = [&](int which, int inst) -> uint32_t { return sBar + (which * 2 + inst) * 8; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int slice = blockIdx.x;
  const int chunk = p.chunk0 + blockIdx.y;
  const int bh = blockIdx.z;
  const int dv_off = slice * DV;
  const int blk_begin = chunk * p.blocks_per_chunk;
  const int blk_end = min(p.nblocks, blk_begin + p.blocks_per_chunk);
  const int nb = blk_end - blk_begin;
  const int reverse = p.reverse;
  // third tensor-map coordinate of this (batch, head) pair
  const int zc = p.layout ? (bh / p.h) * p.n * p.h + (bh % p.h) : bh;
  const int nk16 = p.dk >> 4;
  const long long budget = p.wait_budget;
  const bool have_state_in = (p.state_in != nullptr);

  const float s = p.slopes ? p.slopes[bh % p.h] : 0.f;
  const float s2 = -s * 1.4426950408889634f;

  if (tid == 0) {
    for (int i = 0; i < LAP_NUM_BARS; ++i) {
      const uint32_t count = (i == LAP_P_READY) ? LAP_MASK_THREADS
                           : (i == LAP_O_FREE || i == LAP_D_FREE || i == LAP_STATE_READY || i == LAP_O_STAGED || i == LAP_BM_SCALED) ? LAP_STATE_THREADS : 1u;
      mbar_init(bar(i, 0), count);
      mbar_init(bar(i, 1), count);
    }
    *abort_flag = 0;
    *fail_code = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
    if (MODE == 0) tma_prefetch_desc(&tmO);
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

#define LAP_FAIL(code) { if (*fail_code == 0) *fail_code = (code); }
#define LAP_TRACE(slot, it) if (p.trace != nullptr && bh == 0 && blockIdx.x == 0 && blockIdx.y == 0 && (it) < p.trace_blocks) \
    p.trace[(it) * LA_TRACE_SLOTS + (slot)] = clock64();

  if (warp == 0) {
    // =========================================== TMA producer ===========================================
    // Also issues the TMA stores of the output tiles: a tile is staged in the C stage of its block (P C, the last MMA of a
    // block, has read C by then), and that stage is reloaded (for block it+2) only after the store has read it.
    if (issuer_lane(lane)) {
      auto blk_of = [&](int i) { return reverse ? (blk_end - 1 - i) : (blk_begin + i); };
      auto store_tile = [&](int i) -> bool {  // output tile of block i: wait until it is staged, then store it
        const int sst = i & 1;
        if (!lap_wait(bar(LAP_O_STAGED, sst), (i >> 1) & 1, abort_flag, budget)) return false;
#pragma unroll
        for (int vs = 0; vs < NVS; ++vs)
          tma_store_3d(&tmO, sC + (sst * 2 + vs) * SLAB, dv_off + vs * 64, blk_of(i) * LA_BLOCK, zc);
        tma_store_commit();
        return true;
      };
      bool alive = true;
      for (int it = 0; it < nb && alive; ++it) {
        const int blk = blk_of(it);
        const int st = it & 1;
        const uint32_t prev_par = ((it >> 1) & 1) ^ 1;  // parity of the previous use of this stage (block it-2)
        // A and Bm of block it: their stages are free once every MMA of block it-2 has run (P C is the last one issued; in
        // state-only mode D). They are what S of block it waits for, so they go first and wait for nothing else.
        if (it >= 2) {
          if (!lap_wait(bar(MODE == 0 ? LAP_PC_DONE : LAP_D_DONE, st), prev_par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
        }
        mbar_arrive_expect_tx(bar(LAP_FULL_AB, st), (MODE == 0 ? 2 * NKS : NKS) * SLAB);
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks)
          tma_load_3d(sB + (st * NKS + ks) * SLAB, &tmB, ks * 64, blk * LA_BLOCK, zc, bar(LAP_FULL_AB, st));
        if (MODE == 0) {
#pragma unroll
          for (int ks = 0; ks < NKS; ++ks)
            tma_load_3d(sA + (st * NAS + ks) * SLAB, &tmA, ks * 64, blk * LA_BLOCK, zc, bar(LAP_FULL_AB, st));
        }
        // C of block it: in the full block loop its stage holds the staged output tile of block it-2, which is stored first;
        // C is not needed before D of block it, a whole block later than A and Bm.
        if (MODE == 0 && it >= 2) {
          if (!store_tile(it - 2)) { LAP_FAIL(LA_ERR_WAIT_MMA2) alive = false; break; }
          tma_store_wait_read();
        }
        // Only the slabs of this CTA's dv slice are loaded. D = C^T (w Bm) is an M = 128 MMA and reads both slabs of the stage; with
        // a 64-wide slice the second one holds stale bytes, which only reach accumulator rows >= 64 that nobody reads.
        mbar_arrive_expect_tx(bar(LAP_FULL_C, st), NVS * SLAB);
#pragma unroll
        for (int vs = 0; vs < NVS; ++vs)
          tma_load_3d(sC + (st * 2 + vs) * SLAB, &tmC, dv_off + vs * 64, blk * LA_BLOCK, zc, bar(LAP_FULL_C, st));
      }
      if (MODE == 0 && alive && *abort_flag == 0) {
        for (int i = max(nb - 2, 0); i < nb; ++i) {
          if (!store_tile(i)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
        }
      }
      if (MODE == 0) tma_store_wait_all();
    }
  } else if (warp == 1) {
    // ============================================ MMA issuer ============================================
    // Issue order per block: X_i, D_i, PC_i, S_{i+1}. X_i and D_i need nothing from the mask group, so they run while
    // it turns S_i into P_i; D_i this early also means the next state is ready long before X_{i+1} asks for it.
    // S_{i+1} overwrites the TMEM columns P_i lives in, so it follows PC_i (the tensor pipe executes in issue order).
    // D and P C commit to their own barriers: the state update starts after D_i, the output tile leaves TMEM after
    // PC_i while S_{i+1}, X_{i+1} and D_{i+1} run.
    if (issuer_lane(lane)) {
      auto issue_S = [&](int i) -> bool {
        const int ist = i & 1;
        if (!lap_wait(bar(LAP_FULL_AB, ist), (i >> 1) & 1, abort_flag, budget)) return false;
        tc_fence_after_sync();
        const uint32_t a0 = sA + ist * NAS * SLAB, b0 = sB + ist * NKS * SLAB;
        for (int kq = 0; kq < nk16; ++kq) {  // S = A Bm^T
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_S, smem_desc_sw128(a0 + off, 16), smem_desc_sw128(b0 + off, 16), IDESC_S, kq > 0);
        }
        umma_commit(bar(LAP_S_READY, ist));
        return true;
      };
      bool alive = true;
      if (MODE == 0 && nb > 0) {
        alive = issue_S(0);
        if (!alive) LAP_FAIL(LA_ERR_WAIT_INPUT)
      }
      for (int it = 0; it < nb && alive; ++it) {
        const int st = it & 1;
        const uint32_t par = (it >> 1) & 1;
        const int pst = st ^ 1;                         // instance used by block it-1
        const uint32_t ppar = ((it - 1) >> 1) & 1;      // and its parity
        const uint32_t sAs = sA + st * NAS * SLAB, sBs = sB + st * NKS * SLAB, sCs = sC + st * 2 * SLAB;
        const bool have_state = have_state_in || (it > 0);
        LAP_TRACE(0, it)
        if (MODE == 0) {
          if (have_state) {
            if (!lap_wait(bar(LAP_STATE_READY, st), par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
            if (it > 0 && !lap_wait(bar(LAP_O_FREE, pst), ppar, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
            tc_fence_after_sync();
            for (int kq = 0; kq < nk16; ++kq) {  // X = A State
              const uint32_t offA = (kq >> 2) * SLAB + (kq & 3) * 32;
              const uint32_t offS = (kq >> 2) * (DV * 128) + (kq & 3) * 32;
              umma_f16(tmem + T_OX, smem_desc_sw128(sAs + offA, 16), smem_desc_sw128(sS + offS, 16), IDESC_X, kq > 0);
            }
          }
          LAP_TRACE(1, it)
        }
        if (MODE != 0 && !lap_wait(bar(LAP_FULL_AB, st), par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_INPUT) break; }
        if (!lap_wait(bar(LAP_FULL_C, st), par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_INPUT) break; }
        if (!lap_wait(bar(LAP_BM_SCALED, st), par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
        if (it > 0 && !lap_wait(bar(LAP_D_FREE, pst), ppar, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // local StateT = C^T (w_state Bm)
          umma_f16(tmem + T_D, smem_desc_sw128(sCs + kk * 2048, SLAB), smem_desc_sw128(sBs + kk * 2048, SLAB), IDESC_ST, kk > 0);
        umma_commit(bar(LAP_D_DONE, st));  // also: X_it is done with the bf16 state copy
        LAP_TRACE(3, it)
        if (MODE == 0) {
          if (!lap_wait(bar(LAP_P_READY, st), par, abort_flag, budget)) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
          LAP_TRACE(2, it)
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)  // O_intra = P C, P read from TMEM
            umma_f16_ts(tmem + T_OI, tmem + T_S + kk * 8, smem_desc_sw128(sCs + kk * 2048, SLAB), IDESC_PC, kk > 0);
          umma_commit(bar(LAP_PC_DONE, st));  // O_intra and O_inter are complete; nothing reads A, Bm, C of this block any more
          if (it + 1 < nb) {
            if (!issue_S(it + 1)) { LAP_FAIL(LA_ERR_WAIT_INPUT) break; }
          }
        }
      }
    }
  } else if (warp < 6) {
    // ============================================ mask group ============================================
    // One warp per TMEM lane quadrant, four 32-column tiles each, in column order. P tile t goes back into TMEM at
    // columns [16 t, 16 t + 16), i.e. over S columns of S tile t/2 <= t, which the warp has already pulled into
    // registers by then.
    if (MODE == 0) {
      const int q = warp & 3;
      const int r = q * 32 + lane;
      const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
      const bool tracer = lane == 0 && q == (reverse ? 0 : 3);  // the quadrant with the most unmasked tiles
      float g[32];  // per-column part of the decay inside a live tile: lambda^i (reverse) or lambda^(31-i) (forward)
#pragma unroll
      for (int i = 0; i < 32; ++i) g[i] = ex2f(s2 * static_cast<float>(reverse ? i : 31 - i));
      // Diagonal tile: lambda^(lane-i) = g[i] * lambda^(lane-31) (forward), lambda^(i-lane) = g[i] * lambda^(-lane) (reverse).
      // The row factor is >= 1 here, at most lambda^-31; for decay rates where that could leave the fp32 range the
      // per-element table is used instead (CTA-uniform choice).
      const bool diag_rank1 = s * 31.f < 60.f;
      const float rowd = diag_rank1 ? ex2f(s2 * static_cast<float>(reverse ? -lane : lane - 31)) : 0.f;
      for (int it = 0; it < nb; ++it) {
        const int st = it & 1;
        const uint32_t par = (it >> 1) & 1;
        bool ok = lap_wait(bar(LAP_S_READY, st), par, abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LAP_FAIL(LA_ERR_WAIT_MMA1) break; }
        if (tracer) { LAP_TRACE(4, it) }
        tc_fence_after_sync();
        // kind of tile t for this quadrant: 0 dead (all masked), 1 live (nothing masked), 2 diagonal; warp-uniform
        auto tile_kind = [&](int t) { return (t == q) ? 2 : ((reverse ? (t > q) : (t < q)) ? 1 : 0); };
#pragma unroll 1
        for (int t = 0; t < 4; ++t) {
          const int c0 = t * 32;
          const int kind = tile_kind(t);
          uint32_t v[1][32];
          if (kind) {
            tmem_ld32(tmem + lanebase + T_S + c0, v[0]);
            tmem_wait_ld();
          }
          uint32_t pk[16];
          if (kind == 1) {
            // lambda^|r-c| = (per-row part, one table look-up) x (per-column part g[i]); both factors are <= 1
            const float rowf = decay_tab[reverse ? (c0 - r) : (r - c0 - 31)];
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              pk[i >> 1] = pack2<FMT>(__uint_as_float(v[0][i]) * (rowf * g[i]), __uint_as_float(v[0][i + 1]) * (rowf * g[i + 1]));
          } else if (kind == 2 && diag_rank1) {
            float rd = rowd;
            asm volatile("" : "+f"(rd));  // keeps the 32 products rd * g[i] from being hoisted out of the block loop into registers
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int d0 = reverse ? (i - lane) : (lane - i);
              const int d1 = reverse ? (d0 + 1) : (d0 - 1);
              const float f0 = (d0 >= 0) ? __uint_as_float(v[0][i]) * (rd * g[i]) : 0.f;
              const float f1 = (d1 >= 0) ? __uint_as_float(v[0][i + 1]) * (rd * g[i + 1]) : 0.f;
              pk[i >> 1] = pack2<FMT>(f0, f1);
            }
          } else if (kind == 2) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int d0 = reverse ? (i - lane) : (lane - i);
              const int d1 = reverse ? (d0 + 1) : (d0 - 1);
              const float m0 = decay_tab[max(d0, 0)], m1 = decay_tab[max(d1, 0)];
              const float f0 = (d0 >= 0) ? __uint_as_float(v[0][i]) * m0 : 0.f;
              const float f1 = (d1 >= 0) ? __uint_as_float(v[0][i + 1]) * m1 : 0.f;
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
        mbar_arrive(bar(LAP_P_READY, st));
        if (tracer) { LAP_TRACE(5, it) }
      }
    }
  } else {
    // ========================================= state / output group =====================================
    const int w8 = warp - 6;
    const int q = warp & 3, hf = w8 >> 2;
    const int r = q * 32 + lane;
    const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;
    const float w_out = reverse ? ex2f(s2 * static_cast<float>(LA_BLOCK - r)) : ex2f(s2 * static_cast<float>(r));
    const float decay_blk = ex2f(s2 * static_cast<float>(LA_BLOCK));
    const float w_state = reverse ? ex2f(s2 * static_cast<float>(r)) : ex2f(s2 * static_cast<float>(LA_BLOCK - r));
    const uint32_t w_state2 = pack2<FMT>(w_state, w_state);
    // A forward-time sweep that ends in a ragged block (n not a multiple of 128): the state leaving that block is decayed
    // to token n, not to the end of the 128-token tile, so that state_out chains exactly (rows >= tail are zero padding).
    const int tail = p.n - (p.nblocks - 1) * LA_BLOCK;
    const bool tail_fix = !reverse && tail < LA_BLOCK && blk_end == p.nblocks;
    const float w_tail = (tail_fix && r < tail) ? ex2f(s2 * static_cast<float>(tail - r)) : 0.f;
    const uint32_t w_tail2 = pack2<FMT>(w_tail, w_tail);
    const float decay_tail = ex2f(s2 * static_cast<float>(tail));
    const bool st_row_valid = (r < DV) && (dv_off + r < p.dv);
    const bool store_thread = (w8 == 0 && lane == 0);

    float stt[SC];
#pragma unroll
    for (int i = 0; i < SC; ++i) stt[i] = 0.f;
    if (have_state_in && st_row_valid) {
      const float* src = p.state_in +
          ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.dv + dv_off + r) * p.dk + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.dk) {
          const float4 v4 = *reinterpret_cast<const float4*>(src + i);
          stt[i] = v4.x; stt[i + 1] = v4.y; stt[i + 2] = v4.z; stt[i + 3] = v4.w;
        }
      }
    }
    auto store_state_smem = [&]() {
      if (r < DV) {
#pragma unroll
        for (int i = 0; i < SC; i += 8) {
          const int col = hf * SC + i;
          const uint32_t addr = sS + (col >> 6) * (DV * 128) + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4);
          st_shared_v4(addr, pack2<FMT>(stt[i], stt[i + 1]), pack2<FMT>(stt[i + 2], stt[i + 3]),
                       pack2<FMT>(stt[i + 4], stt[i + 5]), pack2<FMT>(stt[i + 6], stt[i + 7]));
        }
      }
    };
    if (MODE == 0) {
      if (have_state_in) {
        store_state_smem();
        fence_proxy_async_smem();
      }
      mbar_arrive(bar(LAP_STATE_READY, 0));  // state entering block 0
    }

    // Bm rows of block j *= w_state(r), in place, for D_j: this thread's half of the row's 16-byte chunks.
    auto scale_bm = [&](int j) -> bool {
      const int st = j & 1;
      // S_j must be done with the unscaled tile (state-only mode: the tile must have landed)
      bool ok = lap_wait(bar(MODE == 0 ? LAP_S_READY : LAP_FULL_AB, st), (j >> 1) & 1, abort_flag, budget);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return false;
      if (s != 0.f) {
        const uint32_t w2 = (tail_fix && j == nb - 1) ? w_tail2 : w_state2;
        constexpr int NCH = NKS * 4;  // chunks per thread
        const uint32_t sBs = sB + st * NKS * SLAB;
        uint32_t u[NCH][4];
        uint32_t addr[NCH];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int gch = hf * NCH + c;  // chunk index in the row, 0 .. NKS*8-1
          const int ks = gch >> 3, p0 = gch & 7;
          const int pos = (NCH >= 8) ? ((p0 + r) & 7) : ((p0 & 4) | ((p0 + r) & 3));  // spread the warp over the banks
          addr[c] = sBs + ks * SLAB + r * 128 + (pos << 4);
          ld_shared_v4(addr[c], u[c][0], u[c][1], u[c][2], u[c][3]);
        }
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
#pragma unroll
          for (int j2 = 0; j2 < 4; ++j2) u[c][j2] = mul2<FMT>(u[c][j2], w2);
          st_shared_v4(addr[c], u[c][0], u[c][1], u[c][2], u[c][3]);
        }
        fence_proxy_async_smem();
      }
      mbar_arrive(bar(LAP_BM_SCALED, st));
      if (store_thread) { LAP_TRACE(6, j) }
      return true;
    };
    // Order of work per block it: state update (after D_it), output tile (after PC_it), Bm scaling for block it+1
    // (after S_{it+1}) - the order in which the MMA warp completes them.
    bool live = true;
    if (nb > 0) {
      live = scale_bm(0);
      if (!live) LAP_FAIL(LA_ERR_WAIT_MMA1)
    }
    for (int it = 0; it < nb && live; ++it) {
      const int st = it & 1;
      const uint32_t par = (it >> 1) & 1;
      const bool has_next = (it + 1 < nb);
      const bool have_state = have_state_in || (it > 0);
      // state-only mode: the next block's Bm tile is scaled while D of this block runs
      if (MODE != 0 && has_next && !scale_bm(it + 1)) { LAP_FAIL(LA_ERR_WAIT_MMA1) break; }
      {
        bool ok = lap_wait(bar(LAP_D_DONE, st), par, abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
      }
      if (store_thread) { LAP_TRACE(8, it) }
      tc_fence_after_sync();
      // ---- state recurrence --------------------------------------------------------------------------
      if (q * 32 < DV) {
#pragma unroll
        for (int cc = 0; cc < SC; cc += 32) {
          uint32_t dl[32];
          tmem_ld32(tmem + lanebase + T_D + hf * SC + cc, dl);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            stt[cc + i] = fmaf((tail_fix && it == nb - 1) ? decay_tail : decay_blk, stt[cc + i], __uint_as_float(dl[i]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive(bar(LAP_D_FREE, st));
      if (MODE == 0 && has_next) {
        // X_it was issued before D_it, so it is done with the old bf16 copy of the state
        store_state_smem();
        fence_proxy_async_smem();
        mbar_arrive(bar(LAP_STATE_READY, st ^ 1));  // state entering block it+1
      }
      if (store_thread) { LAP_TRACE(9, it) }
      if (MODE == 0) {
        // ---- output tile: TMEM -> registers -> swizzled shared-memory slabs -> TMA store. Runs while S_{it+1},
        //      X_{it+1} and D_{it+1} are in the tensor pipe. --------------------------------------------------------------
        bool ok = lap_wait(bar(LAP_PC_DONE, st), par, abort_flag, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { LAP_FAIL(LA_ERR_WAIT_MMA2) break; }
        if (store_thread) { LAP_TRACE(7, it) }
        tc_fence_after_sync();
        const uint32_t sOs = sC + st * 2 * SLAB;  // P C and D of this block are done with this C stage
#pragma unroll
        for (int cc = 0; cc < OC; cc += 16) {
          uint32_t a[16], b[16];
          tmem_ld16(tmem + lanebase + T_OI + hf * OC + cc, a);
          if (have_state) tmem_ld16(tmem + lanebase + T_OX + hf * OC + cc, b);
          tmem_wait_ld();
          if (cc + 16 >= OC) {  // last read of this block's accumulators
            tc_fence_before_sync();
            mbar_arrive(bar(LAP_O_FREE, st));
            if (store_thread) { LAP_TRACE(10, it) }
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
            const int col = hf * OC + cc + g * 8;  // column inside this CTA's dv slice
            st_shared_v4(sOs + (col >> 6) * SLAB + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4), o4[0], o4[1], o4[2], o4[3]);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(bar(LAP_O_STAGED, st));  // the producer warp stores the tile
        if (store_thread) { LAP_TRACE(11, it) }
      }
      if (MODE == 0 && has_next && !scale_bm(it + 1)) { LAP_FAIL(LA_ERR_WAIT_MMA1) break; }
    }
    if (*abort_flag == 0 && p.state_out != nullptr && st_row_valid) {
      float* dst = p.state_out +
          ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.dv + dv_off + r) * p.dk + hf * SC;
#pragma unroll
      for (int i = 0; i < SC; i += 4) {
        if (hf * SC + i < p.dk) *reinterpret_cast<float4*>(dst + i) = make_float4(stt[i], stt[i + 1], stt[i + 2], stt[i + 3]);
      }
    }
  }
#undef LAP_TRACE
#undef LAP_FAIL

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, *fail_code ? *fail_code : LA_ERR_WAIT_MMA2);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace lab200
