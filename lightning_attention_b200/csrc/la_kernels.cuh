// Lightning Attention-2 device kernels for sm_100a.
//
// One generic kernel covers the forward pass and all three gradients. For row-major inputs
// A (n x dk, "query-like"), Bm (n x dk, "key-like"), C (n x dv, "value-like") of one (batch, head)
// pair and decay rate s (lambda = exp(-s)) it computes, in forward time order,
//
//     out_t = sum_{j <= t} lambda^(t-j) (A_t . Bm_j) C_j                    (reverse = 0)
//
// or, in reverse time order,
//
//     out_t = sum_{j >= t} lambda^(j-t) (A_t . Bm_j) C_j                    (reverse = 1)
//
// The reference computes the same quantities with three Triton kernels
// (lightning_attn/ops/triton/lightning_attn2.py:8-85 forward, :88-183 in-block gradients,
// :186-395 cross-block gradients). With (A,Bm,C) = (q,k,v) forward time gives o; (do,v,k) forward
// time gives dq; (v,do,q) reverse time gives dk; (k,q,do) reverse time gives dv.
//
// The sequence is cut into blocks of 128 tokens. Per block (r, c = row indices inside the block):
//     S      = A Bm^T                                   tcgen05.mma, fp32 in TMEM
//     P      = S (.) M,  M[r,c] = lambda^|r-c| on the causal side, 0 elsewhere   (CUDA cores -> smem)
//     O      = P C + diag(w_out) A State                two tcgen05.mma chains, combined in the epilogue
//     StateT = lambda^128 StateT + C^T (diag(w_state) Bm)   tcgen05.mma + fp32 registers
// with w_out(r) = lambda^r, w_state(r) = lambda^(128-r) in forward time and the two swapped in
// reverse time (lightning_attn2.py:47-48, :352-358, :392-395). StateT (dv x dk, the transposed
// d x e "KV" state of the reference) lives in fp32 registers for the whole block loop; a rounded
// copy in shared memory feeds the tensor cores.
//
// Shared-memory tiles are [128 tokens][64 features] slabs with the 128-byte swizzle, exactly as TMA
// writes them; the same slab serves as a K-major operand (contraction over features) and as an
// MN-major operand (contraction over tokens), so no transposes are ever materialised.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ptx_sm100.cuh"

namespace lab200 {

constexpr int LA_BLOCK = 128;        // tokens per block
constexpr int LA_SLAB_BYTES = 16384; // 128 rows x 128 bytes
constexpr int LA_THREADS = 256;
constexpr int LA_TRACE_SLOTS = 16;    // clock stamps per block in the optional trace buffer

enum LaError : int {
  LA_OK = 0,
  LA_ERR_WAIT_INPUT = 101,  // TMA bytes never arrived
  LA_ERR_WAIT_MMA1 = 102,   // first MMA group never completed
  LA_ERR_WAIT_MMA2 = 103,   // second MMA group never completed
};

struct LaParams {
  void* out;               // [bh][n][dv], input dtype (unused when only the state is wanted)
  const float* slopes;     // [h] decay rates, or nullptr for no decay
  const float* state_in;   // [bh][state_slots][dv][dk] fp32, or nullptr for a zero initial state
  float* state_out;        // same indexing, or nullptr
  int* status;             // device word that receives a LaError on failure
  int n, h, dk, dv;
  int nblocks;             // ceil(n / 128)
  int blocks_per_chunk;
  int chunk0;              // chunk handled by blockIdx.y == 0
  int state_slots;         // chunk slots per (batch, head) in state_in / state_out
  int reverse;
  int layout;              // 0: tensors are (b, h, n, dim) contiguous; 1: (b, n, h, dim) contiguous (pipelined kernel only):
                           // the tensor maps then index their third dimension by batch * n * h + head, see make_tmap
  int nstage;              // 1 or 2 shared-memory stages for the Bm and C tiles
  long long wait_budget;   // clock cycles after which a barrier wait gives up
  long long* trace;        // optional: CTA (0,0,0) records clock64() stamps here, LA_TRACE_SLOTS per block
  int trace_blocks;        // capacity of `trace` in blocks
};

template <int FMT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (FMT == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
// packed multiply of two 16-bit pairs (rounds once per element, in the 16-bit format)
template <int FMT>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
  if constexpr (FMT == 1) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  } else {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
}
template <int FMT>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (FMT == 1) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// MODE 0: full block loop (writes out, optionally the final state).
// MODE 1: state only (reads Bm and C, writes the final state).
// NKS: 64-feature slabs of dk (1..4). NVS: 64-feature slabs of dv handled by this CTA (1..2).
template <int NKS, int NVS, int MODE, int FMT>
__global__ void __launch_bounds__(LA_THREADS, 1)
la_chunk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const LaParams p) {
  constexpr int SLAB = LA_SLAB_BYTES;
  constexpr int DV = 64 * NVS;
  constexpr int DKP = 64 * NKS;
  constexpr int SC = DKP / 2;  // state columns held per thread
  constexpr int OC = DV / 2;   // output columns handled per thread
  constexpr uint32_t T_S = 0, T_OI = 128, T_OX = 128 + DV, T_D = 128 + 2 * DV;
  static_assert(T_D + DKP <= 512, "TMEM budget");
  constexpr uint32_t IDESC_S = umma_idesc(FMT, 128, 128, 0, 0);
  constexpr uint32_t IDESC_X = umma_idesc(FMT, 128, DV, 0, 0);
  constexpr uint32_t IDESC_PC = umma_idesc(FMT, 128, DV, 0, 1);
  constexpr uint32_t IDESC_ST = umma_idesc(FMT, 128, DKP, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int nstage = p.nstage;
  const uint32_t sA = base;
  const uint32_t sB = sA + (MODE == 0 ? NKS * SLAB : 0);
  const uint32_t sC = sB + nstage * NKS * SLAB;
  const uint32_t sP = sC + nstage * 2 * SLAB;
  const uint32_t sS = sP + (MODE == 0 ? 2 * SLAB : 0);
  const uint32_t sBar = sS + (MODE == 0 ? NKS * DV * 128 : 0);
  const uint32_t barA = sBar, barBC0 = sBar + 8, barM1 = sBar + 24, barM2 = sBar + 32;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sBar + 40 - raw));
  // decay table lambda^k, k = 0..127, for the in-block mask (a table look-up per element instead of an
  // exponential; also keeps the compiler from hoisting 64 exponentials per thread into registers)
  volatile float* decay_tab = reinterpret_cast<volatile float*>(smem_raw + (sBar + 64 - raw));

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int q = warp & 3, hf = warp >> 2;
  const int r = q * 32 + lane;  // row inside the block == TMEM lane owned by this thread
  const uint32_t lanebase = static_cast<uint32_t>(q * 32) << 16;

  const int slice = blockIdx.x;
  const int chunk = p.chunk0 + blockIdx.y;
  const int bh = blockIdx.z;
  const int dv_off = slice * DV;
  const int blk_begin = chunk * p.blocks_per_chunk;
  const int blk_end = min(p.nblocks, blk_begin + p.blocks_per_chunk);
  const int nb = blk_end - blk_begin;
  const int reverse = p.reverse;
  const int nk16 = p.dk >> 4;

  if (tid == 0) {
    mbar_init(barA, 1);
    mbar_init(barBC0, 1);
    mbar_init(barBC0 + 8, 1);
    mbar_init(barM1, 1);
    mbar_init(barM2, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 0) {
    tmem_alloc(sBar + 40, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // per-head decay constants (lightning_attn2.py:41-54)
  const float s = p.slopes ? p.slopes[bh % p.h] : 0.f;
  const float s2 = -s * 1.4426950408889634f;  // lambda^x = 2^(s2 x)
  const float w_fwd = ex2f(s2 * static_cast<float>(r));
  const float w_bwd = ex2f(s2 * static_cast<float>(LA_BLOCK - r));
  const float w_out = reverse ? w_bwd : w_fwd;
  const float w_state = reverse ? w_fwd : w_bwd;
  const float decay_blk = ex2f(s2 * static_cast<float>(LA_BLOCK));
  // A forward-time sweep that ends in a ragged block (n not a multiple of 128): the state leaving that block is decayed
  // to token n, not to the end of the 128-token tile, so that state_out chains exactly (rows >= tail are zero padding).
  const int tail = p.n - (p.nblocks - 1) * LA_BLOCK;
  const bool tail_fix = !reverse && tail < LA_BLOCK && blk_end == p.nblocks;
  const float w_tail = (tail_fix && r < tail) ? ex2f(s2 * static_cast<float>(tail - r)) : 0.f;
  const float decay_tail = ex2f(s2 * static_cast<float>(tail));
  if (MODE == 0 && tid < LA_BLOCK) decay_tab[tid] = ex2f(s2 * static_cast<float>(tid));

  auto issue_A = [&](int blk) {
    mbar_arrive_expect_tx(barA, NKS * SLAB);
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) tma_load_3d(sA + ks * SLAB, &tmA, ks * 64, blk * LA_BLOCK, bh, barA);
  };
  auto issue_BC = [&](int blk, int stage) {
    const uint32_t bar = barBC0 + 8 * stage;
    mbar_arrive_expect_tx(bar, (NKS + 2) * SLAB);
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks)
      tma_load_3d(sB + (stage * NKS + ks) * SLAB, &tmB, ks * 64, blk * LA_BLOCK, bh, bar);
#pragma unroll
    for (int vs = 0; vs < 2; ++vs)
      tma_load_3d(sC + (stage * 2 + vs) * SLAB, &tmC, dv_off + vs * 64, blk * LA_BLOCK, bh, bar);
  };

  // first block's loads go out before anything else
  if (tid == 0 && nb > 0) {
    const int blk0 = reverse ? (blk_end - 1) : blk_begin;
    if (MODE == 0) issue_A(blk0);
    issue_BC(blk0, 0);
  }

  // running state StateT[j = r][hf * SC .. hf * SC + SC), fp32
  float st[SC];
  const bool st_row_valid = (r < DV) && (dv_off + r < p.dv);
  const bool have_state_in = (p.state_in != nullptr);
#pragma unroll
  for (int i = 0; i < SC; ++i) st[i] = 0.f;
  if (have_state_in && st_row_valid) {
    const float* src = p.state_in +
        ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.dv + dv_off + r) * p.dk + hf * SC;
#pragma unroll
    for (int i = 0; i < SC; i += 4) {
      if (hf * SC + i < p.dk) {  // dk is a multiple of 16, so groups of 4 never straddle the edge
        const float4 v4 = *reinterpret_cast<const float4*>(src + i);
        st[i] = v4.x; st[i + 1] = v4.y; st[i + 2] = v4.z; st[i + 3] = v4.w;
      }
    }
  }
  // rounded copy of the state for the tensor cores: K-major B operand, rows = dv index, cols = dk index
  auto store_state_smem = [&]() {
    if (r < DV) {
#pragma unroll
      for (int i = 0; i < SC; i += 8) {
        const int col = hf * SC + i;
        const uint32_t addr = sS + (col >> 6) * (DV * 128) + r * 128 + ((((col & 63) >> 3) ^ (r & 7)) << 4);
        st_shared_v4(addr, pack2<FMT>(st[i], st[i + 1]), pack2<FMT>(st[i + 2], st[i + 3]),
                     pack2<FMT>(st[i + 4], st[i + 5]), pack2<FMT>(st[i + 6], st[i + 7]));
      }
    }
  };
  if (MODE == 0 && have_state_in) {
    store_state_smem();
    fence_proxy_async_smem();
  }
  __syncthreads();

  int failed = 0;
  const bool tracing = (p.trace != nullptr) && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#define LA_TRACE(slot) if (tracing && it < p.trace_blocks) p.trace[it * LA_TRACE_SLOTS + (slot)] = clock64();

  for (int it = 0; it < nb; ++it) {
    LA_TRACE(0)
    const int blk = reverse ? (blk_end - 1 - it) : (blk_begin + it);
    const int nxt = reverse ? (blk - 1) : (blk + 1);
    const bool has_next = (it + 1 < nb);
    const int stage = (nstage == 2) ? (it & 1) : 0;
    const uint32_t parBC = (nstage == 2) ? ((it >> 1) & 1) : (it & 1);
    const uint32_t par = it & 1;
    const uint32_t sBs = sB + stage * NKS * SLAB;
    const uint32_t sCs = sC + stage * 2 * SLAB;
    const bool have_state = have_state_in || (it > 0);

    // ---- 1. inputs landed ---------------------------------------------------------------
    {
      bool ok = mbar_wait(barBC0 + 8 * stage, parBC, p.wait_budget);
      if (MODE == 0) ok = ok && mbar_wait(barA, par, p.wait_budget);
      if (__syncthreads_or(!ok)) { failed = LA_ERR_WAIT_INPUT; break; }
    }
    LA_TRACE(1)

    if (MODE == 0) {
      if (tid == 0) {
        tc_fence_after_sync();
        for (int kq = 0; kq < nk16; ++kq) {  // S = A Bm^T
          const uint32_t off = (kq >> 2) * SLAB + (kq & 3) * 32;
          umma_f16(tmem + T_S, smem_desc_sw128(sA + off, 16), smem_desc_sw128(sBs + off, 16), IDESC_S, kq > 0);
        }
        if (have_state) {
          for (int kq = 0; kq < nk16; ++kq) {  // O_inter = A State
            const uint32_t offA = (kq >> 2) * SLAB + (kq & 3) * 32;
            const uint32_t offS = (kq >> 2) * (DV * 128) + (kq & 3) * 32;
            umma_f16(tmem + T_OX, smem_desc_sw128(sA + offA, 16), smem_desc_sw128(sS + offS, 16), IDESC_X, kq > 0);
          }
        }
        umma_commit(barM1);
      }
      // ---- 2. S ready: mask it into P, scale Bm rows for the state update --------------------
      {
        const bool ok = mbar_wait(barM1, par, p.wait_budget);
        if (__syncthreads_or(!ok)) { failed = LA_ERR_WAIT_MMA1; break; }
      }
      LA_TRACE(2)
      tc_fence_after_sync();
      if (tid == 0 && has_next) {
        issue_A(nxt);
        if (nstage == 2) issue_BC(nxt, stage ^ 1);
      }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c0 = hf * 64 + cc * 32;
        // warp-uniform: is this 32x32 tile entirely on the masked side?
        const bool dead = reverse ? (c0 + 31 < q * 32) : (c0 > q * 32 + 31);
        uint32_t v[32];
        if (!dead) {
          tmem_ld32(tmem + lanebase + T_S + c0, v);
          tmem_wait_ld();
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float f0 = 0.f, f1 = 0.f;
          if (!dead) {
            const int d0 = reverse ? (c0 + i - r) : (r - c0 - i);  // distance on the causal side when >= 0
            const int d1 = reverse ? (d0 + 1) : (d0 - 1);
            if (d0 >= 0) f0 = __uint_as_float(v[i]) * decay_tab[d0];
            if (d1 >= 0) f1 = __uint_as_float(v[i + 1]) * decay_tab[d1];
          }
          pk[i >> 1] = pack2<FMT>(f0, f1);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t addr = sP + hf * SLAB + r * 128 + (((cc * 4 + g) ^ (r & 7)) << 4);
          st_shared_v4(addr, pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        }
      }
    } else {
      if (tid == 0 && has_next && nstage == 2) issue_BC(nxt, stage ^ 1);
    }

    // Bm rows *= w_state(r), in place (the S MMA no longer needs the unscaled tile)
    const bool tail_blk = tail_fix && it == nb - 1;
    const float w_st = tail_blk ? w_tail : w_state;
#pragma unroll
    for (int i = 0; i < NKS * 4; ++i) {
      const int g = hf * NKS * 4 + i;
      const int ks = g >> 3, p0 = g & 7;
      const int pos = (p0 & 4) | ((p0 + r) & 3);
      const uint32_t addr = sBs + ks * SLAB + r * 128 + (pos << 4);
      uint32_t u0, u1, u2, u3;
      ld_shared_v4(addr, u0, u1, u2, u3);
      float2 f;
      f = unpack2<FMT>(u0); u0 = pack2<FMT>(f.x * w_st, f.y * w_st);
      f = unpack2<FMT>(u1); u1 = pack2<FMT>(f.x * w_st, f.y * w_st);
      f = unpack2<FMT>(u2); u2 = pack2<FMT>(f.x * w_st, f.y * w_st);
      f = unpack2<FMT>(u3); u3 = pack2<FMT>(f.x * w_st, f.y * w_st);
      st_shared_v4(addr, u0, u1, u2, u3);
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    LA_TRACE(3)

    // ---- 3. O_intra = P C ; StateT_local = C^T (w_state Bm) ------------------------------------
    if (tid == 0) {
      tc_fence_after_sync();
      if (MODE == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          umma_f16(tmem + T_OI, smem_desc_sw128(sP + (kk >> 2) * SLAB + (kk & 3) * 32, 16),
                   smem_desc_sw128(sCs + kk * 2048, SLAB), IDESC_PC, kk > 0);
        }
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        umma_f16(tmem + T_D, smem_desc_sw128(sCs + kk * 2048, SLAB), smem_desc_sw128(sBs + kk * 2048, SLAB),
                 IDESC_ST, kk > 0);
      }
      umma_commit(barM2);
    }
    {
      const bool ok = mbar_wait(barM2, par, p.wait_budget);
      if (__syncthreads_or(!ok)) { failed = LA_ERR_WAIT_MMA2; break; }
    }
    LA_TRACE(4)
    tc_fence_after_sync();
    if (tid == 0 && has_next && nstage == 1) issue_BC(nxt, 0);

    // ---- 4. epilogue: out rows, then the state recurrence ---------------------------------------
    if (MODE == 0) {
      const int tok = blk * LA_BLOCK + r;
#pragma unroll
      for (int cc = 0; cc < OC; cc += 32) {
        uint32_t a[32], b[32];
        tmem_ld32(tmem + lanebase + T_OI + hf * OC + cc, a);
        if (have_state) tmem_ld32(tmem + lanebase + T_OX + hf * OC + cc, b);
        tmem_wait_ld();
        if (tok < p.n) {
          const int col0 = dv_off + hf * OC + cc;
          uint8_t* orow = static_cast<uint8_t*>(p.out) + ((static_cast<size_t>(bh) * p.n + tok) * p.dv + col0) * 2;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + g * 8 < p.dv) {
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
              *reinterpret_cast<uint4*>(orow + g * 16) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
          }
        }
      }
    }
    if (q * 32 < DV) {  // warp-uniform: lanes >= DV of the state accumulator hold nothing useful
#pragma unroll
      for (int cc = 0; cc < SC; cc += 32) {
        uint32_t dl[32];
        tmem_ld32(tmem + lanebase + T_D + hf * SC + cc, dl);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) st[cc + i] = fmaf(tail_blk ? decay_tail : decay_blk, st[cc + i], __uint_as_float(dl[i]));
      }
      if (MODE == 0 && has_next) store_state_smem();
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    LA_TRACE(5)
  }
#undef LA_TRACE

  if (!failed && p.state_out != nullptr && st_row_valid) {
    float* dst = p.state_out +
        ((static_cast<size_t>(bh) * p.state_slots + chunk) * p.dv + dv_off + r) * p.dk + hf * SC;
#pragma unroll
    for (int i = 0; i < SC; i += 4) {
      if (hf * SC + i < p.dk) *reinterpret_cast<float4*>(dst + i) = make_float4(st[i], st[i + 1], st[i + 2], st[i + 3]);
    }
  }
  if (failed && tid == 0) atomicExch(p.status, failed);

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// Exclusive decayed scan over the per-chunk local states, in place:
//   forward time:  prefix[c] = run;  run = lambda^(tokens in chunk c) * run + local[c]   for c = 0..nchunks-1
//   reverse time:  the same for c = nchunks-1..0.
// `init` seeds `run` (state arriving from outside the sequence), `total` receives the final run.
// The reference's unfinished "parallel" variant does the same with one program per head
// (lightning_attn2_parallel.py:198-249, :650-701); here every state element is an independent thread.
// When `skip_last` is set the local state of the last chunk in scan order was not computed and is ignored.
__global__ void la_scan_kernel(float* __restrict__ states, const float* __restrict__ init, float* __restrict__ total,
                               const float* __restrict__ slopes, int h, int nchunks, int elems, int nblocks,
                               int blocks_per_chunk, int n, int reverse, int skip_last, long long total_elems) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total_elems) return;
  const int bh = static_cast<int>(idx / elems);
  const int e = static_cast<int>(idx - static_cast<long long>(bh) * elems);
  const float s = slopes ? slopes[bh % h] : 0.f;
  float run = init ? init[idx] : 0.f;
  for (int k = 0; k < nchunks; ++k) {
    const int c = reverse ? (nchunks - 1 - k) : k;
    const int nb = min(nblocks, (c + 1) * blocks_per_chunk) - c * blocks_per_chunk;
    float* ptr = states + (static_cast<size_t>(bh) * nchunks + c) * elems + e;
    const float loc = (skip_last && k == nchunks - 1) ? 0.f : *ptr;
    *ptr = run;
    // forward time: the last chunk may end in a ragged block, and its local state is decayed to token n (see the block kernels)
    const int tokens = reverse ? nb * LA_BLOCK : min(n, (c * blocks_per_chunk + nb) * LA_BLOCK) - c * blocks_per_chunk * LA_BLOCK;
    run = __expf(-s * static_cast<float>(tokens)) * run + loc;
  }
  if (total) total[idx] = run;
}

// Adds a state that arrives from outside the sequence to per-chunk prefix states that were computed from a zero
// initial state: prefix[c] += lambda^(tokens between the sequence edge and chunk c) * init. Lets a caller compute the
// local states first, learn the incoming state later (sequence parallelism) and still run the chunk pass only once.
__global__ void la_rebase_kernel(float* __restrict__ states, const float* __restrict__ init,
                                 const float* __restrict__ slopes, int h, int nchunks, int elems, int nblocks,
                                 int blocks_per_chunk, int reverse, long long total_elems) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total_elems) return;
  const int bh = static_cast<int>(idx / elems);
  const int e = static_cast<int>(idx - static_cast<long long>(bh) * elems);
  const float s = slopes ? slopes[bh % h] : 0.f;
  const float v = init[idx];
  for (int c = 0; c < nchunks; ++c) {
    const int before = reverse ? (nblocks - min(nblocks, (c + 1) * blocks_per_chunk)) : c * blocks_per_chunk;
    states[(static_cast<size_t>(bh) * nchunks + c) * elems + e] += __expf(-s * static_cast<float>(before * LA_BLOCK)) * v;
  }
}

// State entering this rank's sequence shard from the all-gathered local shard states (sequence parallelism):
//   forward time:  out = sum_{r < rank} lambda^((rank-1-r) L) gathered[r]
//   reverse time:  out = sum_{r > rank} lambda^((r-rank-1) L) gathered[r]
// gathered is (R, bh, X, Y) fp32, L the tokens per shard. `out` (bh, X, Y) and/or `out_t` (bh, Y, X, the same state
// for the product with Bm and C exchanged) may be null. Grid (ceil(Y/32), ceil(X/32), bh), block (32, 8).
__global__ void la_combine_kernel(const float* __restrict__ gathered, const float* __restrict__ slopes,
                                  float* __restrict__ out, float* __restrict__ out_t, int R, int rank, int bh_total, int h,
                                  int X, int Y, float shard_tokens, int reverse) {
  __shared__ float tile[32][33];
  const int bh = blockIdx.z;
  const int x0 = blockIdx.y * 32, y0 = blockIdx.x * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const float s = slopes ? slopes[bh % h] : 0.f;
  const int r_begin = reverse ? rank + 1 : 0, r_end = reverse ? R : rank;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int y = y0 + tx;
  for (int r = r_begin; r < r_end; ++r) {
    const int expo = reverse ? (r - rank - 1) : (rank - 1 - r);
    const float w = expf(-s * shard_tokens * static_cast<float>(expo));
    const float* src = gathered + (static_cast<size_t>(r) * bh_total + bh) * X * Y;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int x = x0 + ty + 8 * k;
      if (x < X && y < Y) acc[k] = fmaf(w, src[static_cast<size_t>(x) * Y + y], acc[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int x = x0 + ty + 8 * k;
    if (out && x < X && y < Y) out[(static_cast<size_t>(bh) * X + x) * Y + y] = acc[k];
    tile[ty + 8 * k][tx] = acc[k];
  }
  if (out_t) {
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int yy = y0 + ty + 8 * k, xx = x0 + tx;  // out_t[yy][xx] = state[xx][yy]
      if (yy < Y && xx < X) out_t[(static_cast<size_t>(bh) * Y + yy) * X + xx] = tile[tx][ty + 8 * k];
    }
  }
}

// In-place transpose of `count` square D x D fp32 matrices stored back to back (the per-chunk states of a product,
// turned into those of the product with Bm and C exchanged). Grid (count, tile pairs i <= j), block (32, 8).
__global__ void la_transpose_square_kernel(float* __restrict__ m, int D) {
  __shared__ float ta[32][33], tb[32][33];
  const int nt = (D + 31) / 32;
  int pair = blockIdx.y, ti = 0;
  for (; ti < nt && pair >= nt - ti; ++ti) pair -= nt - ti;  // row ti of the upper triangle of tile pairs
  if (ti >= nt) return;
  const int tj = ti + pair;
  float* base = m + static_cast<size_t>(blockIdx.x) * D * D;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = ty + 8 * k;
    const int ai = ti * 32 + r, aj = tj * 32 + tx;  // tile (ti, tj)
    const int bi = tj * 32 + r, bj = ti * 32 + tx;  // tile (tj, ti)
    ta[r][tx] = (ai < D && aj < D) ? base[static_cast<size_t>(ai) * D + aj] : 0.f;
    tb[r][tx] = (bi < D && bj < D) ? base[static_cast<size_t>(bi) * D + bj] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = ty + 8 * k;
    const int ai = ti * 32 + r, aj = tj * 32 + tx;
    const int bi = tj * 32 + r, bj = ti * 32 + tx;
    if (ai < D && aj < D) base[static_cast<size_t>(ai) * D + aj] = tb[tx][r];
    if (ti != tj && bi < D && bj < D) base[static_cast<size_t>(bi) * D + bj] = ta[tx][r];
  }
}

// One decode step of the recurrence for every (batch, head) pair (inference; no counterpart in the reference):
//   o = q (S + k^T v),   S <- lambda (S + k^T v),
// S being the (dv, dk) fp32 state entering the token (what the block kernels hand out as state_out). A warp owns
// LA_DECODE_ROWS state rows and keeps one 16-byte load per row in flight; 8 warps per CTA: grid
// (ceil(dv / (8 LA_DECODE_ROWS)), bh), block 256. HBM-bound on the state: 8 bytes per element.
constexpr int LA_DECODE_ROWS = 8;

template <int FMT>
__global__ void __launch_bounds__(256)
la_decode_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k, const uint16_t* __restrict__ v,
                 const float* __restrict__ slopes, float* __restrict__ state, uint16_t* __restrict__ o, int h, int dk,
                 int dv) {
  const int bh = blockIdx.y;
  const int row0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * LA_DECODE_ROWS;
  const int lane = threadIdx.x & 31;
  if (row0 >= dv) return;
  const float lam = slopes ? __expf(-slopes[bh % h]) : 1.f;
  auto to_f = [](uint32_t x) -> float {  // low 16 bits of x
    if constexpr (FMT == 1) return __uint_as_float(x << 16);
    else return __half2float(__ushort_as_half(static_cast<unsigned short>(x & 0xffffu)));
  };
  float ve[LA_DECODE_ROWS], acc[LA_DECODE_ROWS];
#pragma unroll
  for (int j = 0; j < LA_DECODE_ROWS; ++j) {
    ve[j] = (row0 + j < dv) ? to_f(v[static_cast<size_t>(bh) * dv + row0 + j]) : 0.f;
    acc[j] = 0.f;
  }
  const uint16_t* qp = q + static_cast<size_t>(bh) * dk;
  const uint16_t* kp = k + static_cast<size_t>(bh) * dk;
  float* sp = state + (static_cast<size_t>(bh) * dv + row0) * dk;
  for (int c = lane * 4; c < dk; c += 128) {
    float4 st[LA_DECODE_ROWS];
#pragma unroll
    for (int j = 0; j < LA_DECODE_ROWS; ++j)
      st[j] = (row0 + j < dv) ? *reinterpret_cast<const float4*>(sp + static_cast<size_t>(j) * dk + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    const uint2 qq = *reinterpret_cast<const uint2*>(qp + c);
    const uint2 kk = *reinterpret_cast<const uint2*>(kp + c);
    const float k0 = to_f(kk.x & 0xffffu), k1 = to_f(kk.x >> 16), k2 = to_f(kk.y & 0xffffu), k3 = to_f(kk.y >> 16);
    const float q0 = to_f(qq.x & 0xffffu), q1 = to_f(qq.x >> 16), q2 = to_f(qq.y & 0xffffu), q3 = to_f(qq.y >> 16);
#pragma unroll
    for (int j = 0; j < LA_DECODE_ROWS; ++j) {
      float4 nw;
      nw.x = fmaf(k0, ve[j], st[j].x);
      nw.y = fmaf(k1, ve[j], st[j].y);
      nw.z = fmaf(k2, ve[j], st[j].z);
      nw.w = fmaf(k3, ve[j], st[j].w);
      acc[j] = fmaf(q0, nw.x, fmaf(q1, nw.y, fmaf(q2, nw.z, fmaf(q3, nw.w, acc[j]))));
      if (row0 + j < dv)
        *reinterpret_cast<float4*>(sp + static_cast<size_t>(j) * dk + c) = make_float4(lam * nw.x, lam * nw.y, lam * nw.z, lam * nw.w);
    }
  }
#pragma unroll
  for (int j = 0; j < LA_DECODE_ROWS; ++j) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  }
  if (lane < LA_DECODE_ROWS && row0 + lane < dv) {
    float mine = acc[0];
#pragma unroll
    for (int j = 1; j < LA_DECODE_ROWS; ++j) mine = (lane == j) ? acc[j] : mine;
    uint16_t out;
    if constexpr (FMT == 1) {
      const __nv_bfloat16 bb = __float2bfloat16_rn(mine);
      out = *reinterpret_cast<const uint16_t*>(&bb);
    } else {
      const __half hh = __float2half_rn(mine);
      out = *reinterpret_cast<const uint16_t*>(&hh);
    }
    o[static_cast<size_t>(bh) * dv + row0 + lane] = out;
  }
}

}  // namespace lab200
