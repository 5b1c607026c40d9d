// C-ABI entry points of liblightning_b200.so (declared in include/lightning_b200.h).
// Host side only: argument checks, tensor-map encoding, kernel selection and launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "../../include/lightning_b200.h"
#include "la_kernels.cuh"
#include "la_pipe_kernel.cuh"
#include "la_dkdv2_kernel.cuh"
#include "srmsnorm_kernels.cuh"

using namespace lab200;

namespace {

constexpr size_t WS_HEADER = 256;            // status block in front of the workspace
constexpr int SMEM_LIMIT = 232448;           // 227 KB opt-in dynamic shared memory per CTA
constexpr long long WAIT_BUDGET = 2000000000LL;  // ~1 s of SM clocks per barrier wait

std::atomic<long long> g_launches{0};  // kernels launched by this library since load
std::atomic<long long*> g_trace{nullptr};  // optional device buffer for per-block clock stamps
std::atomic<int> g_trace_blocks{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int sm_count() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

// (bh, n, dim) row-major 16-bit tensor -> boxes of 64 features x 128 tokens, 128-byte swizzle,
// out-of-range rows and columns read as zero.
// layout 1: the tensor is (b, n, h, dim) contiguous instead. Token t of pair (b, hd) then starts at element
// ((b n + t) h + hd) dim = (b n h + hd) dim + t (h dim): still a three-dimensional map, with token stride h dim and a
// third dimension of extent b n h and stride dim that the kernel indexes by b n h + hd; tokens >= n stay out of range.
int make_tmap(CUtensorMap* tm, const void* ptr, int bh, int n, int dim, int dtype, int layout = 0, int h = 1) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return LAB200_ERR_DRIVER;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(dim), static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(bh)};
  cuuint64_t gstr[2] = {static_cast<cuuint64_t>(dim) * 2, static_cast<cuuint64_t>(n) * dim * 2};
  if (layout) {
    gdim[2] = static_cast<cuuint64_t>(bh) * n;  // b n h
    gstr[0] = static_cast<cuuint64_t>(h) * dim * 2;
    gstr[1] = static_cast<cuuint64_t>(dim) * 2;
  }
  const cuuint32_t box[3] = {64, LA_BLOCK, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = (dtype == LAB200_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(tm, dt, 3, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LAB200_OK : LAB200_ERR_DRIVER;
}

struct Tiling {
  int nks, nvs, nslices;
};

bool pick_tiling(int dk, int dv, Tiling* t) {
  if (dk < 16 || dv < 16 || (dk % 16) || (dv % 16) || dk > 256) return false;
  t->nks = (dk + 63) / 64;
  t->nvs = (t->nks <= 2 && dv > 64) ? 2 : 1;
  t->nslices = (dv + 64 * t->nvs - 1) / (64 * t->nvs);
  if (t->nslices > 65535) return false;
  return true;
}

int smem_bytes(int nks, int nvs, int mode, int nstage) {
  const int slab = LA_SLAB_BYTES;
  int b = nstage * (nks + 2) * slab;
  if (mode == 0) b += nks * slab + 2 * slab + nks * nvs * 64 * 128;
  return b + 64 + 512 + 1024;  // barriers + decay table + alignment slack
}

int plan_chunks(int bh, int n, int dk, int dv) {
  Tiling t;
  if (!pick_tiling(dk, dv, &t)) return 1;
  const int nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  const long long units = static_cast<long long>(bh) * t.nslices;
  const int sms = sm_count();
  if (units * 10 >= sms * 8LL) return 1;  // a serial sweep per unit already fills >= 80 % of the SMs
  long long c = sms / (units > 0 ? units : 1);
  const int max_c = nblocks / 2 > 0 ? nblocks / 2 : 1;  // at least two blocks per chunk
  if (c > max_c) c = max_c;
  if (c < 1) c = 1;
  return static_cast<int>(c);
}

template <int NKS, int NVS, int MODE, int FMT>
int launch_one(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const LaParams& p, dim3 grid,
               int smem, cudaStream_t st) {
  auto kern = la_chunk_kernel<NKS, NVS, MODE, FMT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    cudaGetLastError();
    return LAB200_ERR_CUDA;
  }
  kern<<<grid, LA_THREADS, smem, st>>>(tA, tB, tC, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

template <int MODE, int FMT>
int launch_tiled(int nks, int nvs, const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                 const LaParams& p, dim3 grid, int smem, cudaStream_t st) {
#define LAB200_CASE(K, V) \
  if (nks == K && nvs == V) return launch_one<K, V, MODE, FMT>(tA, tB, tC, p, grid, smem, st);
  LAB200_CASE(1, 1)
  LAB200_CASE(1, 2)
  LAB200_CASE(2, 1)
  LAB200_CASE(2, 2)
  LAB200_CASE(3, 1)
  LAB200_CASE(4, 1)
#undef LAB200_CASE
  return LAB200_ERR_SHAPE;
}

// ---- pipelined kernel (dk <= 128) ---------------------------------------------------------------
int smem_bytes_pipe(int nks, int nvs, int mode) {
  const int slab = LA_SLAB_BYTES;
  int b = 2 * nks * slab + 4 * slab;
  if (mode == 0) b += 2 * (nks > nvs ? nks : nvs) * slab + nks * nvs * 64 * 128;  // A stages also stage the output tile
  return b + 2 * LAP_NUM_BARS * 8 + 16 + 512 + 1024;  // barriers, flags, decay table, alignment slack
}

template <int NKS, int NVS, int MODE, int FMT>
int launch_pipe_one(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, const CUtensorMap& tO,
                    const LaParams& p, dim3 grid, int smem, cudaStream_t st) {
  auto kern = la_pipe_kernel<NKS, NVS, MODE, FMT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    cudaGetLastError();
    return LAB200_ERR_CUDA;
  }
  kern<<<grid, LAP_THREADS, smem, st>>>(tA, tB, tC, tO, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

template <int MODE, int FMT>
int launch_pipe(int nks, int nvs, const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC,
                const CUtensorMap& tO, const LaParams& p, dim3 grid, int smem, cudaStream_t st) {
#define LAB200_CASE(K, V) \
  if (nks == K && nvs == V) return launch_pipe_one<K, V, MODE, FMT>(tA, tB, tC, tO, p, grid, smem, st);
  LAB200_CASE(1, 1)
  LAB200_CASE(1, 2)
  LAB200_CASE(2, 1)
  LAB200_CASE(2, 2)
#undef LAB200_CASE
  return LAB200_ERR_SHAPE;
}

// LIGHTNING_B200_SERIAL=1 in the environment selects the serial block kernel for every shape (A/B comparisons).
bool use_pipelined_kernel() {
  static const bool on = [] {
    const char* e = getenv("LIGHTNING_B200_SERIAL");
    return !(e && e[0] == '1');
  }();
  return on;
}

int launch_la(int mode, int dtype, const Tiling& t, const CUtensorMap& tA, const CUtensorMap& tB,
              const CUtensorMap& tC, const CUtensorMap& tO, LaParams p, int nchunks_grid, int bh, cudaStream_t st) {
  if (t.nks <= 2 && use_pipelined_kernel()) {
    const int smem = smem_bytes_pipe(t.nks, t.nvs, mode);
    if (smem <= SMEM_LIMIT) {
      p.nstage = 2;
      const dim3 grid(t.nslices, nchunks_grid, bh);
      if (mode == 0) {
        return dtype == LAB200_BF16 ? launch_pipe<0, 1>(t.nks, t.nvs, tA, tB, tC, tO, p, grid, smem, st)
                                    : launch_pipe<0, 0>(t.nks, t.nvs, tA, tB, tC, tO, p, grid, smem, st);
      }
      return dtype == LAB200_BF16 ? launch_pipe<1, 1>(t.nks, t.nvs, tA, tB, tC, tO, p, grid, smem, st)
                                  : launch_pipe<1, 0>(t.nks, t.nvs, tA, tB, tC, tO, p, grid, smem, st);
    }
  }
  int nstage = 2;
  int smem = smem_bytes(t.nks, t.nvs, mode, nstage);
  if (smem > SMEM_LIMIT) {
    nstage = 1;
    smem = smem_bytes(t.nks, t.nvs, mode, nstage);
  }
  if (smem > SMEM_LIMIT) return LAB200_ERR_SHAPE;
  p.nstage = nstage;
  const dim3 grid(t.nslices, nchunks_grid, bh);
  if (mode == 0) {
    return dtype == LAB200_BF16 ? launch_tiled<0, 1>(t.nks, t.nvs, tA, tB, tC, p, grid, smem, st)
                                : launch_tiled<0, 0>(t.nks, t.nvs, tA, tB, tC, p, grid, smem, st);
  }
  return dtype == LAB200_BF16 ? launch_tiled<1, 1>(t.nks, t.nvs, tA, tB, tC, p, grid, smem, st)
                              : launch_tiled<1, 0>(t.nks, t.nvs, tA, tB, tC, p, grid, smem, st);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int la_validate(const void* a, const void* bm, const void* c, const void* out, const float* state_in,
                const float* state_out, const void* workspace, int bh, int h, int n, int dk, int dv, int state_only,
                int dtype);

// The generic product without the status reset (so that composite calls share one status word).
// PREFIX_ONLY: stop once the state entering every chunk is in the workspace (computed, or with RESUME taken over from
// an earlier call and rebased); the block loop is the caller's business (the fused dk+dv sweep). a and out may be null.
enum : int { RESUME = 1, RESUME_SWAPPED = 2, RESUME_NO_REBASE = 4, PREFIX_ONLY = 8 };

// Number of chunks la_generic_impl cuts the sequence into.
int chunk_count(int bh, int n, int dk, int dv, int chunks) {
  const int nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  int nchunks = chunks > 0 ? chunks : plan_chunks(bh, n, dk, dv);
  if (nchunks > nblocks) nchunks = nblocks;
  const int bpc = (nblocks + nchunks - 1) / nchunks;
  return (nblocks + bpc - 1) / bpc;  // drop empty trailing chunks
}

int la_generic_impl(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                    const float* state_in, float* state_out, void* workspace, size_t workspace_bytes, int bh, int h,
                    int n, int dk, int dv, int reverse, int state_only, int chunks, int dtype, cudaStream_t st,
                    int resume = 0) {
  const bool prefix_only = (resume & PREFIX_ONLY) != 0;
  int rc = la_validate(a, bm, c, out, state_in, state_out, workspace, bh, h, n, dk, dv, prefix_only ? 2 : state_only, dtype);
  if (rc != LAB200_OK) return rc;
  const int layout = (dtype & LAB200_LAYOUT_BNHD) ? 1 : 0;
  dtype &= 0xff;
  Tiling t;
  pick_tiling(dk, dv, &t);
  const int nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  const int nchunks = chunk_count(bh, n, dk, dv, chunks);
  const int bpc = (nblocks + nchunks - 1) / nchunks;
  if (nchunks > 65535) return LAB200_ERR_SHAPE;
  const size_t need = WS_HEADER + (nchunks > 1 ? static_cast<size_t>(bh) * nchunks * dv * dk * sizeof(float) : 0);
  if (!workspace || workspace_bytes < need) return LAB200_ERR_WORKSPACE;

  CUtensorMap tA, tB, tC, tO;
  if ((rc = make_tmap(&tB, bm, bh, n, dk, dtype, layout, h)) != LAB200_OK) return rc;
  if ((rc = make_tmap(&tC, c, bh, n, dv, dtype, layout, h)) != LAB200_OK) return rc;
  if (state_only || prefix_only) {
    tA = tB;
    tO = tC;
  } else {
    if ((rc = make_tmap(&tA, a, bh, n, dk, dtype, layout, h)) != LAB200_OK) return rc;
    if ((rc = make_tmap(&tO, out, bh, n, dv, dtype, layout, h)) != LAB200_OK) return rc;  // output tiles leave through TMA stores
  }

  LaParams p;
  p.out = out;
  p.slopes = slopes;
  p.status = static_cast<int*>(workspace);
  p.n = n; p.h = h; p.dk = dk; p.dv = dv;
  p.nblocks = nblocks;
  p.blocks_per_chunk = bpc;
  p.reverse = reverse ? 1 : 0;
  p.layout = layout;
  p.nstage = 2;
  p.wait_budget = WAIT_BUDGET;
  p.trace = g_trace.load(std::memory_order_relaxed);
  p.trace_blocks = g_trace_blocks.load(std::memory_order_relaxed);

  if (nchunks == 1) {
    if (prefix_only) return LAB200_OK;  // a single sweep takes state_in as it is
    p.chunk0 = 0;
    p.state_slots = 1;
    p.state_in = state_in;
    p.state_out = state_out;
    return launch_la(state_only ? 1 : 0, dtype, t, tA, tB, tC, tO, p, 1, bh, st);
  }

  // three phases: local chunk states -> decayed scan -> block loop per chunk with its incoming state
  float* states = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + WS_HEADER);
  if (resume & RESUME) {
    // the workspace already holds the per-chunk prefix states of a preceding call: go straight to the block loop.
    // RESUME_SWAPPED: they belong to the product with Bm and C exchanged, i.e. they are the transposes (dk == dv).
    // Unless RESUME_NO_REBASE is set they were computed from a zero initial state and the decayed incoming state is added.
    if (resume & RESUME_SWAPPED) {
      if (dk != dv) return LAB200_ERR_SHAPE;
      const int nt = (dk + 31) / 32;
      la_transpose_square_kernel<<<dim3(static_cast<unsigned>(bh) * nchunks, nt * (nt + 1) / 2), dim3(32, 8), 0, st>>>(states, dk);
      g_launches.fetch_add(1, std::memory_order_relaxed);
      if (cudaGetLastError() != cudaSuccess) return LAB200_ERR_CUDA;
    }
    if (state_in != nullptr && !(resume & RESUME_NO_REBASE)) {
      const int elems_r = dv * dk;
      const long long total_r = static_cast<long long>(bh) * elems_r;
      la_rebase_kernel<<<static_cast<unsigned>((total_r + 255) / 256), 256, 0, st>>>(states, state_in, slopes, h, nchunks, elems_r,
                                                                                  nblocks, bpc, p.reverse, total_r);
      g_launches.fetch_add(1, std::memory_order_relaxed);
      if (cudaGetLastError() != cudaSuccess) return LAB200_ERR_CUDA;
    }
    if (prefix_only) return LAB200_OK;
    p.state_slots = nchunks;
    p.chunk0 = 0;
    p.state_in = states;
    p.state_out = nullptr;
    return launch_la(0, dtype, t, tA, tB, tC, tO, p, nchunks, bh, st);
  }
  const bool need_total = (state_out != nullptr);
  const int skip_last = need_total ? 0 : 1;
  p.state_slots = nchunks;
  p.state_in = nullptr;
  p.state_out = states;
  p.chunk0 = (skip_last && reverse) ? 1 : 0;
  // The state-only pass runs one CTA per (dv slice, chunk that feeds a later one, pair): with two chunks per pair that is half as
  // many CTAs as the block loop gets. When twice as many still fit in one wave, it runs on 64-wide dv slices instead of 128-wide
  // ones (the states land in the same [dv][dk] layout; Bm is then read twice, the second time from L2).
  Tiling ts = t;
  if (t.nvs == 2 && 2LL * t.nslices * (nchunks - skip_last) * bh <= sm_count()) {
    ts.nvs = 1;
    ts.nslices = (dv + 63) / 64;
  }
  if ((rc = launch_la(1, dtype, ts, tB, tB, tC, tC, p, nchunks - skip_last, bh, st)) != LAB200_OK) return rc;

  const int elems = dv * dk;
  const long long total = static_cast<long long>(bh) * elems;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  la_scan_kernel<<<blocks, threads, 0, st>>>(states, state_in, state_out, slopes, h, nchunks, elems, nblocks, bpc, n,
                                             p.reverse, skip_last, total);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (cudaGetLastError() != cudaSuccess) return LAB200_ERR_CUDA;
  if (state_only || prefix_only) return LAB200_OK;

  p.chunk0 = 0;
  p.state_in = states;
  p.state_out = nullptr;
  return launch_la(0, dtype, t, tA, tB, tC, tO, p, nchunks, bh, st);
}

// ---- fused dk + dv (one reverse sweep) -----------------------------------------------------------------
int smem_bytes_dkdv(int ne) {
  return 12 * LA_SLAB_BYTES + ne * LA_SLAB_BYTES + 2 * LD2_NUM_BARS * 8 + 16 + 512 + 1024;  // q 2, do 4, k 2, v 2, staging 2, state copy ne
}

template <int ND, int NE, int FMT>
int launch_dkdv_one(const CUtensorMap (&tm)[6], const LaDkdvParams& p, dim3 grid, int smem, cudaStream_t st) {
  auto kern = la_dkdv2_kernel<ND, NE, FMT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    cudaGetLastError();
    return LAB200_ERR_CUDA;
  }
  kern<<<grid, LD2_THREADS, smem, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

// lab200_la2_bwd computes dk and dv with the fused sweep (6 tensor passes instead of the 8 of two generic launches)
// unless LIGHTNING_B200_FUSED_BWD=0 is set (A/B comparisons). lab200_la2_dkdv always uses it.
bool use_fused_dkdv() {
  static const bool on = [] {
    const char* e = getenv("LIGHTNING_B200_FUSED_BWD");
    return !(e && e[0] == '0');
  }();
  return on && use_pipelined_kernel();
}

bool dkdv_shape_ok(int d, int e) { return d <= 128 && e <= 128 && (d % 16) == 0 && (e % 16) == 0 && d >= 16 && e >= 16; }

// dk and dv in one launch per chunk of the sequence. `states`: nullptr (one chunk: the sweep starts from a zero state) or
// the reverse-time state entering every chunk, [bh][nchunks][d][e] fp32. Returns LAB200_ERR_SHAPE if the shape is not
// covered, in which case the caller falls back to two generic launches.
int la_dkdv_impl(const void* q, const void* k, const void* v, const void* dout, const float* slopes, void* dk, void* dv,
                 void* workspace, const float* states, int nchunks, int bpc, int bh, int h, int n, int d, int e, int dtype,
                 cudaStream_t st) {
  const int layout = (dtype & LAB200_LAYOUT_BNHD) ? 1 : 0;
  dtype &= 0xff;
  if (!dkdv_shape_ok(d, e)) return LAB200_ERR_SHAPE;
  const int nd = (d + 63) / 64, ne = (e + 63) / 64;
  const int smem = smem_bytes_dkdv(ne);
  if (smem > SMEM_LIMIT) return LAB200_ERR_SHAPE;
  CUtensorMap tm[6];
  int rc;
  if ((rc = make_tmap(&tm[0], q, bh, n, d, dtype, layout, h)) != LAB200_OK) return rc;
  if ((rc = make_tmap(&tm[1], k, bh, n, d, dtype, layout, h)) != LAB200_OK) return rc;
  if ((rc = make_tmap(&tm[2], v, bh, n, e, dtype, layout, h)) != LAB200_OK) return rc;
  if ((rc = make_tmap(&tm[3], dout, bh, n, e, dtype, layout, h)) != LAB200_OK) return rc;
  if ((rc = make_tmap(&tm[4], dk, bh, n, d, dtype, layout, h)) != LAB200_OK) return rc;  // the output tiles leave through TMA stores
  if ((rc = make_tmap(&tm[5], dv, bh, n, e, dtype, layout, h)) != LAB200_OK) return rc;
  LaDkdvParams p;
  p.slopes = slopes;
  p.state_in = states;
  p.state_out = nullptr;
  p.status = static_cast<int*>(workspace);
  p.n = n; p.h = h; p.d = d; p.e = e;
  p.nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  p.blocks_per_chunk = states ? bpc : p.nblocks;
  p.chunk0 = 0;
  p.state_slots = states ? nchunks : 1;
  p.layout = layout;
  p.wait_budget = WAIT_BUDGET;
  p.trace = g_trace.load(std::memory_order_relaxed);
  p.trace_blocks = g_trace_blocks.load(std::memory_order_relaxed);
  const dim3 grid(1, states ? nchunks : 1, bh);
  const bool bf = (dtype == LAB200_BF16);
#define LAB200_CASE(D_, E_) \
  if (nd == D_ && ne == E_) return bf ? launch_dkdv_one<D_, E_, 1>(tm, p, grid, smem, st) : launch_dkdv_one<D_, E_, 0>(tm, p, grid, smem, st);
  LAB200_CASE(1, 1)
  LAB200_CASE(1, 2)
  LAB200_CASE(2, 1)
  LAB200_CASE(2, 2)
#undef LAB200_CASE
  return LAB200_ERR_SHAPE;
}

// The whole fused sweep: in chunk mode first the reverse-time state entering every chunk (state-only pass over do and q
// plus scan, or - resume - taken over from an earlier state-only call on (do, q) and rebased on state_in), then one
// launch over all chunks. state_in: (bh, d, e) fp32 state entering the sequence from its far end, or nullptr.
int la_dkdv_full(const void* q, const void* k, const void* v, const void* dout, const float* slopes, void* dk, void* dv,
                 const float* state_in, void* workspace, size_t workspace_bytes, int bh, int h, int n, int d, int e,
                 int chunks, int resume, int dtype, cudaStream_t st) {
  if (!dkdv_shape_ok(d, e)) return LAB200_ERR_SHAPE;
  const int nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  const int nchunks = chunk_count(bh, n, e, d, chunks);
  const int bpc = (nblocks + nchunks - 1) / nchunks;
  if (nchunks > 1) {
    // chunk states of the product (v, do, q): sum lambda^t q_t^T do_t laid out (d, e), exactly the kernel's dKV
    int rc = la_generic_impl(nullptr, dout, q, slopes, nullptr, state_in, nullptr, workspace, workspace_bytes, bh, h, n, e, d,
                             1, 0, chunks, dtype, st, PREFIX_ONLY | (resume ? RESUME : 0));
    if (rc != LAB200_OK) return rc;
    const float* states = reinterpret_cast<const float*>(static_cast<const uint8_t*>(workspace) + WS_HEADER);
    return la_dkdv_impl(q, k, v, dout, slopes, dk, dv, workspace, states, nchunks, bpc, bh, h, n, d, e, dtype, st);
  }
  return la_dkdv_impl(q, k, v, dout, slopes, dk, dv, workspace, state_in, 1, nblocks, bh, h, n, d, e, dtype, st);
}

// A reverse-time sweep starts in the last block; the state arriving there is taken to sit at the end of a full tile.
bool reverse_chain_ok(int reverse, const float* state_in, int n) {
  return !(reverse && state_in != nullptr && (n % LA_BLOCK) != 0);
}

// Argument checks that need no CUDA call; run before anything is enqueued.
int la_validate(const void* a, const void* bm, const void* c, const void* out, const float* state_in,
                const float* state_out, const void* workspace, int bh, int h, int n, int dk, int dv, int state_only,
                int dtype) {
  const int layout = dtype & LAB200_LAYOUT_BNHD;
  dtype &= 0xff;
  if (dtype != LAB200_BF16 && dtype != LAB200_F16) return LAB200_ERR_DTYPE;
  Tiling t;
  if (bh < 1 || bh > 65535 || h < 1 || n < 1 || !pick_tiling(dk, dv, &t)) return LAB200_ERR_SHAPE;
  // (b, n, h, dim) tensors: whole batches of h heads, third tensor-map coordinate b n h + head within int range, and
  // only the pipelined kernel (dk <= 128) reads and writes them
  if (layout && ((bh % h) != 0 || static_cast<long long>(bh) * n >= (1LL << 31) || t.nks > 2 || !use_pipelined_kernel()))
    return LAB200_ERR_SHAPE;
  if (!bm || !c || (!state_only && (!a || !out)) || (state_only == 1 && !state_out)) return LAB200_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(bm) || !aligned16(c) || !aligned16(out) || !aligned16(state_in) ||
      !aligned16(state_out) || !aligned16(workspace))
    return LAB200_ERR_ALIGN;
  return LAB200_OK;
}

int reset_status(void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!workspace || workspace_bytes < WS_HEADER) return LAB200_ERR_WORKSPACE;
  return cudaMemsetAsync(workspace, 0, 16, st) == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// SRMSNorm launch selection
// ---------------------------------------------------------------------------------------------
bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// LIGHTNING_B200_SRMS_WIDE=0 keeps every SRMSNorm kernel on 128-bit accesses (A/B comparisons).
bool use_wide_srms() {
  static const bool on = [] {
    const char* e = getenv("LIGHTNING_B200_SRMS_WIDE");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <int DT, int G, int VPT, int W>
void srms_launch(bool fwd, const void* x, const void* dy, void* out, float* rstd, long long M, int N, float eps,
                 cudaStream_t st) {
  constexpr int CTA = (G > 256 ? G : 256);
  constexpr int RPC = CTA / G;
  const unsigned grid = static_cast<unsigned>((M + RPC - 1) / RPC);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (fwd) {
    srmsnorm_fwd_kernel<DT, G, VPT, W><<<grid, CTA, 0, st>>>(x, out, rstd, static_cast<int>(M), N, eps);
  } else {
    srmsnorm_bwd_kernel<DT, G, VPT, W><<<grid, CTA, 0, st>>>(x, dy, rstd, out, static_cast<int>(M), N);
  }
}

template <int DT>
int srms_dispatch(bool fwd, const void* x, const void* dy, void* out, float* rstd, long long M, int N, float eps,
                  cudaStream_t st) {
  constexpr int EPV = SrmsVec<DT>::EPV;
  const bool vec_ok = (N % EPV == 0) && aligned16(x) && aligned16(out) && (fwd || aligned16(dy));
  if (!vec_ok) {
    const unsigned grid = static_cast<unsigned>(M);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (fwd) {
      srmsnorm_fwd_generic_kernel<DT><<<grid, 256, 0, st>>>(x, out, rstd, static_cast<int>(M), N, eps);
    } else {
      srmsnorm_bwd_generic_kernel<DT><<<grid, 256, 0, st>>>(x, dy, rstd, out, static_cast<int>(M), N);
    }
    return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
  }
#define LAB200_SRMS(G, V, W) \
  if (np <= G * V) { srms_launch<DT, G, V, W>(fwd, x, dy, out, rstd, M, N, eps, st); return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA; }
  // 256-bit accesses with L2 evict-first hints when the rows allow it (a multiple of two vectors, 32-byte aligned): one or two
  // packs per thread (the backward kernel holds two tensors' packs; with more per thread too few CTAs are resident to
  // overlap one row's loads with another row's reduction and stores)
  if (use_wide_srms() && (N % (2 * EPV)) == 0 && aligned32(x) && aligned32(out) && (fwd || aligned32(dy))) {
    const int np = N / (2 * EPV);
    LAB200_SRMS(32, 1, 2)
    LAB200_SRMS(32, 2, 2)
    LAB200_SRMS(128, 1, 2)
    LAB200_SRMS(128, 2, 2)
    LAB200_SRMS(256, 2, 2)
    LAB200_SRMS(512, 2, 2)
    LAB200_SRMS(512, 4, 2)
  }
  {
    const int np = N / EPV;
    // smallest G * VPT that covers the row; two to four vectors per thread stream best (measured on 2048- and 4096-wide rows)
    LAB200_SRMS(32, 2, 1)
    LAB200_SRMS(32, 4, 1)
    LAB200_SRMS(128, 2, 1)
    LAB200_SRMS(128, 4, 1)
    if (!fwd) {
      LAB200_SRMS(256, 4, 1)
      LAB200_SRMS(512, 4, 1)
    }
    LAB200_SRMS(128, 8, 1)
    LAB200_SRMS(256, 8, 1)
    LAB200_SRMS(512, 8, 1)
  }
#undef LAB200_SRMS
  return LAB200_ERR_SHAPE;
}

// Gated SRMSNorm: vectorised rows only (row length a multiple of the vector width, 16-byte aligned pointers, at most
// 2048 vectors so that three rows' worth of registers fit); callers compose the plain kernels otherwise.
template <int DT, int G, int VPT, int W>
void srms_gate_launch(bool fwd, const void* x, const void* g, const void* dy, void* out, void* dg, float* rstd, long long M,
                      int N, float eps, cudaStream_t st) {
  constexpr int CTA = (G > 256 ? G : 256);
  constexpr int RPC = CTA / G;
  const unsigned grid = static_cast<unsigned>((M + RPC - 1) / RPC);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (fwd) srmsnorm_gate_fwd_kernel<DT, G, VPT, W><<<grid, CTA, 0, st>>>(x, g, out, rstd, static_cast<int>(M), N, eps);
  else srmsnorm_gate_bwd_kernel<DT, G, VPT, W><<<grid, CTA, 0, st>>>(x, g, dy, rstd, out, dg, static_cast<int>(M), N);
}

template <int DT>
int srms_gate_dispatch(bool fwd, const void* x, const void* g, const void* dy, void* out, void* dg, float* rstd, long long M,
                       int N, float eps, cudaStream_t st) {
  constexpr int EPV = SrmsVec<DT>::EPV;
  if ((N % EPV) != 0) return LAB200_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(g) || !aligned16(out) || (!fwd && (!aligned16(dy) || !aligned16(dg)))) return LAB200_ERR_ALIGN;
  if (N / EPV > 2048) return LAB200_ERR_SHAPE;
#define LAB200_SRMSG(G, V, W) \
  if (np <= G * V) { srms_gate_launch<DT, G, V, W>(fwd, x, g, dy, out, dg, rstd, M, N, eps, st); return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA; }
  if (use_wide_srms() && (N % (2 * EPV)) == 0 && aligned32(x) && aligned32(g) && aligned32(out) &&
      (fwd || (aligned32(dy) && aligned32(dg)))) {
    const int np = N / (2 * EPV);
    LAB200_SRMSG(32, 1, 2)
    LAB200_SRMSG(32, 2, 2)
    LAB200_SRMSG(128, 1, 2)
    LAB200_SRMSG(128, 2, 2)
    LAB200_SRMSG(256, 2, 2)
    LAB200_SRMSG(512, 2, 2)
  }
  {
    const int np = N / EPV;
    LAB200_SRMSG(32, 2, 1)
    LAB200_SRMSG(32, 4, 1)
    LAB200_SRMSG(128, 2, 1)
    LAB200_SRMSG(128, 4, 1)
    LAB200_SRMSG(256, 4, 1)
    LAB200_SRMSG(512, 4, 1)
  }
#undef LAB200_SRMSG
  return LAB200_ERR_SHAPE;
}

int srms_gate_entry(bool fwd, const void* x, const void* g, const void* dy, void* out, void* dg, float* rstd, long long M,
                    int N, float eps, int dtype, cudaStream_t st) {
  if (M < 0 || N < 1 || M > 2147483647LL) return LAB200_ERR_SHAPE;
  if (!x || !g || !out || !rstd || (!fwd && (!dy || !dg))) return M == 0 ? LAB200_OK : LAB200_ERR_SHAPE;
  if (M == 0) return LAB200_OK;
  switch (dtype) {
    case LAB200_F32: return srms_gate_dispatch<SRMS_F32>(fwd, x, g, dy, out, dg, rstd, M, N, eps, st);
    case LAB200_F16: return srms_gate_dispatch<SRMS_F16>(fwd, x, g, dy, out, dg, rstd, M, N, eps, st);
    case LAB200_BF16: return srms_gate_dispatch<SRMS_BF16>(fwd, x, g, dy, out, dg, rstd, M, N, eps, st);
    default: return LAB200_ERR_DTYPE;
  }
}

int srms_entry(bool fwd, const void* x, const void* dy, void* out, float* rstd, long long M, int N, float eps,
               int dtype, cudaStream_t st) {
  if (M < 0 || N < 1 || M > 2147483647LL) return LAB200_ERR_SHAPE;
  if (!x || !out || !rstd || (!fwd && !dy)) return M == 0 ? LAB200_OK : LAB200_ERR_SHAPE;
  if (M == 0) return LAB200_OK;
  const int esz = (dtype == LAB200_F32) ? 4 : 2;
  if (static_cast<long long>(N) * esz > 65536) return LAB200_ERR_SHAPE;  // same limit as srmsnorm.py:94-97
  switch (dtype) {
    case LAB200_F32: return srms_dispatch<SRMS_F32>(fwd, x, dy, out, rstd, M, N, eps, st);
    case LAB200_F16: return srms_dispatch<SRMS_F16>(fwd, x, dy, out, rstd, M, N, eps, st);
    case LAB200_BF16: return srms_dispatch<SRMS_BF16>(fwd, x, dy, out, rstd, M, N, eps, st);
    default: return LAB200_ERR_DTYPE;
  }
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for lab200_la2_fwd_static: lives in the library's device image, so it exists on every
// GPU that loads the library, from load until the process ends.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[LAB200_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_static_scratch_addr[MAX_DEVICES] = {};
std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device. In host code the array's name is only a handle
// for the runtime, not an address a kernel could use; cudaGetSymbolAddress translates it, once per device.
int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    cudaGetLastError();
    return LAB200_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return LAB200_ERR_CUDA;
    }
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return LAB200_OK;
}

// ---------------------------------------------------------------------------------------------
// Device status without a host synchronisation: after the last launch of an attention call the library copies the
// call's status word into a slot of a small ring of pinned host memory (one ring per device, allocated on the first
// attention call on that device). lab200_last_status() scans the ring: a non-zero word means a bounded wait of an
// EARLIER call ran out. The copy is ordered behind the call's kernels, so the report is one or more calls late.
// ---------------------------------------------------------------------------------------------
constexpr int STATUS_RING = 64;
struct StatusRing {
  int* slots = nullptr;
  unsigned next = 0;
  bool tried = false;
};
StatusRing g_status_ring[MAX_DEVICES];
std::mutex g_status_mutex;

void post_status(const void* workspace, cudaStream_t st) {
  int dev = -1;
  if (!workspace || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  StatusRing& ring = g_status_ring[dev];
  if (!ring.slots && !ring.tried) {
    ring.tried = true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, STATUS_RING * sizeof(int), cudaHostAllocDefault) == cudaSuccess && p) {
      ring.slots = static_cast<int*>(p);
      for (int i = 0; i < STATUS_RING; ++i) ring.slots[i] = 0;
    } else {
      cudaGetLastError();
    }
  }
  if (!ring.slots) return;
  int* slot = ring.slots + (ring.next++ % STATUS_RING);
  if (cudaMemcpyAsync(slot, workspace, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) cudaGetLastError();
}

int finish_call(int rc, const void* workspace, cudaStream_t st) {
  if (rc == LAB200_OK) post_status(workspace, st);
  return rc;
}

// One CTA that waits, with the same bounded wait the block kernels use, on an mbarrier that nothing ever arrives on, and
// reports the expiry through the status word: exercises the error path (wait budget -> status word -> host) with no
// asynchronous copy, tensor-memory allocation or MMA in flight.
__global__ void la_wait_expiry_kernel(int* status, long long budget) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const bool ok = lap_wait(bar, 0, &abort_flag, budget);
  __syncthreads();
  if (threadIdx.x == 0 && !ok) atomicExch(status, LA_ERR_WAIT_INPUT);
}

}  // namespace

extern "C" {

int lab200_version(void) { return 100; }

void lab200_la_debug_trace(long long* device_buffer, int blocks) {
  g_trace_blocks.store(device_buffer ? blocks : 0, std::memory_order_relaxed);
  g_trace.store(device_buffer, std::memory_order_relaxed);
}

long long lab200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* lab200_error_string(int code) {
  switch (code) {
    case LAB200_OK: return "ok";
    case LAB200_ERR_SHAPE: return "unsupported or inconsistent sizes";
    case LAB200_ERR_DTYPE: return "unsupported dtype";
    case LAB200_ERR_WORKSPACE: return "workspace missing or too small";
    case LAB200_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
    case LAB200_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or refused the tensor map";
    case LAB200_ERR_ALIGN: return "pointer not 16-byte aligned";
    case LAB200_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the library's built-in 16 MiB";
    case LAB200_ERR_WAIT_INPUT: return "device: bounded wait for TMA input ran out";
    case LAB200_ERR_WAIT_MMA1: return "device: bounded wait for the first MMA group ran out";
    case LAB200_ERR_WAIT_MMA2: return "device: bounded wait for the second MMA group ran out";
    default: return "unknown error";
  }
}

int lab200_la_plan_chunks(int bh, int n, int dk, int dv) { return plan_chunks(bh, n, dk, dv); }

size_t lab200_la_workspace_bytes(int bh, int n, int dk, int dv, int chunks) {
  if (bh < 1 || n < 1 || dk < 1 || dv < 1) return WS_HEADER;
  const int nblocks = (n + LA_BLOCK - 1) / LA_BLOCK;
  int nchunks = chunks > 0 ? chunks : plan_chunks(bh, n, dk, dv);
  if (nchunks > nblocks) nchunks = nblocks;
  if (nchunks <= 1) return WS_HEADER;
  return WS_HEADER + static_cast<size_t>(bh) * nchunks * dv * dk * sizeof(float);
}

int lab200_la_generic(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                      const float* state_in, float* state_out, void* workspace, size_t workspace_bytes, int bh,
                      int h, int n, int dk, int dv, int reverse, int state_only, int chunks, int dtype,
                      void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = la_validate(a, bm, c, out, state_in, state_out, workspace, bh, h, n, dk, dv, state_only, dtype);
  if (rc != LAB200_OK) return rc;
  if (!reverse_chain_ok(reverse, state_in, n)) return LAB200_ERR_SHAPE;
  if ((rc = reset_status(workspace, workspace_bytes, st)) != LAB200_OK) return rc;
  return finish_call(la_generic_impl(a, bm, c, slopes, out, state_in, state_out, workspace, workspace_bytes, bh, h, n, dk, dv,
                         reverse, state_only, chunks, dtype, st), workspace, st);
}

int lab200_la_generic_resume(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                             const float* state_in, void* workspace, size_t workspace_bytes, int bh, int h, int n, int dk,
                             int dv, int reverse, int chunks, int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = la_validate(a, bm, c, out, state_in, nullptr, workspace, bh, h, n, dk, dv, 0, dtype);
  if (rc != LAB200_OK) return rc;
  if (!reverse_chain_ok(reverse, state_in, n)) return LAB200_ERR_SHAPE;
  if ((rc = reset_status(workspace, workspace_bytes, st)) != LAB200_OK) return rc;
  return finish_call(la_generic_impl(a, bm, c, slopes, out, state_in, nullptr, workspace, workspace_bytes, bh, h, n, dk, dv, reverse, 0,
                         chunks, dtype, st, RESUME), workspace, st);
}

int lab200_la_generic_resume_swapped(const void* a, const void* bm, const void* c, const float* slopes, void* out,
                                     const float* state_in, void* workspace, size_t workspace_bytes, int bh, int h, int n,
                                     int dk, int dv, int reverse, int chunks, int rebase, int dtype, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dk != dv) return LAB200_ERR_SHAPE;
  int rc = la_validate(a, bm, c, out, state_in, nullptr, workspace, bh, h, n, dk, dv, 0, dtype);
  if (rc != LAB200_OK) return rc;
  if (!reverse_chain_ok(reverse, state_in, n)) return LAB200_ERR_SHAPE;
  if ((rc = reset_status(workspace, workspace_bytes, st)) != LAB200_OK) return rc;
  return finish_call(la_generic_impl(a, bm, c, slopes, out, state_in, nullptr, workspace, workspace_bytes, bh, h, n, dk, dv, reverse, 0,
                         chunks, dtype, st, RESUME | RESUME_SWAPPED | (rebase ? 0 : RESUME_NO_REBASE)), workspace, st);
}

int lab200_la_combine_states(const float* gathered, const float* slopes, float* out, float* out_t, int ranks, int rank,
                             int bh, int h, int x, int y, long long shard_tokens, int reverse, void* stream) {
  if (!gathered || (!out && !out_t) || ranks < 1 || rank < 0 || rank >= ranks || bh < 1 || h < 1 || x < 1 || y < 1 ||
      shard_tokens < 0 || bh > 65535)
    return LAB200_ERR_SHAPE;
  if (!aligned16(gathered) || !aligned16(out) || !aligned16(out_t)) return LAB200_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  la_combine_kernel<<<dim3((y + 31) / 32, (x + 31) / 32, bh), dim3(32, 8), 0, st>>>(
      gathered, slopes, out, out_t, ranks, rank, bh, h, x, y, static_cast<float>(shard_tokens), reverse ? 1 : 0);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

int lab200_la_decode_step(const void* q, const void* k, const void* v, const float* slopes, float* state, void* o,
                          int bh, int h, int dk, int dv, int dtype, void* stream) {
  if (!q || !k || !v || !state || !o || bh < 1 || bh > 65535 || h < 1 || dk < 16 || dv < 1 || (dk % 16) != 0)
    return LAB200_ERR_SHAPE;
  if (dtype != LAB200_BF16 && dtype != LAB200_F16) return LAB200_ERR_DTYPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(state)) return LAB200_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((dv + 8 * LA_DECODE_ROWS - 1) / (8 * LA_DECODE_ROWS), bh);
  auto qq = static_cast<const uint16_t*>(q);
  auto kk = static_cast<const uint16_t*>(k);
  auto vv = static_cast<const uint16_t*>(v);
  auto oo = static_cast<uint16_t*>(o);
  if (dtype == LAB200_BF16) la_decode_kernel<1><<<grid, 256, 0, st>>>(qq, kk, vv, slopes, state, oo, h, dk, dv);
  else la_decode_kernel<0><<<grid, 256, 0, st>>>(qq, kk, vv, slopes, state, oo, h, dk, dv);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? LAB200_OK : LAB200_ERR_CUDA;
}

int lab200_la2_fwd(const void* q, const void* k, const void* v, const float* slopes, void* o, void* workspace,
                   size_t workspace_bytes, int b, int h, int n, int d, int e, int chunks, int dtype, void* stream) {
  if (b < 1 || h < 1 || b > 65535 / h) return LAB200_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = la_validate(q, k, v, o, nullptr, nullptr, workspace, b * h, h, n, d, e, 0, dtype);
  if (rc != LAB200_OK) return rc;
  if ((rc = reset_status(workspace, workspace_bytes, st)) != LAB200_OK) return rc;
  return finish_call(la_generic_impl(q, k, v, slopes, o, nullptr, nullptr, workspace, workspace_bytes, b * h, h, n, d, e, 0, 0,
                         chunks, dtype, st), workspace, st);
}

int lab200_la2_fwd_static(const void* q, const void* k, const void* v, const float* slopes, void* o, int b, int h,
                          int n, int d, int e, int chunks, int dtype, void* stream) {
  if (b < 1 || h < 1 || b > 65535 / h) return LAB200_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the scratch pointer is not known yet; validate everything else against a stand-in aligned address
  int rc = la_validate(q, k, v, o, nullptr, nullptr, reinterpret_cast<const void*>(uintptr_t{256}), b * h, h, n, d, e, 0,
                       dtype);
  if (rc != LAB200_OK) return rc;
  if (lab200_la_workspace_bytes(b * h, n, d, e, chunks) > static_cast<size_t>(LAB200_STATIC_SCRATCH_BYTES))
    return LAB200_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  if ((rc = static_scratch_address(&scratch)) != LAB200_OK) return rc;
  // the array keeps whatever the previous call left: the status word must start at zero; the chunk states
  // need no clearing because the state kernel writes every slot that the scan reads
  if ((rc = reset_status(scratch, LAB200_STATIC_SCRATCH_BYTES, st)) != LAB200_OK) return rc;
  return la_generic_impl(q, k, v, slopes, o, nullptr, nullptr, scratch, LAB200_STATIC_SCRATCH_BYTES, b * h, h, n, d, e,
                         0, 0, chunks, dtype, st);
}

static int la2_bwd_body(const void* q, const void* k, const void* v, const float* slopes, const void* dout, void* dq,
                   void* dk, void* dv, void* workspace, size_t workspace_bytes, int b, int h, int n, int d, int e,
                   int chunks, int dtype, void* stream) {
  if (b < 1 || h < 1 || b > 65535 / h) return LAB200_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int bh = b * h;
  int rc = la_validate(dout, v, k, dq, nullptr, nullptr, workspace, bh, h, n, e, d, 0, dtype);
  if (rc == LAB200_OK) rc = la_validate(k, q, dout, dv, nullptr, nullptr, workspace, bh, h, n, d, e, 0, dtype);
  if (rc == LAB200_OK && (!q || !dk || !aligned16(q) || !aligned16(dk))) rc = q && dk ? LAB200_ERR_ALIGN : LAB200_ERR_SHAPE;
  if (rc != LAB200_OK) return rc;
  if ((rc = reset_status(workspace, workspace_bytes, st)) != LAB200_OK) return rc;
  // dq_t = sum_{j<=t} lambda^(t-j) (do_t . v_j) k_j
  rc = la_generic_impl(dout, v, k, slopes, dq, nullptr, nullptr, workspace, workspace_bytes, bh, h, n, e, d, 0, 0,
                       chunks, dtype, st);
  if (rc != LAB200_OK) return rc;
  // dk_t = sum_{j>=t} lambda^(j-t) (v_t . do_j) q_j  and  dv_t = sum_{j>=t} lambda^(j-t) (k_t . q_j) do_j:
  // one fused reverse sweep (d, e <= 128), else two launches of the generic kernel
  if (use_fused_dkdv() && dkdv_shape_ok(d, e)) {
    rc = la_dkdv_full(q, k, v, dout, slopes, dk, dv, nullptr, workspace, workspace_bytes, bh, h, n, d, e, chunks, 0, dtype, st);
    if (rc != LAB200_ERR_SHAPE) return rc;
  }
  rc = la_generic_impl(v, dout, q, slopes, dk, nullptr, nullptr, workspace, workspace_bytes, bh, h, n, e, d, 1, 0,
                       chunks, dtype, st);
  if (rc != LAB200_OK) return rc;
  // In chunk mode the dk launch leaves the reverse-time state entering every chunk, sum lambda^t q_t^T do_t as (d, e), in
  // the workspace; dv needs the same states as (e, d). With d == e they are transposed in place instead of recomputed.
  const int resume = (d == e && chunk_count(bh, n, e, d, chunks) > 1) ? (RESUME | RESUME_SWAPPED | RESUME_NO_REBASE) : 0;
  return la_generic_impl(k, q, dout, slopes, dv, nullptr, nullptr, workspace, workspace_bytes, bh, h, n, d, e, 1, 0,
                         chunks, dtype, st, resume);
}

int lab200_la2_bwd(const void* q, const void* k, const void* v, const float* slopes, const void* dout, void* dq,
                   void* dk, void* dv, void* workspace, size_t workspace_bytes, int b, int h, int n, int d, int e,
                   int chunks, int dtype, void* stream) {
  return finish_call(la2_bwd_body(q, k, v, slopes, dout, dq, dk, dv, workspace, workspace_bytes, b, h, n, d, e, chunks, dtype,
                                  stream),
                     workspace, static_cast<cudaStream_t>(stream));
}

size_t lab200_la2_bwd_workspace_bytes(int b, int h, int n, int d, int e, int chunks) {
  if (b < 1 || h < 1) return WS_HEADER;
  // the three products inside lab200_la2_bwd run as (dk, dv) = (e, d) for dq and dk and (d, e) for dv; each plans its own chunks
  const size_t x = lab200_la_workspace_bytes(b * h, n, e, d, chunks), y = lab200_la_workspace_bytes(b * h, n, d, e, chunks);
  return x > y ? x : y;
}

int lab200_la2_dkdv(const void* q, const void* k, const void* v, const float* slopes, const void* dout, void* dk,
                    void* dv, const float* state_in, void* workspace, size_t workspace_bytes, int b, int h, int n, int d,
                    int e, int chunks, int resume, int dtype, void* stream) {
  if (b < 1 || h < 1 || b > 65535 / h || n < 1) return LAB200_ERR_SHAPE;
  const int dt = dtype & 0xff;
  if (dt != LAB200_BF16 && dt != LAB200_F16) return LAB200_ERR_DTYPE;
  if (!q || !k || !v || !dout || !dk || !dv) return LAB200_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(dout) || !aligned16(dk) || !aligned16(dv) ||
      !aligned16(workspace) || !aligned16(state_in))
    return LAB200_ERR_ALIGN;
  if (!dkdv_shape_ok(d, e)) return LAB200_ERR_SHAPE;
  if ((dtype & LAB200_LAYOUT_BNHD) && static_cast<long long>(b) * h * n >= (1LL << 31)) return LAB200_ERR_SHAPE;
  if (!reverse_chain_ok(1, state_in, n)) return LAB200_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = reset_status(workspace, workspace_bytes, st);
  if (rc != LAB200_OK) return rc;
  return finish_call(la_dkdv_full(q, k, v, dout, slopes, dk, dv, state_in, workspace, workspace_bytes, b * h, h, n, d, e, chunks,
                      resume, dtype, st), workspace, st);
}

int lab200_read_status(const void* workspace, void* stream) {
  if (!workspace) return -1;
  int v = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -2;
  if (cudaStreamSynchronize(st) != cudaSuccess) return -3;
  return v;
}

int lab200_last_status(void) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  StatusRing& ring = g_status_ring[dev];
  if (!ring.slots) return 0;
  for (int i = 0; i < STATUS_RING; ++i) {
    const int v = *const_cast<volatile int*>(ring.slots + i);
    if (v != 0) {
      ring.slots[i] = 0;
      return v;
    }
  }
  return 0;
}

int lab200_static_status(void* stream) {
  void* scratch = nullptr;
  if (static_scratch_address(&scratch) != LAB200_OK) return -1;
  return lab200_read_status(scratch, stream);
}

int lab200_debug_wait_expiry(void* workspace, size_t workspace_bytes, long long budget_cycles, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (budget_cycles < 1 || budget_cycles > 100000000LL) return LAB200_ERR_SHAPE;  // at most ~50 ms of SM clocks
  int rc = reset_status(workspace, workspace_bytes, st);
  if (rc != LAB200_OK) return rc;
  la_wait_expiry_kernel<<<1, 32, 0, st>>>(static_cast<int*>(workspace), budget_cycles);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (cudaGetLastError() != cudaSuccess) return LAB200_ERR_CUDA;
  post_status(workspace, st);
  return LAB200_OK;
}

int lab200_srmsnorm_fwd(const void* x, void* y, float* rstd, long long M, int N, float eps, int dtype, void* stream) {
  return srms_entry(true, x, nullptr, y, rstd, M, N, eps, dtype, static_cast<cudaStream_t>(stream));
}

int lab200_srmsnorm_bwd(const void* x, const void* dy, const float* rstd, void* dx, long long M, int N, int dtype,
                        void* stream) {
  return srms_entry(false, x, dy, dx, const_cast<float*>(rstd), M, N, 0.f, dtype, static_cast<cudaStream_t>(stream));
}

int lab200_srmsnorm_gate_fwd(const void* x, const void* gate, void* y, float* rstd, long long M, int N, float eps,
                             int dtype, void* stream) {
  return srms_gate_entry(true, x, gate, nullptr, y, nullptr, rstd, M, N, eps, dtype, static_cast<cudaStream_t>(stream));
}

int lab200_srmsnorm_gate_bwd(const void* x, const void* gate, const void* dy, const float* rstd, void* dx, void* dgate,
                             long long M, int N, int dtype, void* stream) {
  return srms_gate_entry(false, x, gate, dy, dx, dgate, const_cast<float*>(rstd), M, N, 0.f, dtype,
                         static_cast<cudaStream_t>(stream));
}

}  // extern "C"
