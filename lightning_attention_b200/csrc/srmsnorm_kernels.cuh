// SimpleRMSNorm (no learnable weight) forward and backward for sm_100a.
//
//   forward : rstd = 1 / sqrt(mean(x^2) + eps);  y = x * rstd            (reference: srmsnorm.py:12-33)
//   backward: xhat = x * rstd; c = mean(xhat * dy); dx = (dy - xhat * c) * rstd   (srmsnorm.py:38-74)
//
// Both are pure streaming kernels (4 and 6 bytes per bf16 element). A row is owned by a group of G
// threads; every thread keeps its part of the row in registers as 128-bit vectors, so each element
// is read from HBM exactly once. Sums are fp32: warp shuffles first, then (G > 32) a few words of
// shared memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lab200 {

constexpr int SRMS_MAX_VPT = 8;  // most 128-bit vectors a thread may hold

enum SrmsDtype : int { SRMS_F32 = 0, SRMS_F16 = 1, SRMS_BF16 = 2 };

template <int DT> struct SrmsVec;
template <> struct SrmsVec<SRMS_F32> {
  static constexpr int EPV = 4;
  __device__ static void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  __device__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <> struct SrmsVec<SRMS_F16> {
  static constexpr int EPV = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct SrmsVec<SRMS_BF16> {
  static constexpr int EPV = 8;
  __device__ static void unpack(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&t);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// A thread's unit of global access: W = 1 is one 128-bit vector, W = 2 one 256-bit access (sm_100: ld/st .v8.b32). The
// 256-bit forms also take an L2 eviction hint: every input is read exactly once and no output is read again, so all of them
// are marked evict-first and do not push each other's still-unread sectors out of L2 (measured on 32768 x 4096 bf16 rows:
// backward 5.8 -> 6.8 TB/s). W = 2 needs rows that are a multiple of two vectors and 32-byte aligned pointers.
template <int W> struct SrmsPack { uint4 q[W]; };

template <int W>
__device__ __forceinline__ SrmsPack<W> ld_stream(const SrmsPack<W>* p) {
  SrmsPack<W> v;
  if constexpr (W == 2) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.q[0].x), "=r"(v.q[0].y), "=r"(v.q[0].z), "=r"(v.q[0].w), "=r"(v.q[1].x), "=r"(v.q[1].y), "=r"(v.q[1].z), "=r"(v.q[1].w)
                 : "l"(p));
  } else {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.q[0].x), "=r"(v.q[0].y), "=r"(v.q[0].z), "=r"(v.q[0].w)
                 : "l"(p));
  }
  return v;
}
template <int W>
__device__ __forceinline__ void st_stream(SrmsPack<W>* p, const SrmsPack<W>& v) {
  if constexpr (W == 2) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.u32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v.q[0].x),
                 "r"(v.q[0].y), "r"(v.q[0].z), "r"(v.q[0].w), "r"(v.q[1].x), "r"(v.q[1].y), "r"(v.q[1].z), "r"(v.q[1].w) : "memory");
  } else {
    asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.q[0].x), "r"(v.q[0].y), "r"(v.q[0].z), "r"(v.q[0].w) : "memory");
  }
}

// Sum over the G threads that own one row. `slot` is this row group's scratch in shared memory.
template <int G>
__device__ __forceinline__ float group_sum(float v, float* slot, int tig) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if constexpr (G > 32) {
    constexpr int NW = G / 32;
    if ((tig & 31) == 0) slot[tig >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) t += slot[w];
    __syncthreads();  // slot is reused by the next reduction
    v = t;
  }
  return v;
}

// Row bookkeeping shared by the four kernels: G threads per row holding VPT packs each; CTA = max(G, 256) threads =>
// CTA / G rows per CTA. Whole groups are (in)active together; inactive ones still reach the barriers.
template <int DT, int G, int W>
struct SrmsRow {
  using V = SrmsVec<DT>;
  static constexpr int CTA = (G > 256 ? G : 256);
  static constexpr int RPC = CTA / G;
  static constexpr int EPP = W * V::EPV;  // elements per pack
  int grp, tig, npack;
  long long row;
  bool active;
  size_t off;
  __device__ SrmsRow(int M, int N) {
    grp = threadIdx.x / G; tig = threadIdx.x % G;
    row = static_cast<long long>(blockIdx.x) * RPC + grp;
    active = row < M;
    npack = N / EPP;
    off = static_cast<size_t>(active ? row : 0) * npack;
  }
};

template <int DT, int G, int VPT, int W>
__global__ void __launch_bounds__((G > 256 ? G : 256))
srmsnorm_fwd_kernel(const void* __restrict__ x_, void* __restrict__ y_, float* __restrict__ rstd_, int M, int N, float eps) {
  using R = SrmsRow<DT, G, W>; using V = SrmsVec<DT>; using P = SrmsPack<W>;
  __shared__ float red[R::RPC][16];
  const R r(M, N);
  const P* x = reinterpret_cast<const P*>(x_) + r.off;
  P* y = reinterpret_cast<P*>(y_) + r.off;

  P xv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) xv[i] = ld_stream<W>(x + v);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float f[V::EPV];
        V::unpack(xv[i].q[w], f);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
  }
  ss = group_sum<G>(ss, red[r.grp], r.tig);
  const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
  if (r.active && r.tig == 0) rstd_[r.row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      P o;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float f[V::EPV];
        V::unpack(xv[i].q[w], f);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) f[j] *= rstd;
        o.q[w] = V::pack(f);
      }
      st_stream<W>(y + v, o);
    }
  }
}

template <int DT, int G, int VPT, int W>
__global__ void __launch_bounds__((G > 256 ? G : 256))
srmsnorm_bwd_kernel(const void* __restrict__ x_, const void* __restrict__ dy_, const float* __restrict__ rstd_,
                    void* __restrict__ dx_, int M, int N) {
  using R = SrmsRow<DT, G, W>; using V = SrmsVec<DT>; using P = SrmsPack<W>;
  __shared__ float red[R::RPC][16];
  const R r(M, N);
  const P* x = reinterpret_cast<const P*>(x_) + r.off;
  const P* dy = reinterpret_cast<const P*>(dy_) + r.off;
  P* dx = reinterpret_cast<P*>(dx_) + r.off;
  const float rstd = r.active ? rstd_[r.row] : 0.f;

  P xv[VPT], gv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      xv[i] = ld_stream<W>(x + v);
      gv[i] = ld_stream<W>(dy + v);
    }
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float fx[V::EPV], fg[V::EPV];
        V::unpack(xv[i].q[w], fx);
        V::unpack(gv[i].q[w], fg);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) dot = fmaf(fx[j] * rstd, fg[j], dot);
      }
    }
  }
  dot = group_sum<G>(dot, red[r.grp], r.tig);
  const float c = dot / static_cast<float>(N);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      P o;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float fx[V::EPV], fg[V::EPV];
        V::unpack(xv[i].q[w], fx);
        V::unpack(gv[i].q[w], fg);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) fg[j] = (fg[j] - fx[j] * rstd * c) * rstd;
        o.q[w] = V::pack(fg);
      }
      st_stream<W>(dx + v, o);
    }
  }
}

// Gated form used by callers that multiply the normalised output by a sigmoid gate (examples/module/tnl_attn.py:66-69):
//   forward : y = x * rstd * sigmoid(g)                                              6 bytes per 16-bit element
//   backward: sg = sigmoid(g); xhat = x * rstd; t = dy * sg; c = mean(xhat * t);
//             dx = (t - xhat * c) * rstd;  dg = dy * xhat * sg * (1 - sg)           10 bytes per element
// One pass each instead of norm + sigmoid + multiply as three kernels (14 and 26 bytes per element).
__device__ __forceinline__ float sigmoidf_fast(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }

template <int DT, int G, int VPT, int W>
__global__ void __launch_bounds__((G > 256 ? G : 256))
srmsnorm_gate_fwd_kernel(const void* __restrict__ x_, const void* __restrict__ g_, void* __restrict__ y_,
                         float* __restrict__ rstd_, int M, int N, float eps) {
  using R = SrmsRow<DT, G, W>; using V = SrmsVec<DT>; using P = SrmsPack<W>;
  __shared__ float red[R::RPC][16];
  const R r(M, N);
  const P* x = reinterpret_cast<const P*>(x_) + r.off;
  const P* g = reinterpret_cast<const P*>(g_) + r.off;
  P* y = reinterpret_cast<P*>(y_) + r.off;

  P xv[VPT], gv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      xv[i] = ld_stream<W>(x + v);
      gv[i] = ld_stream<W>(g + v);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float f[V::EPV];
        V::unpack(xv[i].q[w], f);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
  }
  ss = group_sum<G>(ss, red[r.grp], r.tig);
  const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
  if (r.active && r.tig == 0) rstd_[r.row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      P o;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float f[V::EPV], fg[V::EPV];
        V::unpack(xv[i].q[w], f);
        V::unpack(gv[i].q[w], fg);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) f[j] = f[j] * rstd * sigmoidf_fast(fg[j]);
        o.q[w] = V::pack(f);
      }
      st_stream<W>(y + v, o);
    }
  }
}

template <int DT, int G, int VPT, int W>
__global__ void __launch_bounds__((G > 256 ? G : 256))
srmsnorm_gate_bwd_kernel(const void* __restrict__ x_, const void* __restrict__ g_, const void* __restrict__ dy_,
                         const float* __restrict__ rstd_, void* __restrict__ dx_, void* __restrict__ dg_, int M, int N) {
  using R = SrmsRow<DT, G, W>; using V = SrmsVec<DT>; using P = SrmsPack<W>;
  __shared__ float red[R::RPC][16];
  const R r(M, N);
  const P* x = reinterpret_cast<const P*>(x_) + r.off;
  const P* g = reinterpret_cast<const P*>(g_) + r.off;
  const P* dy = reinterpret_cast<const P*>(dy_) + r.off;
  P* dx = reinterpret_cast<P*>(dx_) + r.off;
  P* dg = reinterpret_cast<P*>(dg_) + r.off;
  const float rstd = r.active ? rstd_[r.row] : 0.f;

  P xv[VPT], gv[VPT], dv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      xv[i] = ld_stream<W>(x + v);
      gv[i] = ld_stream<W>(g + v);
      dv[i] = ld_stream<W>(dy + v);
    }
  }
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float fx[V::EPV], fg[V::EPV], fd[V::EPV];
        V::unpack(xv[i].q[w], fx);
        V::unpack(gv[i].q[w], fg);
        V::unpack(dv[i].q[w], fd);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) dot = fmaf(fx[j] * rstd, fd[j] * sigmoidf_fast(fg[j]), dot);
      }
    }
  }
  dot = group_sum<G>(dot, red[r.grp], r.tig);
  const float c = dot / static_cast<float>(N);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = r.tig + i * G;
    if (r.active && v < r.npack) {
      P ox, og;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        float fx[V::EPV], fg[V::EPV], fd[V::EPV];
        V::unpack(xv[i].q[w], fx);
        V::unpack(gv[i].q[w], fg);
        V::unpack(dv[i].q[w], fd);
#pragma unroll
        for (int j = 0; j < V::EPV; ++j) {
          const float sg = sigmoidf_fast(fg[j]);
          const float xh = fx[j] * rstd;
          const float t = fd[j] * sg;
          fg[j] = fd[j] * xh * sg * (1.0f - sg);  // dg
          fx[j] = (t - xh * c) * rstd;            // dx
        }
        ox.q[w] = V::pack(fx);
        og.q[w] = V::pack(fg);
      }
      st_stream<W>(dx + v, ox);
      st_stream<W>(dg + v, og);
    }
  }
}

// Fallback for rows whose length or base address does not allow 128-bit vectors: one 256-thread
// CTA per row, element-wise loads, the row is read twice (the second read normally hits L2).
template <int DT> struct SrmsElem;
template <> struct SrmsElem<SRMS_F32> { using T = float;
  __device__ static float ld(const T* p) { return *p; } __device__ static void st(T* p, float v) { *p = v; } };
template <> struct SrmsElem<SRMS_F16> { using T = __half;
  __device__ static float ld(const T* p) { return __half2float(*p); } __device__ static void st(T* p, float v) { *p = __float2half_rn(v); } };
template <> struct SrmsElem<SRMS_BF16> { using T = __nv_bfloat16;
  __device__ static float ld(const T* p) { return __bfloat162float(*p); } __device__ static void st(T* p, float v) { *p = __float2bfloat16_rn(v); } };

template <int DT>
__global__ void __launch_bounds__(256)
srmsnorm_fwd_generic_kernel(const void* __restrict__ x_, void* __restrict__ y_, float* __restrict__ rstd_, int M, int N, float eps) {
  using E = SrmsElem<DT>;
  __shared__ float red[1][16];
  const size_t off = static_cast<size_t>(blockIdx.x) * N;
  const typename E::T* x = static_cast<const typename E::T*>(x_) + off;
  typename E::T* y = static_cast<typename E::T*>(y_) + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < N; i += 256) { const float f = E::ld(x + i); ss = fmaf(f, f, ss); }
  ss = group_sum<256>(ss, red[0], threadIdx.x);
  const float rstd = 1.0f / sqrtf(ss / static_cast<float>(N) + eps);
  if (threadIdx.x == 0) rstd_[blockIdx.x] = rstd;
  for (int i = threadIdx.x; i < N; i += 256) E::st(y + i, E::ld(x + i) * rstd);
}

template <int DT>
__global__ void __launch_bounds__(256)
srmsnorm_bwd_generic_kernel(const void* __restrict__ x_, const void* __restrict__ dy_, const float* __restrict__ rstd_,
                            void* __restrict__ dx_, int M, int N) {
  using E = SrmsElem<DT>;
  __shared__ float red[1][16];
  const size_t off = static_cast<size_t>(blockIdx.x) * N;
  const typename E::T* x = static_cast<const typename E::T*>(x_) + off;
  const typename E::T* dy = static_cast<const typename E::T*>(dy_) + off;
  typename E::T* dx = static_cast<typename E::T*>(dx_) + off;
  const float rstd = rstd_[blockIdx.x];
  float dot = 0.f;
  for (int i = threadIdx.x; i < N; i += 256) dot = fmaf(E::ld(x + i) * rstd, E::ld(dy + i), dot);
  dot = group_sum<256>(dot, red[0], threadIdx.x);
  const float c = dot / static_cast<float>(N);
  for (int i = threadIdx.x; i < N; i += 256) E::st(dx + i, (E::ld(dy + i) - E::ld(x + i) * rstd * c) * rstd);
}

}  // namespace lab200
