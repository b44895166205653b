// Row-wise kernels of the block's FFN branch: RMSNorm and the activation (GELU-tanh or SwiGLU), forward
// and backward.  With them the FFN branch is rematerialised in the backward pass (only the branch input
// is kept), as the reference does: block_ffn_residual, slinoss/ops/block/training.py:193-354, with the
// kernels of slinoss/ops/block/cute/norm.py:85,173 and activation.py:78,153.  The two GEMMs stay library
// calls in the caller.  All four kernels are HBM-bound: 16-byte accesses, one pass over their rows.
#include "common.cuh"

namespace sl {
namespace {

// out = x * rsqrt(mean(x^2) + eps) * w.  One warp per row; the row stays packed in registers (16-byte
// pieces, MAXP per lane), so it is read once.
template <typename T, int MAXP>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                          T* __restrict__ out, long long rows, int C, float eps) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int pieces = C / V;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
  uint4 raw[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pc = lane + 32 * i;
    if (pc < pieces) raw[i] = xr[pc];
  }
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    if (lane + 32 * i < pieces) {
      float v[V];
      unpack16<T>(raw[i], v);
#pragma unroll
      for (int k = 0; k < V; ++k) ss += v[k] * v[k];
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)C + eps);
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int pc = lane + 32 * i;
    if (pc < pieces) {
      float v[V], wv[V], o[V];
      unpack16<T>(raw[i], v);
      load16<T>(w + pc * V, wv);
#pragma unroll
      for (int k = 0; k < V; ++k) o[k] = v[k] * rstd * wv[k];
      store16<T>(out + row * C + pc * V, o);
    }
  }
}

// dx = rstd (g - xhat mean(g xhat)),  g = dy w,  xhat = x rstd;   dw += sum_rows dy xhat.
// A CTA walks its rows (grid-stride), one warp per row with x and dy packed in registers; every warp adds
// its rows' part of dw into a float row of its own in shared memory (plain 16-byte read-modify-writes: 128
// wavefronts per row against the ~280 cycles the row's bytes take at the SM's share of the HBM bandwidth),
// and the CTA sums the warps' rows and issues one global float atomic per channel at the end.  Keeping dw
// out of the registers leaves room for two CTAs per SM (shared-memory float atomics into one row were
// slower than this, and dw in registers allowed one CTA per SM).  The weight sits packed in shared memory.
template <typename T, int MAXP>
__global__ void __launch_bounds__(256, 2) rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                          const T* __restrict__ dy, T* __restrict__ dx,
                                                          float* __restrict__ dw, long long rows, int C, float eps) {
  constexpr int V = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char s_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float* s_dw = reinterpret_cast<float*>(s_raw);                        // [nw][C]
  uint4* s_w = reinterpret_cast<uint4*>(s_raw + (size_t)nw * C * sizeof(float));   // [C / V]
  float* my_dw = s_dw + (size_t)warp * C;
  const int pieces = C / V;
  for (int c = threadIdx.x; c < nw * C; c += blockDim.x) s_dw[c] = 0.f;
  for (int c = threadIdx.x; c < pieces; c += blockDim.x) s_w[c] = reinterpret_cast<const uint4*>(w)[c];
  __syncthreads();
  for (long long row = (long long)blockIdx.x * nw + warp; row < rows; row += (long long)gridDim.x * nw) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * C);
    uint4 xraw[MAXP], graw[MAXP];
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pc = lane + 32 * i;
      if (pc < pieces) { xraw[i] = xr[pc]; graw[i] = gr[pc]; }
    }
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pc = lane + 32 * i;
      if (pc < pieces) {
        float xv[V], gv[V], wv[V];
        unpack16<T>(xraw[i], xv); unpack16<T>(graw[i], gv); unpack16<T>(s_w[pc], wv);
#pragma unroll
        for (int k = 0; k < V; ++k) { ss += xv[k] * xv[k]; dot += gv[k] * wv[k] * xv[k]; }
      }
    }
    ss = warp_sum(ss); dot = warp_sum(dot);
    const float rstd = rsqrtf(ss / (float)C + eps);
    const float coef = dot * rstd * rstd / (float)C;     // mean(g xhat) rstd
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int pc = lane + 32 * i;
      if (pc < pieces) {
        float xv[V], gv[V], wv[V], o[V];
        unpack16<T>(xraw[i], xv); unpack16<T>(graw[i], gv); unpack16<T>(s_w[pc], wv);
#pragma unroll
        float4* acc = reinterpret_cast<float4*>(my_dw + pc * V);
#pragma unroll
        for (int q = 0; q < V / 4; ++q) {
          float4 a = acc[q];
          a.x += gv[4 * q] * (xv[4 * q] * rstd); a.y += gv[4 * q + 1] * (xv[4 * q + 1] * rstd);
          a.z += gv[4 * q + 2] * (xv[4 * q + 2] * rstd); a.w += gv[4 * q + 3] * (xv[4 * q + 3] * rstd);
          acc[q] = a;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] = rstd * (gv[k] * wv[k] - xv[k] * coef);
        store16<T>(dx + row * C + pc * V, o);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float v = 0.f;
    for (int q = 0; q < nw; ++q) v += s_dw[(size_t)q * C + c];
    atomicAdd(dw + c, v);
  }
}

// 16-bit rows take the one-instruction tanh (relative error 2^-11, below the rounding of the output);
// float32 rows the precise one.
template <bool FAST> __device__ __forceinline__ float tanh_io(float x) {
  if (FAST) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return tanhf(x);
}
template <bool FAST> __device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanh_io<FAST>(u));
}
template <bool FAST> __device__ __forceinline__ float dgelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanh_io<FAST>(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
}

// kind 0: hidden = gelu_tanh(projected) (same width).  kind 1 (SwiGLU): projected = [value | gate] of
// width 2 H per row, hidden = value * silu(gate).  One 16-byte piece of the hidden row per thread.
template <typename T>
__global__ void __launch_bounds__(256) ffn_act_fwd_kernel(const T* __restrict__ proj, T* __restrict__ hidden,
                                                          long long rows, int H, int kind) {
  constexpr int V = Vec16<T>::N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int ppr = H / V;
  if (i >= rows * ppr) return;
  const long long row = i / ppr;
  const int pc = (int)(i % ppr);
  float a[V], o[V];
  if (kind == 0) {
    load16<T>(proj + row * H + pc * V, a);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = gelu_tanh_f<sizeof(T) == 2>(a[k]);
  } else {
    float g[V];
    load16<T>(proj + row * 2 * H + pc * V, a);
    load16<T>(proj + row * 2 * H + H + pc * V, g);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = a[k] * silu_f(g[k]);
  }
  store16<T>(hidden + row * H + pc * V, o);
}

template <typename T>
__global__ void __launch_bounds__(256) ffn_act_bwd_kernel(const T* __restrict__ proj, const T* __restrict__ dhid,
                                                          T* __restrict__ dproj, long long rows, int H, int kind) {
  constexpr int V = Vec16<T>::N;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int ppr = H / V;
  if (i >= rows * ppr) return;
  const long long row = i / ppr;
  const int pc = (int)(i % ppr);
  float a[V], d[V], o[V];
  load16<T>(dhid + row * H + pc * V, d);
  if (kind == 0) {
    load16<T>(proj + row * H + pc * V, a);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = d[k] * dgelu_tanh_f<sizeof(T) == 2>(a[k]);
    store16<T>(dproj + row * H + pc * V, o);
  } else {
    float g[V], og[V];
    load16<T>(proj + row * 2 * H + pc * V, a);
    load16<T>(proj + row * 2 * H + H + pc * V, g);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float s = sigmoid_f(g[k]);
      o[k] = d[k] * g[k] * s;                                  // d value
      og[k] = d[k] * a[k] * (s + g[k] * s * (1.f - s));        // d gate
    }
    store16<T>(dproj + row * 2 * H + pc * V, o);
    store16<T>(dproj + row * 2 * H + H + pc * V, og);
  }
}

constexpr int RMS_MAXP_NARROW = 2;   // rows up to 512 (256) channels keep the registers low
constexpr int RMS_MAXP = 8;   // 16-byte pieces per lane: rows up to 8 * 32 * (4 or 8) channels

bool rows_ok(long long rows, int C, int dt, const void* a, const void* b) {
  const int V = dt == SL_F32 ? 4 : 8;
  return rows >= 1 && C >= V && C % V == 0 && C / V <= 32 * RMS_MAXP && aligned(a, 16) && aligned(b, 16);
}

}  // namespace
}  // namespace sl

extern "C" int sl_rmsnorm_fwd(const void* x, const void* weight, float eps, void* out, long long rows, int C,
                              int io_dtype, void* stream) {
  using namespace sl;
  if (!x || !weight || !out) return SL_ERR_NULL_POINTER;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  if (!rows_ok(rows, C, io_dtype, x, out) || !aligned(weight, 16)) return SL_ERR_BAD_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows + 7) / 8);
  const bool narrow = C / (io_dtype == SL_F32 ? 4 : 8) <= 32 * RMS_MAXP_NARROW;
  SL_DISPATCH_DTYPE(io_dtype, T, {
    auto kern = narrow ? rmsnorm_fwd_kernel<T, RMS_MAXP_NARROW> : rmsnorm_fwd_kernel<T, RMS_MAXP>;
    kern<<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(weight),
                               reinterpret_cast<T*>(out), rows, C, eps);
  });
  note_launches(1);
  return launch_status();
}

extern "C" int sl_rmsnorm_bwd(const void* x, const void* weight, float eps, const void* d_out, void* d_x,
                              float* d_weight, long long rows, int C, int io_dtype, void* stream) {
  using namespace sl;
  if (!x || !weight || !d_out || !d_x || !d_weight) return SL_ERR_NULL_POINTER;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  if (!rows_ok(rows, C, io_dtype, x, d_x) || !aligned(weight, 16) || !aligned(d_out, 16)) return SL_ERR_BAD_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long want = (rows + 7) / 8;
  const bool narrow = C / (io_dtype == SL_F32 ? 4 : 8) <= 32 * RMS_MAXP_NARROW;
  const long long cap = narrow ? 148 * 4 : 148 * 2;   // CTAs that walk the rows: all resident at once
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  const size_t smem = (size_t)8 * C * sizeof(float) + (size_t)C * dtype_size(io_dtype);   // 8 warps' dw rows + w
  SL_DISPATCH_DTYPE(io_dtype, T, {
    auto kern = narrow ? rmsnorm_bwd_kernel<T, RMS_MAXP_NARROW> : rmsnorm_bwd_kernel<T, RMS_MAXP>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return SL_ERR_LAUNCH_FAILED;
    kern<<<grid, 256, smem, st>>>(
        reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(weight), reinterpret_cast<const T*>(d_out),
        reinterpret_cast<T*>(d_x), d_weight, rows, C, eps);
  });
  note_launches(1);
  return launch_status();
}

extern "C" int sl_ffn_activation_fwd(const void* projected, void* hidden, long long rows, int hidden_dim,
                                     int kind, int io_dtype, void* stream) {
  using namespace sl;
  if (!projected || !hidden) return SL_ERR_NULL_POINTER;
  if (!dtype_ok(io_dtype) || (kind != 0 && kind != 1)) return SL_ERR_UNSUPPORTED;
  const int V = io_dtype == SL_F32 ? 4 : 8;
  if (rows < 1 || hidden_dim < V || hidden_dim % V || !aligned(projected, 16) || !aligned(hidden, 16))
    return SL_ERR_BAD_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long n = rows * (hidden_dim / V);
  SL_DISPATCH_DTYPE(io_dtype, T, {
    ffn_act_fwd_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const T*>(projected), reinterpret_cast<T*>(hidden), rows, hidden_dim, kind);
  });
  note_launches(1);
  return launch_status();
}

extern "C" int sl_ffn_activation_bwd(const void* projected, const void* d_hidden, void* d_projected,
                                     long long rows, int hidden_dim, int kind, int io_dtype, void* stream) {
  using namespace sl;
  if (!projected || !d_hidden || !d_projected) return SL_ERR_NULL_POINTER;
  if (!dtype_ok(io_dtype) || (kind != 0 && kind != 1)) return SL_ERR_UNSUPPORTED;
  const int V = io_dtype == SL_F32 ? 4 : 8;
  if (rows < 1 || hidden_dim < V || hidden_dim % V || !aligned(projected, 16) || !aligned(d_hidden, 16) ||
      !aligned(d_projected, 16))
    return SL_ERR_BAD_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long n = rows * (hidden_dim / V);
  SL_DISPATCH_DTYPE(io_dtype, T, {
    ffn_act_bwd_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const T*>(projected), reinterpret_cast<const T*>(d_hidden),
        reinterpret_cast<T*>(d_projected), rows, hidden_dim, kind);
  });
  note_launches(1);
  return launch_status();
}
