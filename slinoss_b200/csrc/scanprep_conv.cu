// Scan preparation fused with the causal depthwise conv1d + SiLU of the value stream.
//
// Forward (one C-ABI call, three coalesced elementwise kernels on one stream):
//   value kernel  out[b,t,c] = SiLU(bias_c + sum_j W[c,j] x[b,t-(d_conv-1)+j,c]) written
//                 straight into the (batch,heads,T,P) layout of U
//                 (reference: slinoss/ops/mixer/convolution.py:68-101 followed by the
//                 transpose of slinoss/layers/scanprep.py:307-321)
//   bc kernel     amplitude = softplus, phase = pi*tanh, pair = amp*(cos,sin)/rms_n(amp)
//                 (slinoss/ops/scanprep/parameterization.py:45-107)
//   coeff kernel  dt/alpha/theta maps, rho = r e^{i theta}, exact first-order-hold taps
//                 (slinoss/layers/scanprep.py:237-283, slinoss/ops/scanprep/reference.py:25-56)
// The tap formulas cancel catastrophically in float32 for small |z| (the
// numerator of kappa2 loses ~1/|z|^2 ulps), so the coefficient kernels evaluate them
// in float64; the count is one complex per (batch, head, token), which is negligible.
//
// Backward mirrors the three kernels; parameter-bias and conv weight/bias
// gradients are reduced per CTA and accumulated with float atomics.
#include <type_traits>

#include <mutex>

#include "common.cuh"

namespace sl {
namespace {

#include "scanprep_math.cuh"

constexpr int CONV_TT = 32;  // tokens per CTA in the value kernels

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  } else {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const float2 a = unpack_pair<T>(r.x), b = unpack_pair<T>(r.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_pair<T>(v[0], v[1]), pack_pair<T>(v[2], v[3]));
  }
}

struct ValueParams {
  const void *x, *w, *bias, *state_in;
  void *state_out, *U;
  int64_t xs;                   // row stride of x (elements)
  int64_t usb, ush, ust;        // strides of U
  int batch, T, C, P, W;
};

template <typename T>
__device__ __forceinline__ float load_x(const ValueParams& p, const T* x, const T* st, int b,
                                        int t, int c) {
  // input at time t (t may be negative: carried conv state or zero)
  if (t >= 0) return to_f32(x[((size_t)b * p.T + t) * p.xs + c]);
  const int j = p.W - 1 + t;
  if (st && j >= 0) return to_f32(st[((size_t)b * p.C + c) * (p.W - 1) + j]);
  return 0.f;
}

template <typename T>
__global__ void __launch_bounds__(256) value_fwd_kernel(ValueParams p) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
  if (c >= p.C) return;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* st = reinterpret_cast<const T*>(p.state_in);
  T* U = reinterpret_cast<T*>(p.U);
  const int h = c / p.P, pp = c - h * p.P;
  const int t1 = min(t0 + CONV_TT, p.T);
  if (!p.w) {
    for (int t = t0; t < t1; ++t)
      U[(size_t)b * p.usb + (size_t)h * p.ush + (size_t)t * p.ust + pp] =
          x[((size_t)b * p.T + t) * p.xs + c];
    return;
  }
  const T* w = reinterpret_cast<const T*>(p.w);
  float wj[4] = {0.f, 0.f, 0.f, 0.f}, win[4] = {0.f, 0.f, 0.f, 0.f};
  // right-align the taps in a width-4 window: wj[4-W+j] = W[c][j]
  for (int j = 0; j < p.W; ++j) wj[4 - p.W + j] = to_f32(w[(size_t)c * p.W + j]);
  const float bias = p.bias ? to_f32(reinterpret_cast<const T*>(p.bias)[c]) : 0.f;
  // win[k] holds x at time t-3+k
  for (int k = 1; k < 4; ++k) win[k] = (4 - k <= p.W - 1) ? load_x(p, x, st, b, t0 - 4 + k, c) : 0.f;
  for (int t = t0; t < t1; ++t) {
    win[0] = win[1]; win[1] = win[2]; win[2] = win[3];
    win[3] = to_f32(x[((size_t)b * p.T + t) * p.xs + c]);
    const float a = bias + wj[0] * win[0] + wj[1] * win[1] + wj[2] * win[2] + wj[3] * win[3];
    U[(size_t)b * p.usb + (size_t)h * p.ush + (size_t)t * p.ust + pp] = from_f32<T>(silu_f(a));
  }
  if (p.state_out && t1 == p.T) {
    T* so = reinterpret_cast<T*>(p.state_out);
    for (int j = 0; j < p.W - 1; ++j)
      so[((size_t)b * p.C + c) * (p.W - 1) + j] =
          from_f32<T>(load_x(p, x, st, b, p.T - (p.W - 1) + j, c));
  }
}

struct ValueBwdParams {
  ValueParams f;
  const void* dU;
  void *dx, *dstate;
  float *dw, *dbias;
};

__device__ __forceinline__ float dsilu_f(float a) {
  const float s = sigmoid_f(a);
  return s * (1.f + a * (1.f - s));
}

// One thread per channel walks CONV_TT tokens; da at tokens t..t+W-1 is needed
// for dx[t], so da is recomputed over a (W-1)-token look-ahead halo.
template <typename T>
__global__ void __launch_bounds__(256) value_bwd_kernel(ValueBwdParams q) {
  const ValueParams& p = q.f;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.y * CONV_TT, b = blockIdx.z;
  if (c >= p.C) return;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* st = reinterpret_cast<const T*>(p.state_in);
  const T* dU = reinterpret_cast<const T*>(q.dU);
  T* dx = reinterpret_cast<T*>(q.dx);
  const int h = c / p.P, pp = c - h * p.P;
  const int t1 = min(t0 + CONV_TT, p.T);
  auto dy_at = [&](int t) -> float {
    return to_f32(dU[(size_t)b * p.usb + (size_t)h * p.ush + (size_t)t * p.ust + pp]);
  };
  if (!p.w) {
    for (int t = t0; t < t1; ++t) dx[((size_t)b * p.T + t) * p.C + c] = from_f32<T>(dy_at(t));
    return;
  }
  const T* w = reinterpret_cast<const T*>(p.w);
  const int W = p.W;
  float wj[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < W; ++j) wj[4 - W + j] = to_f32(w[(size_t)c * W + j]);
  const float bias = p.bias ? to_f32(reinterpret_cast<const T*>(p.bias)[c]) : 0.f;
  float win[4] = {0.f, 0.f, 0.f, 0.f};   // x at times s-3..s for the da being formed
  float da[4] = {0.f, 0.f, 0.f, 0.f};    // da at times s-3..s
  float dwacc[4] = {0.f, 0.f, 0.f, 0.f}, dbacc = 0.f;
  // The first tile also owns the gradient of the carried conv state (times < 0).
  const int s_begin = (t0 == 0) ? 0 : t0;
  for (int k = 1; k < 4; ++k) win[k] = (4 - k <= W - 1) ? load_x(p, x, st, b, s_begin - 4 + k, c) : 0.f;
  // s runs over the tokens whose da is formed; dx[s-3] becomes complete at step s
  // when W == 4 (in general dx[t] needs da[t .. t+W-1]).
  const int s_end = min(t1 + 3, p.T + 3);
  for (int s = s_begin; s < s_end; ++s) {
    win[0] = win[1]; win[1] = win[2]; win[2] = win[3];
    da[0] = da[1]; da[1] = da[2]; da[2] = da[3];
    float d = 0.f;
    if (s < p.T) {
      win[3] = to_f32(x[((size_t)b * p.T + s) * p.xs + c]);
      const float a = bias + wj[0] * win[0] + wj[1] * win[1] + wj[2] * win[2] + wj[3] * win[3];
      d = dy_at(s) * dsilu_f(a);
      if (s >= t0 && s < t1) {  // each token's weight/bias contribution is counted once
        dwacc[0] += d * win[0]; dwacc[1] += d * win[1];
        dwacc[2] += d * win[2]; dwacc[3] += d * win[3];
        dbacc += d;
      }
    } else {
      win[3] = 0.f;
    }
    da[3] = d;
    // dx[t] = sum_k wj[k] * da[t + 3 - k], complete for t = s - 3
    const int t = s - 3;
    const float g = wj[3] * da[0] + wj[2] * da[1] + wj[1] * da[2] + wj[0] * da[3];
    if (t >= t0 && t < t1) dx[((size_t)b * p.T + t) * p.C + c] = from_f32<T>(g);
    else if (t < 0 && t0 == 0 && q.dstate && t >= -(W - 1))
      reinterpret_cast<T*>(q.dstate)[((size_t)b * p.C + c) * (W - 1) + (W - 1 + t)] = from_f32<T>(g);
  }
  for (int j = 0; j < W; ++j) atomicAdd(q.dw + (size_t)c * W + j, dwacc[4 - W + j]);
  if (q.dbias) atomicAdd(q.dbias + c, dbacc);
}

// ---- vector path of the value kernels ----------------------------------------------------------------
// A thread owns 4 consecutive channels (one 8- or 16-byte access per token) and walks CONV_TT
// tokens; a warp covers 128 consecutive channels, a CTA of 256 threads 8 token sub-tiles of the
// same 128 channels, so that the conv weight / bias gradients of the 8 sub-tiles are combined in
// shared memory and added to the float32 accumulators once per CTA.
// Needs P % 4 == 0 (a piece stays inside one head), strides that are multiples of 4 and aligned
// pointers; anything else takes the one-channel-per-thread kernels above.
constexpr int CONV_V = 4;
constexpr int CONV_SUB = 8;   // token sub-tiles per CTA

template <typename T>
__device__ __forceinline__ void load_xv(const ValueParams& p, const T* x, const T* st, int b, int t, int c,
                                        float (&v)[CONV_V]) {
  if (t >= 0) { load4<T>(x + ((size_t)b * p.T + t) * p.xs + c, v); return; }
  const int j = p.W - 1 + t;
#pragma unroll
  for (int k = 0; k < CONV_V; ++k)
    v[k] = (st && j >= 0) ? to_f32(st[((size_t)b * p.C + c + k) * (p.W - 1) + j]) : 0.f;
}

template <typename T, int V> __device__ __forceinline__ void loadv(const T* p, float (&v)[V]) {
  if constexpr (V == 4) load4<T>(p, v); else load16<T>(p, v);
}
template <typename T, int V> __device__ __forceinline__ void storev(T* p, const float (&v)[V]) {
  if constexpr (V == 4) store4<T>(p, v); else store16<T>(p, v);
}

// Forward (instantiated with V = CONV_V channels per thread).
template <typename T, int V>
__global__ void __launch_bounds__(256, 3) value_fwd_vec_kernel(ValueParams p) {
  const int c = (blockIdx.x * 32 + (threadIdx.x & 31)) * V;
  const int t0 = (blockIdx.y * CONV_SUB + (threadIdx.x >> 5)) * CONV_TT, b = blockIdx.z;
  if (c >= p.C || t0 >= p.T) return;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* st = reinterpret_cast<const T*>(p.state_in);
  T* U = reinterpret_cast<T*>(p.U);
  const int h = c / p.P, pp = c - h * p.P;
  T* Ub = U + (size_t)b * p.usb + (size_t)h * p.ush + pp;
  const T* xb = x + (size_t)b * p.T * p.xs + c;
  const int t1 = min(t0 + CONV_TT, p.T);
  if (!p.w) {
    for (int t = t0; t < t1; ++t) {
      float v[V];
      loadv<T, V>(xb + (size_t)t * p.xs, v);
      storev<T, V>(Ub + (size_t)t * p.ust, v);
    }
    return;
  }
  const T* w = reinterpret_cast<const T*>(p.w);
  float wj[4][V], win[4][V], bias[V];
  auto x_at = [&](int t, int k) -> float {   // scalar access for the halo (t may be negative)
    if (t >= 0) return to_f32(xb[(size_t)t * p.xs + k]);
    const int j = p.W - 1 + t;
    return (st && j >= 0) ? to_f32(st[((size_t)b * p.C + c + k) * (p.W - 1) + j]) : 0.f;
  };
  if (p.W == 4 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
    // taps of V channels are 4 V contiguous values; bias and the three halo rows are one piece each
    float wf[4 * V];
#pragma unroll
    for (int i = 0; i < 4 * V / Vec16<T>::N; ++i) {
      float q[Vec16<T>::N];
      load16<T>(w + (size_t)c * 4 + i * Vec16<T>::N, q);
#pragma unroll
      for (int e = 0; e < Vec16<T>::N; ++e) wf[i * Vec16<T>::N + e] = q[e];
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) wj[j][k] = wf[4 * k + j];
      bias[k] = 0.f; win[0][k] = 0.f;
    }
    if (p.bias) loadv<T, V>(reinterpret_cast<const T*>(p.bias) + c, bias);
#pragma unroll
    for (int q = 1; q < 4; ++q) {
      const int t = t0 - 4 + q;
      if (t >= 0) loadv<T, V>(xb + (size_t)t * p.xs, win[q]);
      else {
#pragma unroll
        for (int k = 0; k < V; ++k) win[q][k] = x_at(t, k);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < V; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j)   // right-aligned taps; static indices keep wj in registers
        wj[j][k] = (j >= 4 - p.W) ? to_f32(w[(size_t)(c + k) * p.W + (j - (4 - p.W))]) : 0.f;
      bias[k] = p.bias ? to_f32(reinterpret_cast<const T*>(p.bias)[c + k]) : 0.f;
      win[0][k] = 0.f;
#pragma unroll
      for (int q = 1; q < 4; ++q) win[q][k] = (4 - q <= p.W - 1) ? x_at(t0 - 4 + q, k) : 0.f;
    }
  }
  auto step = [&](int t, const float (&xin)[V]) {
    float o[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      win[0][k] = win[1][k]; win[1][k] = win[2][k]; win[2][k] = win[3][k]; win[3][k] = xin[k];
      const float a = bias[k] + wj[0][k] * win[0][k] + wj[1][k] * win[1][k] + wj[2][k] * win[2][k] +
                      wj[3][k] * win[3][k];
      o[k] = silu_f(a);
    }
    storev<T, V>(Ub + (size_t)t * p.ust, o);
  };
  if (t1 - t0 == CONV_TT) {
    // full tile: batches of 8 tokens whose loads are all issued (unconditionally) before the first
    // store of the batch - the compiler cannot move loads of x over stores to U by itself
    constexpr int TB = 8;
    using Raw = typename std::conditional<V * sizeof(T) == 16, uint4, uint2>::type;
#pragma unroll 1
    for (int tb = t0; tb < t1; tb += TB) {
      Raw raw[TB];
#pragma unroll
      for (int i = 0; i < TB; ++i) raw[i] = *reinterpret_cast<const Raw*>(xb + (size_t)(tb + i) * p.xs);
#pragma unroll
      for (int i = 0; i < TB; ++i) {
        float xin[V];
        const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
        for (int k = 0; k < V; ++k) xin[k] = to_f32(e[k]);
        step(tb + i, xin);
      }
    }
  } else {
    for (int t = t0; t < t1; ++t) {
      float xin[V];
      loadv<T, V>(xb + (size_t)t * p.xs, xin);
      step(t, xin);
    }
  }
  if (p.state_out && t1 == p.T) {
    T* so = reinterpret_cast<T*>(p.state_out);
    for (int j = 0; j < p.W - 1; ++j) {
#pragma unroll
      for (int k = 0; k < V; ++k)
        so[((size_t)b * p.C + c + k) * (p.W - 1) + j] = from_f32<T>(x_at(p.T - (p.W - 1) + j, k));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256, 2) value_bwd_vec_kernel(ValueBwdParams q) {
  const ValueParams& p = q.f;
  __shared__ float s_acc[CONV_SUB][5][32 * CONV_V];   // dw (4 taps) and dbias partials per sub-tile
  const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * CONV_V;
  const int t0 = (blockIdx.y * CONV_SUB + sub) * CONV_TT, b = blockIdx.z;
  const bool live = c < p.C && t0 < p.T;
  float dwacc[4][CONV_V], dbacc[CONV_V];
#pragma unroll
  for (int k = 0; k < CONV_V; ++k) {
    dbacc[k] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) dwacc[j][k] = 0.f;
  }
  if (live) {
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* st = reinterpret_cast<const T*>(p.state_in);
    const T* dU = reinterpret_cast<const T*>(q.dU);
    T* dx = reinterpret_cast<T*>(q.dx);
    const int h = c / p.P, pp = c - h * p.P;
    const T* dUb = dU + (size_t)b * p.usb + (size_t)h * p.ush + pp;
    const int t1 = min(t0 + CONV_TT, p.T);
    if (!p.w) {
      for (int t = t0; t < t1; ++t) {
        float v[CONV_V];
        load4<T>(dUb + (size_t)t * p.ust, v);
        store4<T>(dx + ((size_t)b * p.T + t) * p.C + c, v);
      }
    } else {
      const T* w = reinterpret_cast<const T*>(p.w);
      const int W = p.W;
      float wj[4][CONV_V], win[4][CONV_V], da[4][CONV_V], bias[CONV_V];
      const int s_begin = t0;   // the first tile also owns the gradient of the carried conv state
#pragma unroll
      for (int k = 0; k < CONV_V; ++k) {
#pragma unroll
        for (int j = 0; j < 4; ++j) da[j][k] = 0.f;
        win[0][k] = 0.f; bias[k] = 0.f;
      }
      if (W == 4 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
        // the taps of the 4 channels are 16 contiguous values; bias is one 4-wide piece
#pragma unroll
        for (int k = 0; k < CONV_V; ++k) {
          float q4[4];
          load4<T>(w + (size_t)(c + k) * 4, q4);
#pragma unroll
          for (int j = 0; j < 4; ++j) wj[j][k] = q4[j];
        }
        if (p.bias) load4<T>(reinterpret_cast<const T*>(p.bias) + c, bias);
      } else {
#pragma unroll
        for (int k = 0; k < CONV_V; ++k) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            wj[j][k] = (j >= 4 - W) ? to_f32(w[(size_t)(c + k) * W + (j - (4 - W))]) : 0.f;
          bias[k] = p.bias ? to_f32(reinterpret_cast<const T*>(p.bias)[c + k]) : 0.f;
        }
      }
#pragma unroll
      for (int r = 1; r < 4; ++r) {
        if (4 - r <= W - 1) load_xv<T>(p, x, st, b, s_begin - 4 + r, c, win[r]);
        else {
#pragma unroll
          for (int k = 0; k < CONV_V; ++k) win[r][k] = 0.f;
        }
      }
      // s runs over the tokens whose da is formed; dx[s-3] is complete at step s
      const int s_end = min(t1 + 3, p.T + 3);
      auto step = [&](int s, bool in, const float (&xin)[CONV_V], const float (&gy)[CONV_V]) {
        float g[CONV_V];
        const bool mine = s < t1;   // each token's weight / bias contribution is counted once
#pragma unroll
        for (int k = 0; k < CONV_V; ++k) {
          win[0][k] = win[1][k]; win[1][k] = win[2][k]; win[2][k] = win[3][k];
          da[0][k] = da[1][k]; da[1][k] = da[2][k]; da[2][k] = da[3][k];
          float d = 0.f;
          if (in) {
            win[3][k] = xin[k];
            const float a = bias[k] + wj[0][k] * win[0][k] + wj[1][k] * win[1][k] + wj[2][k] * win[2][k] +
                            wj[3][k] * win[3][k];
            d = gy[k] * dsilu_f(a);
            if (mine) {
              dwacc[0][k] += d * win[0][k]; dwacc[1][k] += d * win[1][k];
              dwacc[2][k] += d * win[2][k]; dwacc[3][k] += d * win[3][k];
              dbacc[k] += d;
            }
          } else {
            win[3][k] = 0.f;
          }
          da[3][k] = d;
          g[k] = wj[3][k] * da[0][k] + wj[2][k] * da[1][k] + wj[1][k] * da[2][k] + wj[0][k] * da[3][k];
        }
        const int t = s - 3;
        if (t >= t0 && t < t1) store4<T>(dx + ((size_t)b * p.T + t) * p.C + c, g);
        else if (t < 0 && t0 == 0 && q.dstate && t >= -(W - 1)) {
#pragma unroll
          for (int k = 0; k < CONV_V; ++k)
            reinterpret_cast<T*>(q.dstate)[((size_t)b * p.C + c + k) * (W - 1) + (W - 1 + t)] = from_f32<T>(g[k]);
        }
      };
      if (s_end - s_begin == CONV_TT + 3 && s_end <= p.T) {
        // full tile with its look-ahead inside the sequence: 35 steps as 5 batches of 7 whose loads
        // are all issued (unconditionally) before the first store of the batch
        constexpr int SB = 7;
        static_assert((CONV_TT + 3) % SB == 0, "batching of the backward walk");
#pragma unroll 1
        for (int sb = s_begin; sb < s_end; sb += SB) {
          using Raw = typename std::conditional<sizeof(T) == 4, uint4, uint2>::type;   // 4 channels
          Raw xr[SB], gr[SB];
#pragma unroll
          for (int i = 0; i < SB; ++i) {
            xr[i] = *reinterpret_cast<const Raw*>(x + ((size_t)b * p.T + sb + i) * p.xs + c);
            gr[i] = *reinterpret_cast<const Raw*>(dUb + (size_t)(sb + i) * p.ust);
          }
#pragma unroll
          for (int i = 0; i < SB; ++i) {
            float xin[CONV_V], gy[CONV_V];
            const T* ex = reinterpret_cast<const T*>(&xr[i]);
            const T* eg = reinterpret_cast<const T*>(&gr[i]);
#pragma unroll
            for (int k = 0; k < CONV_V; ++k) { xin[k] = to_f32(ex[k]); gy[k] = to_f32(eg[k]); }
            step(sb + i, true, xin, gy);
          }
        }
      } else {
        for (int s = s_begin; s < s_end; ++s) {
          float xin[CONV_V], gy[CONV_V];
          const bool in = s < p.T;
          if (in) {
            load4<T>(x + ((size_t)b * p.T + s) * p.xs + c, xin);
            load4<T>(dUb + (size_t)s * p.ust, gy);
          }
          step(s, in, xin, gy);
        }
      }
    }
  }
  if (!p.w) return;
#pragma unroll
  for (int k = 0; k < CONV_V; ++k) {
#pragma unroll
    for (int j = 0; j < 4; ++j) s_acc[sub][j][lane * CONV_V + k] = dwacc[j][k];
    s_acc[sub][4][lane * CONV_V + k] = dbacc[k];
  }
  __syncthreads();
  // 5 x 128 sums of CONV_SUB partials; one atomic per (channel, tap) per CTA
  for (int i = threadIdx.x; i < 5 * 32 * CONV_V; i += blockDim.x) {
    const int j = i / (32 * CONV_V), cc = i - j * (32 * CONV_V);
    const int ch = blockIdx.x * 32 * CONV_V + cc;
    if (ch >= p.C) continue;
    float v = 0.f;
#pragma unroll
    for (int r = 0; r < CONV_SUB; ++r) v += s_acc[r][j][cc];
    if (j < 4) { if (j >= 4 - p.W) atomicAdd(q.dw + (size_t)ch * p.W + (j - (4 - p.W)), v); }
    else if (q.dbias) atomicAdd(q.dbias + ch, v);
  }
}

inline bool value_vec_ok(const ValueParams& p, const void* a, const void* b, int V = CONV_V) {
  const int align = 16;
  return p.P % V == 0 && p.C % V == 0 && p.xs % V == 0 && p.usb % V == 0 &&
         p.ush % V == 0 && p.ust % V == 0 && aligned(p.x, align) && aligned(p.U, align) &&
         (a == nullptr || aligned(a, align)) && (b == nullptr || aligned(b, align));
}

// ---- B / C parameterisation ------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(256) bc_fwd_kernel(const T* __restrict__ bc, T* __restrict__ Bo,
                                                     T* __restrict__ Co, int batch, int Tn,
                                                     int G, int N, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long long)batch * Tn * G) return;
  const int g = (int)(row % G);
  const long long bt = row / G;
  const int t = (int)(bt % Tn), b = (int)(bt / Tn);
  const T* src = bc + (size_t)row * 4 * N;
  T* outs[2] = {Bo + (((size_t)b * G + g) * Tn + t) * 2 * N, Co + (((size_t)b * G + g) * Tn + t) * 2 * N};
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const T* amp_row = src + (size_t)(2 * which) * N;
    const T* ph_row = amp_row + N;
    float ss = 0.f;
    for (int n = lane; n < N; n += 32) {
      const float a = softplus_f(to_f32(amp_row[n]));
      ss += a * a;
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(fmaxf(ss / (float)N, eps));
    for (int n = lane; n < N; n += 32) {
      const float a = softplus_f(to_f32(amp_row[n])) * inv;
      const float ph = 3.14159265358979323846f * tanhf(to_f32(ph_row[n]));
      float sn, cs;
      sincosf(ph, &sn, &cs);
      outs[which][2 * n] = from_f32<T>(a * cs);
      outs[which][2 * n + 1] = from_f32<T>(a * sn);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bc_bwd_kernel(const T* __restrict__ bc,
                                                     const T* __restrict__ dBo,
                                                     const T* __restrict__ dCo,
                                                     T* __restrict__ dbc, int batch, int Tn,
                                                     int G, int N, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long long)batch * Tn * G) return;
  const int g = (int)(row % G);
  const long long bt = row / G;
  const int t = (int)(bt % Tn), b = (int)(bt / Tn);
  const T* src = bc + (size_t)row * 4 * N;
  T* dst = dbc + (size_t)row * 4 * N;
  const T* gs[2] = {dBo + (((size_t)b * G + g) * Tn + t) * 2 * N, dCo + (((size_t)b * G + g) * Tn + t) * 2 * N};
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const T* amp_row = src + (size_t)(2 * which) * N;
    const T* ph_row = amp_row + N;
    float ss = 0.f, gsum = 0.f;
    for (int n = lane; n < N; n += 32) {
      const float a = softplus_f(to_f32(amp_row[n]));
      const float ph = 3.14159265358979323846f * tanhf(to_f32(ph_row[n]));
      float sn, cs;
      sincosf(ph, &sn, &cs);
      ss += a * a;
      gsum += a * (cs * to_f32(gs[which][2 * n]) + sn * to_f32(gs[which][2 * n + 1]));
    }
    ss = warp_sum(ss); gsum = warp_sum(gsum);
    const float ms = ss / (float)N;
    const float inv = rsqrtf(fmaxf(ms, eps));
    const float g_ms = ms > eps ? -0.5f * inv * inv * inv * gsum : 0.f;
    for (int n = lane; n < N; n += 32) {
      const float xa = to_f32(amp_row[n]);
      const float a = softplus_f(xa);
      const float th = tanhf(to_f32(ph_row[n]));
      const float ph = 3.14159265358979323846f * th;
      float sn, cs;
      sincosf(ph, &sn, &cs);
      const float gre = to_f32(gs[which][2 * n]), gim = to_f32(gs[which][2 * n + 1]);
      const float g_amp = inv * (cs * gre + sn * gim) + g_ms * 2.f * a / (float)N;
      const float g_ph = a * inv * (cs * gim - sn * gre);
      dst[(size_t)(2 * which) * N + n] = from_f32<T>(g_amp * sigmoid_f(xa));
      dst[(size_t)(2 * which + 1) * N + n] = from_f32<T>(g_ph * 3.14159265358979323846f * (1.f - th * th));
    }
  }
}

// ---- vector path of the B / C kernels (N % 4 == 0, N <= 64) ----------------------------------------
// One warp per (batch, token, group) record of 4 rows x N: lanes 0-15 produce B, lanes 16-31 C;
// a lane owns 4 consecutive n: two 8-byte loads (amplitude and phase logits), one 16-byte store of
// 4 complex values.  The mean over n is a shuffle reduction inside the 16-lane half.  With 16-bit
// io the transcendental functions are the fast intrinsics (their error is far below the output's
// rounding); float32 io keeps the precise ones.
template <bool FAST> __device__ __forceinline__ float softplus_v(float x) {
  if (FAST) return fmaxf(x, 0.f) + __logf(1.f + __expf(-fabsf(x)));
  return softplus_f(x);
}
template <bool FAST> __device__ __forceinline__ float tanh_v(float x) {
  if (FAST) {   // one MUFU op, relative error 2^-11: below the rounding of 16-bit outputs
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return tanhf(x);
}
template <bool FAST> __device__ __forceinline__ float sigmoid_v(float x) {
  if (FAST) return 0.5f * tanh_v<true>(0.5f * x) + 0.5f;
  return sigmoid_f(x);
}
template <bool FAST> __device__ __forceinline__ void sincos_v(float x, float* s, float* c) {
  if (FAST) __sincosf(x, s, c);   // |x| <= pi here
  else sincosf(x, s, c);
}
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float q[4];
    load4<T>(p + 4 * h, q);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[4 * h + i] = q[i];
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    store16<T>(p, v);
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h)
      *reinterpret_cast<float4*>(p + 4 * h) = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
  }
}
__device__ __forceinline__ float half_warp_sum(float v) {   // over the 16 lanes of a half-warp
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int BC_GCH = 8;   // groups one warp walks: grid = (tokens / 8, groups / BC_GCH, batch)

// One warp per (batch, token, run of up to BC_GCH groups); the grid carries batch and the run, so no
// index is divided at run time.  The next record's logits are requested before the current one is
// evaluated.  (The kernels are bound by instruction issue and the XU pipe - five to six MUFU operations per
// complex pair - not by DRAM.)
template <typename T>
__global__ void __launch_bounds__(256) bc_fwd_vec_kernel(const T* __restrict__ bc, T* __restrict__ Bo,
                                                         T* __restrict__ Co, int Tn, int G, int N, float eps) {
  constexpr bool FAST = sizeof(T) == 2;
  const int lane = threadIdx.x & 31, which = lane >> 4, n0 = 4 * (lane & 15);
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), b = blockIdx.z;
  const int g0 = blockIdx.y * BC_GCH, g1 = min(G, g0 + BC_GCH);
  if (t >= Tn) return;
  const bool act = n0 < N;
  const T* src = bc + (((size_t)b * Tn + t) * G + g0) * 4 * N + (size_t)(2 * which) * N + n0;
  T* dst = (which ? Co : Bo) + (((size_t)b * G + g0) * Tn + t) * 2 * N + 2 * n0;
  const size_t dstep = (size_t)Tn * 2 * N;
  const float inv_n = 1.f / (float)N;
  float amp[4] = {0.f, 0.f, 0.f, 0.f}, ph[4] = {0.f, 0.f, 0.f, 0.f};
  if (act) { load4<T>(src, amp); load4<T>(src + N, ph); }
  for (int g = g0; g < g1; ++g) {
    float namp[4] = {0.f, 0.f, 0.f, 0.f}, nph[4] = {0.f, 0.f, 0.f, 0.f};
    src += 4 * N;
    if (act && g + 1 < g1) { load4<T>(src, namp); load4<T>(src + N, nph); }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      amp[i] = act ? softplus_v<FAST>(amp[i]) : 0.f;
      ss += amp[i] * amp[i];
    }
    ss = half_warp_sum(ss);
    if (act) {
      const float inv = rsqrtf(fmaxf(ss * inv_n, eps));
      float o[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sn, cs;
        sincos_v<FAST>(3.14159265358979323846f * tanh_v<FAST>(ph[i]), &sn, &cs);
        const float a = amp[i] * inv;
        o[2 * i] = a * cs; o[2 * i + 1] = a * sn;
      }
      store8<T>(dst, o);
    }
    dst += dstep;
#pragma unroll
    for (int i = 0; i < 4; ++i) { amp[i] = namp[i]; ph[i] = nph[i]; }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bc_bwd_vec_kernel(const T* __restrict__ bc,
                                                         const T* __restrict__ dBo,
                                                         const T* __restrict__ dCo,
                                                         T* __restrict__ dbc, int Tn, int G, int N, float eps) {
  constexpr bool FAST = sizeof(T) == 2;
  const int lane = threadIdx.x & 31, which = lane >> 4, n0 = 4 * (lane & 15);
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), b = blockIdx.z;
  const int g0 = blockIdx.y * BC_GCH, g1 = min(G, g0 + BC_GCH);
  if (t >= Tn) return;
  const bool act = n0 < N;
  const size_t in_off = (((size_t)b * Tn + t) * G + g0) * 4 * N + (size_t)(2 * which) * N + n0;
  const T* src = bc + in_off;
  T* dst = dbc + in_off;
  const T* grad = (which ? dCo : dBo) + (((size_t)b * G + g0) * Tn + t) * 2 * N + 2 * n0;
  const size_t gstep = (size_t)Tn * 2 * N;
  const float inv_n = 1.f / (float)N;
  float xa[4] = {0.f, 0.f, 0.f, 0.f}, xp[4] = {0.f, 0.f, 0.f, 0.f}, gr[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) gr[i] = 0.f;
  if (act) { load4<T>(src, xa); load4<T>(src + N, xp); load8<T>(grad, gr); }
  for (int g = g0; g < g1; ++g) {
    float nxa[4] = {0.f, 0.f, 0.f, 0.f}, nxp[4] = {0.f, 0.f, 0.f, 0.f}, ngr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) ngr[i] = 0.f;
    src += 4 * N; grad += gstep;
    if (act && g + 1 < g1) { load4<T>(src, nxa); load4<T>(src + N, nxp); load8<T>(grad, ngr); }
    float a[4], th[4], sn[4], cs[4];
    float ss = 0.f, gsum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[i] = act ? softplus_v<FAST>(xa[i]) : 0.f;
      th[i] = tanh_v<FAST>(xp[i]);
      sincos_v<FAST>(3.14159265358979323846f * th[i], &sn[i], &cs[i]);
      ss += a[i] * a[i];
      gsum += a[i] * (cs[i] * gr[2 * i] + sn[i] * gr[2 * i + 1]);
    }
    ss = half_warp_sum(ss); gsum = half_warp_sum(gsum);
    if (act) {
      const float ms = ss * inv_n;
      const float inv = rsqrtf(fmaxf(ms, eps));
      const float g_ms = ms > eps ? -0.5f * inv * inv * inv * gsum : 0.f;
      float da[4], dp[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float gre = gr[2 * i], gim = gr[2 * i + 1];
        const float g_amp = inv * (cs[i] * gre + sn[i] * gim) + g_ms * 2.f * a[i] * inv_n;
        const float g_ph = a[i] * inv * (cs[i] * gim - sn[i] * gre);
        da[i] = g_amp * sigmoid_v<FAST>(xa[i]);
        dp[i] = g_ph * 3.14159265358979323846f * (1.f - th[i] * th[i]);
      }
      store4<T>(dst, da);
      store4<T>(dst + N, dp);
    }
    dst += 4 * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) { xa[i] = nxa[i]; xp[i] = nxp[i]; }
#pragma unroll
    for (int i = 0; i < 8; ++i) gr[i] = ngr[i];
  }
}

inline bool bc_vec_ok(int batch, int groups, int N, const void* a, const void* b, const void* c, const void* d) {
  return batch <= 65535 && (groups + BC_GCH - 1) / BC_GCH <= 65535 && N % 4 == 0 && N <= 64 && aligned(a, 16) &&
         aligned(b, 16) && aligned(c, 16) && (d == nullptr || aligned(d, 16));
}

// (the coefficient arithmetic - zc, CoeffOut, wrap_angle_f, coeff_eval - lives in scanprep_math.cuh)
struct CoeffParams {
  const void* params;
  const float *dt_bias, *alpha_bias, *theta_mod_bias, *theta_bias, *theta_sign;
  sl_scanprep_config cfg;
  float *M, *K;
  const float *dM, *dK;
  void* dparams;
  float *d_dt_bias, *d_alpha_bias, *d_theta_mod_bias, *d_theta_bias;
  int batch, T, H;
};

// grid (ceil(T/128), H, batch), thread = token: outputs are coalesced along T.
template <typename T>
__global__ void __launch_bounds__(128) coeff_fwd_kernel(CoeffParams p) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, b = blockIdx.z;
  if (t >= p.T) return;
  const T* pr = reinterpret_cast<const T*>(p.params) + ((size_t)b * p.T + t) * 3 * p.H + 3 * h;
  const CoeffOut o = coeff_eval<false>(to_f32(pr[0]) + p.dt_bias[h], to_f32(pr[1]) + p.alpha_bias[h],
                                to_f32(pr[2]) + p.theta_mod_bias[h], p.theta_bias[h],
                                p.theta_sign[h], p.cfg);
  const size_t i = ((size_t)b * p.H + h) * p.T + t;
  reinterpret_cast<float2*>(p.M)[i] = make_float2((float)o.rho.re, (float)o.rho.im);
  const zc kp = {o.dt * o.k2.re, o.dt * o.k2.im};
  const zc kc = {o.dt * o.k1.re - kp.re, o.dt * o.k1.im - kp.im};
  reinterpret_cast<float4*>(p.K)[i] = make_float4((float)kp.re, (float)kp.im, (float)kc.re, (float)kc.im);
}

template <typename T>
__global__ void __launch_bounds__(128) coeff_bwd_kernel(CoeffParams p) {
  __shared__ float s_red[4][4];
  const int t = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y, b = blockIdx.z;
  float g0 = 0.f, g1 = 0.f, g2 = 0.f, gx = 0.f;
  if (t < p.T) {
    const T* pr = reinterpret_cast<const T*>(p.params) + ((size_t)b * p.T + t) * 3 * p.H + 3 * h;
    const CoeffOut o = coeff_eval(to_f32(pr[0]) + p.dt_bias[h], to_f32(pr[1]) + p.alpha_bias[h],
                                  to_f32(pr[2]) + p.theta_mod_bias[h], p.theta_bias[h],
                                  p.theta_sign[h], p.cfg);
    const size_t i = ((size_t)b * p.H + h) * p.T + t;
    const float2 gm = reinterpret_cast<const float2*>(p.dM)[i];
    const float4 gk = reinterpret_cast<const float4*>(p.dK)[i];
    const zc gM = {gm.x, gm.y}, gKp = {gk.x, gk.y}, gKc = {gk.z, gk.w};
    // kp = dt k2 ; kc = dt (k1 - k2)
    const zc gk1 = {o.dt * gKc.re, o.dt * gKc.im};
    const zc gk2 = {o.dt * (gKp.re - gKc.re), o.dt * (gKp.im - gKc.im)};
    const zc k12 = {o.k1.re - o.k2.re, o.k1.im - o.k2.im};
    const double g_dt = (o.k2.re * gKp.re + o.k2.im * gKp.im) + (k12.re * gKc.re + k12.im * gKc.im);
    zc gz = zconj_mul(o.rho, gM);
    const zc a1 = zconj_mul(o.dk1, gk1), a2 = zconj_mul(o.dk2, gk2);
    gz.re += a1.re + a2.re; gz.im += a1.im + a2.im;
    const double g_r = gz.re / o.r;
    const double g_alpha = -(double)(p.cfg.r_max - p.cfg.r_min) * o.ea * g_r;
    const double span = fmax((double)p.cfg.theta_init_max - (double)p.cfg.theta_init_min, 1.0e-6);
    const double g_thu = span * (double)p.theta_sign[h] * gz.im;
    const double g_x = o.dsg_thu * g_thu;
    g0 = (float)((double)(p.cfg.dt_max - p.cfg.dt_min) * o.dsg_dt * g_dt);
    g1 = (float)((double)(p.cfg.alpha_max - p.cfg.alpha_min) * o.dsg_al * g_alpha);
    g2 = (float)((double)p.cfg.theta_mod_scale * (1.0 - o.tanh2) * g_x);
    gx = (float)g_x;
    T* dp = reinterpret_cast<T*>(p.dparams) + ((size_t)b * p.T + t) * 3 * p.H + 3 * h;
    dp[0] = from_f32<T>(g0); dp[1] = from_f32<T>(g1); dp[2] = from_f32<T>(g2);
  }
  g0 = warp_sum(g0); g1 = warp_sum(g1); g2 = warp_sum(g2); gx = warp_sum(gx);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { s_red[w][0] = g0; s_red[w][1] = g1; s_red[w][2] = g2; s_red[w][3] = gx; }
  __syncthreads();
  if (threadIdx.x < 4) {
    const float s = s_red[0][threadIdx.x] + s_red[1][threadIdx.x] + s_red[2][threadIdx.x] + s_red[3][threadIdx.x];
    float* dst = threadIdx.x == 0 ? p.d_dt_bias : threadIdx.x == 1 ? p.d_alpha_bias
                 : threadIdx.x == 2 ? p.d_theta_mod_bias : p.d_theta_bias;
    if (dst) atomicAdd(dst + h, s);
  }
}

int check_common(int batch, int heads, int groups, int T, int P, int N, int io_dtype, int d_conv) {
  if (batch < 1 || heads < 1 || groups < 1 || heads % groups || T < 1 || P < 1 || N < 1)
    return SL_ERR_BAD_SHAPE;
  if (d_conv < 1 || d_conv > 4) return SL_ERR_UNSUPPORTED;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  return SL_OK;
}

// ---- the three parts of a call (value, B/C, coefficients) touch disjoint tensors -----------------------
// For sequence-sized calls they are launched on three streams between a fork and a join on the caller's
// stream: the B/C kernels are bound by instruction issue, the value kernels by latency, and each leaves most
// of the DRAM bandwidth idle, so they overlap well.  The side streams and events are created on the first
// such call of a device (do that call outside stream capture); fork and join are ordinary event
// dependencies, so a captured call records them as edges of the graph.  SLINOSS_B200_SERIAL_PARTS=1 keeps
// every part on the caller's stream.
struct PartStreams {
  cudaStream_t side[2];
  cudaEvent_t start, done[2];
  bool tried, ok;
  std::mutex in_use;   // held from fork to join: the events are shared by all calls on the device
};
PartStreams* part_streams() {
  static PartStreams table[16];
  static std::mutex guard;   // forward and backward may arrive from different host threads
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  std::lock_guard<std::mutex> lock(guard);
  PartStreams& ps = table[dev];
  if (!ps.tried) {
    ps.tried = true;
    const char* e = getenv("SLINOSS_B200_SERIAL_PARTS");
    ps.ok = !(e && e[0] == '1');
    for (int i = 0; i < 2 && ps.ok; ++i)
      ps.ok = cudaStreamCreateWithFlags(&ps.side[i], cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&ps.done[i], cudaEventDisableTiming) == cudaSuccess;
    ps.ok = ps.ok && cudaEventCreateWithFlags(&ps.start, cudaEventDisableTiming) == cudaSuccess;
    if (!ps.ok) cudaGetLastError();
  }
  return ps.ok ? &ps : nullptr;
}
// Streams of the (value, B/C, coefficient) parts of one call; join() orders the caller's stream after all.
struct PartFork {
  cudaStream_t v, b, c;
  PartStreams* ps = nullptr;
  cudaStream_t main;
  ~PartFork() { join(); }
  PartFork(cudaStream_t st, int parts, long long rows) : v(st), b(st), c(st), main(st) {
    if (parts < 2 || rows < 2048) return;
    ps = part_streams();
    if (!ps) return;
    ps->in_use.lock();
    if (cudaEventRecord(ps->start, st) != cudaSuccess || cudaStreamWaitEvent(ps->side[0], ps->start, 0) != cudaSuccess ||
        cudaStreamWaitEvent(ps->side[1], ps->start, 0) != cudaSuccess) {
      cudaGetLastError();
      ps->in_use.unlock();
      ps = nullptr;
      return;
    }
    b = ps->side[0];
    c = ps->side[1];
  }
  void join() {
    if (!ps) return;
    for (int i = 0; i < 2; ++i) {
      cudaEventRecord(ps->done[i], ps->side[i]);
      cudaStreamWaitEvent(main, ps->done[i], 0);
    }
    ps->in_use.unlock();
    ps = nullptr;
  }
};

}  // namespace
}  // namespace sl

extern "C" int sl_scanprep_conv_fwd(const void* value, int64_t value_row_stride,
                                    const void* conv_weight, const void* conv_bias,
                                    const void* conv_state_in, void* conv_state_out, int d_conv,
                                    const void* params, const void* bc, const float* dt_bias,
                                    const float* alpha_bias, const float* theta_mod_bias,
                                    const float* theta_bias, const float* theta_sign,
                                    const sl_scanprep_config* cfg, void* U, int64_t u_stride_b,
                                    int64_t u_stride_h, int64_t u_stride_t, float* M, float* K,
                                    void* Bo, void* Co, int batch, int heads, int groups, int T,
                                    int P, int N, int io_dtype, void* stream) {
  using namespace sl;
  if (int e = check_common(batch, heads, groups, T, P, N, io_dtype, conv_weight ? d_conv : 1)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (value && !U) return SL_ERR_NULL_POINTER;
  if (bc && (!Bo || !Co || !cfg)) return SL_ERR_NULL_POINTER;
  if (params) {
    if (!M || !K || !cfg || !dt_bias || !alpha_bias || !theta_mod_bias || !theta_bias || !theta_sign)
      return SL_ERR_NULL_POINTER;
    if (!aligned(M, 8) || !aligned(K, 16)) return SL_ERR_BAD_ALIGNMENT;
  }
  PartFork fork(st, (value != nullptr) + (bc != nullptr) + (params != nullptr), (long long)batch * T);
  if (value) {
    ValueParams p{};
    p.x = value; p.w = conv_weight; p.bias = conv_bias; p.state_in = conv_state_in;
    p.state_out = conv_state_out; p.U = U; p.xs = value_row_stride;
    p.usb = u_stride_b; p.ush = u_stride_h; p.ust = u_stride_t;
    p.batch = batch; p.T = T; p.C = heads * P; p.P = P; p.W = conv_weight ? d_conv : 1;
    const int vf = CONV_V;   // 4 channels per thread (8- or 16-byte pieces)
    if (value_vec_ok(p, nullptr, nullptr, vf)) {
      dim3 grid((p.C + 32 * vf - 1) / (32 * vf), (T + CONV_SUB * CONV_TT - 1) / (CONV_SUB * CONV_TT), batch);
      SL_DISPATCH_DTYPE(io_dtype, Tt, { value_fwd_vec_kernel<Tt, CONV_V><<<grid, 256, 0, fork.v>>>(p); });
    } else {
      dim3 grid((p.C + 255) / 256, (T + CONV_TT - 1) / CONV_TT, batch);
      SL_DISPATCH_DTYPE(io_dtype, Tt, { value_fwd_kernel<Tt><<<grid, 256, 0, fork.v>>>(p); });
    }
    note_launches(1);
  }
  if (bc) {
    const long long rows = (long long)batch * T * groups;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    const dim3 vgrid((T + 7) / 8, (groups + BC_GCH - 1) / BC_GCH, batch);
    SL_DISPATCH_DTYPE(io_dtype, Tt, {
      if (bc_vec_ok(batch, groups, N, bc, Bo, Co, nullptr))
        bc_fwd_vec_kernel<Tt><<<vgrid, 256, 0, fork.b>>>(reinterpret_cast<const Tt*>(bc), reinterpret_cast<Tt*>(Bo),
                                                     reinterpret_cast<Tt*>(Co), T, groups, N, cfg->eps);
      else
        bc_fwd_kernel<Tt><<<blocks, 256, 0, fork.b>>>(reinterpret_cast<const Tt*>(bc), reinterpret_cast<Tt*>(Bo),
                                                  reinterpret_cast<Tt*>(Co), batch, T, groups, N, cfg->eps);
    });
    note_launches(1);
  }
  if (params) {
    CoeffParams p{};
    p.params = params; p.dt_bias = dt_bias; p.alpha_bias = alpha_bias;
    p.theta_mod_bias = theta_mod_bias; p.theta_bias = theta_bias; p.theta_sign = theta_sign;
    p.cfg = *cfg; p.M = M; p.K = K; p.batch = batch; p.T = T; p.H = heads;
    dim3 grid((T + 127) / 128, heads, batch);
    SL_DISPATCH_DTYPE(io_dtype, Tt, { coeff_fwd_kernel<Tt><<<grid, 128, 0, fork.c>>>(p); });
    note_launches(1);
  }
  fork.join();
  return launch_status();
}

extern "C" int sl_scanprep_conv_bwd(
    const void* value, int64_t value_row_stride, const void* conv_weight, const void* conv_bias,
    const void* conv_state_in, int d_conv, const void* params, const void* bc,
    const float* dt_bias, const float* alpha_bias, const float* theta_mod_bias,
    const float* theta_bias, const float* theta_sign, const sl_scanprep_config* cfg,
    const void* dU, int64_t u_stride_b, int64_t u_stride_h, int64_t u_stride_t, const float* dM,
    const float* dK, const void* dBo, const void* dCo, void* d_value, float* d_conv_weight,
    float* d_conv_bias, void* d_conv_state, void* d_params, void* d_bc, float* d_dt_bias,
    float* d_alpha_bias, float* d_theta_mod_bias, float* d_theta_bias, int batch, int heads,
    int groups, int T, int P, int N, int io_dtype, void* stream) {
  using namespace sl;
  if (int e = check_common(batch, heads, groups, T, P, N, io_dtype, conv_weight ? d_conv : 1)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dU && (!d_value || !value || (conv_weight && !d_conv_weight))) return SL_ERR_NULL_POINTER;
  if (dBo && (!dCo || !bc || !d_bc || !cfg)) return SL_ERR_NULL_POINTER;
  if (dM) {
    if (!dK || !params || !d_params || !cfg || !dt_bias || !alpha_bias || !theta_mod_bias ||
        !theta_bias || !theta_sign)
      return SL_ERR_NULL_POINTER;
    if (!aligned(dM, 8) || !aligned(dK, 16)) return SL_ERR_BAD_ALIGNMENT;
  }
  PartFork fork(st, (dU != nullptr) + (dBo != nullptr) + (dM != nullptr), (long long)batch * T);
  if (dU) {
    ValueBwdParams q{};
    ValueParams& p = q.f;
    p.x = value; p.w = conv_weight; p.bias = conv_bias; p.state_in = conv_state_in;
    p.xs = value_row_stride; p.usb = u_stride_b; p.ush = u_stride_h; p.ust = u_stride_t;
    p.batch = batch; p.T = T; p.C = heads * P; p.P = P; p.W = conv_weight ? d_conv : 1;
    q.dU = dU; q.dx = d_value; q.dstate = d_conv_state; q.dw = d_conv_weight; q.dbias = d_conv_bias;
    ValueParams pv = p;
    pv.U = const_cast<void*>(dU);
    if (value_vec_ok(pv, d_value, nullptr)) {
      dim3 grid((p.C + 32 * CONV_V - 1) / (32 * CONV_V), (T + CONV_SUB * CONV_TT - 1) / (CONV_SUB * CONV_TT), batch);
      SL_DISPATCH_DTYPE(io_dtype, Tt, { value_bwd_vec_kernel<Tt><<<grid, 256, 0, fork.v>>>(q); });
    } else {
      dim3 grid((p.C + 255) / 256, (T + CONV_TT - 1) / CONV_TT, batch);
      SL_DISPATCH_DTYPE(io_dtype, Tt, { value_bwd_kernel<Tt><<<grid, 256, 0, fork.v>>>(q); });
    }
    note_launches(1);
  }
  if (dBo) {
    const long long rows = (long long)batch * T * groups;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    const dim3 vgrid((T + 7) / 8, (groups + BC_GCH - 1) / BC_GCH, batch);
    SL_DISPATCH_DTYPE(io_dtype, Tt, {
      if (bc_vec_ok(batch, groups, N, bc, dBo, dCo, d_bc))
        bc_bwd_vec_kernel<Tt><<<vgrid, 256, 0, fork.b>>>(reinterpret_cast<const Tt*>(bc),
                                                     reinterpret_cast<const Tt*>(dBo),
                                                     reinterpret_cast<const Tt*>(dCo), reinterpret_cast<Tt*>(d_bc),
                                                     T, groups, N, cfg->eps);
      else
        bc_bwd_kernel<Tt><<<blocks, 256, 0, fork.b>>>(reinterpret_cast<const Tt*>(bc), reinterpret_cast<const Tt*>(dBo),
                                                  reinterpret_cast<const Tt*>(dCo), reinterpret_cast<Tt*>(d_bc),
                                                  batch, T, groups, N, cfg->eps);
    });
    note_launches(1);
  }
  if (dM) {
    CoeffParams p{};
    p.params = params; p.dt_bias = dt_bias; p.alpha_bias = alpha_bias;
    p.theta_mod_bias = theta_mod_bias; p.theta_bias = theta_bias; p.theta_sign = theta_sign;
    p.cfg = *cfg; p.dM = dM; p.dK = dK; p.dparams = d_params; p.d_dt_bias = d_dt_bias;
    p.d_alpha_bias = d_alpha_bias; p.d_theta_mod_bias = d_theta_mod_bias;
    p.d_theta_bias = d_theta_bias; p.batch = batch; p.T = T; p.H = heads;
    dim3 grid((T + 127) / 128, heads, batch);
    SL_DISPATCH_DTYPE(io_dtype, Tt, { coeff_bwd_kernel<Tt><<<grid, 128, 0, fork.c>>>(p); });
    note_launches(1);
  }
  fork.join();
  return launch_status();
}
