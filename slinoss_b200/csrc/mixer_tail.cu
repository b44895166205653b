// Row-wise part of the mixer tail: skip connection, SiLU gate and RMSNorm.
//
//   pre    = Y + d_skip[h] * U                 (float32, rounded to the io dtype)
//   hidden = pre * SiLU(gate)                  (float32, rounded to the io dtype)
//   normed = hidden * rsqrt(mean(hidden^2) + eps) * w
//
// Reference: slinoss/ops/mixer/tail.py:63-142 (the roundings above are the ones
// the reference makes between its steps).  One CTA owns one (batch, token) row of
// heads*P channels; Y and U are read in their (batch, heads, T, P) layout and the
// result is written channel-last, ready for the out_proj GEMM.
#include "common.cuh"

namespace sl {
namespace {

constexpr int TAIL_THREADS = 256;
constexpr int TAIL_MAX_PER_THREAD = 16;  // channels <= 4096

template <typename T>
__device__ __forceinline__ float round_io(float v) { return to_f32(from_f32<T>(v)); }

__device__ __forceinline__ float block_sum(float v, float* s_red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) s_red[w] = v;
  __syncthreads();
  float s = 0.f;
  for (int k = 0; k < (int)(blockDim.x >> 5); ++k) s += s_red[k];
  return s;
}

struct TailParams {
  const void *Y, *gate, *skip, *w, *dn;
  const float* d_skip;
  void *normed, *dY, *dgate, *dskip_in;
  float *d_d_skip, *d_w;
  int64_t gs;
  float eps;
  int batch, H, T, P;
};

template <typename T>
__global__ void __launch_bounds__(TAIL_THREADS) tail_fwd_kernel(TailParams p) {
  __shared__ float s_red[TAIL_THREADS / 32];
  const int C = p.H * p.P;
  const T* Y = reinterpret_cast<const T*>(p.Y);
  const T* S = reinterpret_cast<const T*>(p.skip);
  const T* gate = reinterpret_cast<const T*>(p.gate);
  const T* w = reinterpret_cast<const T*>(p.w);
  T* out = reinterpret_cast<T*>(p.normed);
  for (long long row = blockIdx.x; row < (long long)p.batch * p.T; row += gridDim.x) {
    const int t = (int)(row % p.T), b = (int)(row / p.T);
    float hid[TAIL_MAX_PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * TAIL_THREADS;
      hid[i] = 0.f;
      if (c < C) {
        const int h = c / p.P, pp = c - h * p.P;
        const size_t yi = (((size_t)b * p.H + h) * p.T + t) * p.P + pp;
        float pre = to_f32(Y[yi]);
        if (S) pre = round_io<T>(pre + to_f32(S[yi]) * p.d_skip[h]);
        const float g = to_f32(gate[(size_t)row * p.gs + c]);
        hid[i] = round_io<T>(pre * silu_f(g));
        ss += hid[i] * hid[i];
      }
    }
    ss = block_sum(ss, s_red);
    const float rstd = rsqrtf(ss / (float)C + p.eps);
#pragma unroll
    for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * TAIL_THREADS;
      if (c < C) out[(size_t)row * C + c] = from_f32<T>(hid[i] * rstd * to_f32(w[c]));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(TAIL_THREADS) tail_bwd_kernel(TailParams p) {
  __shared__ float s_red[TAIL_THREADS / 32];
  extern __shared__ float s_dskip[];  // H floats
  const int C = p.H * p.P;
  const T* Y = reinterpret_cast<const T*>(p.Y);
  const T* S = reinterpret_cast<const T*>(p.skip);
  const T* gate = reinterpret_cast<const T*>(p.gate);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* dn = reinterpret_cast<const T*>(p.dn);
  T* dY = reinterpret_cast<T*>(p.dY);
  T* dgate = reinterpret_cast<T*>(p.dgate);
  T* dS = reinterpret_cast<T*>(p.dskip_in);
  float dw_acc[TAIL_MAX_PER_THREAD];
#pragma unroll
  for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) dw_acc[i] = 0.f;
  for (int i = threadIdx.x; i < p.H; i += blockDim.x) s_dskip[i] = 0.f;
  __syncthreads();
  for (long long row = blockIdx.x; row < (long long)p.batch * p.T; row += gridDim.x) {
    const int t = (int)(row % p.T), b = (int)(row / p.T);
    float hid[TAIL_MAX_PER_THREAD], gw[TAIL_MAX_PER_THREAD];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * TAIL_THREADS;
      hid[i] = gw[i] = 0.f;
      if (c < C) {
        const int h = c / p.P, pp = c - h * p.P;
        const size_t yi = (((size_t)b * p.H + h) * p.T + t) * p.P + pp;
        float pre = to_f32(Y[yi]);
        if (S) pre = round_io<T>(pre + to_f32(S[yi]) * p.d_skip[h]);
        const float g = to_f32(gate[(size_t)row * p.gs + c]);
        hid[i] = round_io<T>(pre * silu_f(g));
        gw[i] = to_f32(dn[(size_t)row * C + c]) * to_f32(w[c]);
        ss += hid[i] * hid[i];
        dot += hid[i] * gw[i];
      }
    }
    ss = block_sum(ss, s_red);
    dot = block_sum(dot, s_red);
    const float rstd = rsqrtf(ss / (float)C + p.eps);
    const float coef = dot * rstd * rstd * rstd / (float)C;
#pragma unroll
    for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * TAIL_THREADS;
      if (c < C) {
        const int h = c / p.P, pp = c - h * p.P;
        const size_t yi = (((size_t)b * p.H + h) * p.T + t) * p.P + pp;
        const float dnv = to_f32(dn[(size_t)row * C + c]);
        dw_acc[i] += dnv * hid[i] * rstd;
        const float dh = rstd * gw[i] - hid[i] * coef;
        float pre = to_f32(Y[yi]);
        float sv = 0.f;
        if (S) { sv = to_f32(S[yi]); pre = round_io<T>(pre + sv * p.d_skip[h]); }
        const float g = to_f32(gate[(size_t)row * p.gs + c]);
        const float sg = sigmoid_f(g);
        const float dpre = dh * g * sg;
        dgate[(size_t)row * C + c] = from_f32<T>(dh * pre * sg * (1.f + g * (1.f - sg)));
        dY[yi] = from_f32<T>(dpre);
        if (S) {
          if (dS) dS[yi] = from_f32<T>(dpre * p.d_skip[h]);
          atomicAdd(&s_dskip[h], dpre * sv);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < TAIL_MAX_PER_THREAD; ++i) {
    const int c = threadIdx.x + i * TAIL_THREADS;
    if (c < C) atomicAdd(p.d_w + c, dw_acc[i]);
  }
  if (S && p.d_d_skip)
    for (int i = threadIdx.x; i < p.H; i += blockDim.x) atomicAdd(p.d_d_skip + i, s_dskip[i]);
}

// ---- vector path: every thread owns 16-byte pieces (8 or 4 channels of one head) ---------------
// Needs P % V == 0 (a piece never straddles two heads), 16-byte aligned pointers and a gate row
// stride that is a multiple of V.  One CTA owns one row at a time; a thread keeps the same
// channels for every row it visits, so the weight / skip gradients are accumulated in registers
// over the CTA's rows and added to the float32 accumulators once at the end.
constexpr int TAIL_VIT_MAX = 2;   // pieces per thread: channels <= 2 * 256 * V

template <typename T, int TAIL_VIT>
__global__ void __launch_bounds__(TAIL_THREADS) tail_fwd_vec_kernel(TailParams p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float s_red[TAIL_THREADS / 32];
  const int C = p.H * p.P;
  const T* Y = reinterpret_cast<const T*>(p.Y);
  const T* S = reinterpret_cast<const T*>(p.skip);
  const T* gate = reinterpret_cast<const T*>(p.gate);
  const T* w = reinterpret_cast<const T*>(p.w);
  T* out = reinterpret_cast<T*>(p.normed);
  float wv[TAIL_VIT][V], dsk[TAIL_VIT];
  int hh[TAIL_VIT], pp[TAIL_VIT];
#pragma unroll
  for (int i = 0; i < TAIL_VIT; ++i) {
    const int c = (threadIdx.x + i * TAIL_THREADS) * V;
    hh[i] = 0; pp[i] = 0; dsk[i] = 0.f;
    if (c < C) {
      hh[i] = c / p.P; pp[i] = c - hh[i] * p.P;
      load16<T>(w + c, wv[i]);
      if (S) dsk[i] = p.d_skip[hh[i]];
    }
  }
  // The raw 16-byte pieces of the NEXT row are fetched before the current row is reduced, so the
  // loads overlap the block reduction and the stores.
  const unsigned rows = (unsigned)p.batch * (unsigned)p.T;   // < 2^31, checked by the launcher
  uint4 nY[TAIL_VIT], nG[TAIL_VIT], nS[TAIL_VIT];
  auto fetch = [&](unsigned row) {
    const int t = (int)(row % (unsigned)p.T), b = (int)(row / (unsigned)p.T);
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        const size_t yi = (((size_t)b * p.H + hh[i]) * p.T + t) * p.P + pp[i];
        nY[i] = *reinterpret_cast<const uint4*>(Y + yi);
        nG[i] = *reinterpret_cast<const uint4*>(gate + (size_t)row * p.gs + c);
        if (S) nS[i] = *reinterpret_cast<const uint4*>(S + yi);
      }
    }
  };
  if (blockIdx.x < rows) fetch(blockIdx.x);
  for (unsigned row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 cY[TAIL_VIT], cG[TAIL_VIT], cS[TAIL_VIT];
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) { cY[i] = nY[i]; cG[i] = nG[i]; cS[i] = nS[i]; }
    if (row + gridDim.x < rows) fetch(row + gridDim.x);
    float hid[TAIL_VIT][V];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        float y[V], g[V];
        unpack16<T>(cY[i], y);
        unpack16<T>(cG[i], g);
        if (S) {
          float sv[V];
          unpack16<T>(cS[i], sv);
#pragma unroll
          for (int k = 0; k < V; k += 2) {
            y[k] += sv[k] * dsk[i]; y[k + 1] += sv[k + 1] * dsk[i];
            round_pair<T>(y[k], y[k + 1]);
          }
        }
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          hid[i][k] = y[k] * silu_f(g[k]); hid[i][k + 1] = y[k + 1] * silu_f(g[k + 1]);
          round_pair<T>(hid[i][k], hid[i][k + 1]);
          ss += hid[i][k] * hid[i][k] + hid[i][k + 1] * hid[i][k + 1];
        }
      }
    }
    ss = block_sum(ss, s_red);
    const float rstd = rsqrtf(ss / (float)C + p.eps);
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        float o[V];
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] = hid[i][k] * rstd * wv[i][k];
        store16<T>(out + (size_t)row * C + c, o);
      }
    }
  }
}

template <typename T, int TAIL_VIT>
__global__ void __launch_bounds__(TAIL_THREADS) tail_bwd_vec_kernel(TailParams p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float s_red[TAIL_THREADS / 32];
  const int C = p.H * p.P;
  const T* Y = reinterpret_cast<const T*>(p.Y);
  const T* S = reinterpret_cast<const T*>(p.skip);
  const T* gate = reinterpret_cast<const T*>(p.gate);
  const T* w = reinterpret_cast<const T*>(p.w);
  const T* dn = reinterpret_cast<const T*>(p.dn);
  T* dY = reinterpret_cast<T*>(p.dY);
  T* dgate = reinterpret_cast<T*>(p.dgate);
  T* dS = reinterpret_cast<T*>(p.dskip_in);
  float wv[TAIL_VIT][V], dw_acc[TAIL_VIT][V], dsk[TAIL_VIT], dsk_acc[TAIL_VIT];
  int hh[TAIL_VIT], pp[TAIL_VIT];
#pragma unroll
  for (int i = 0; i < TAIL_VIT; ++i) {
    const int c = (threadIdx.x + i * TAIL_THREADS) * V;
    hh[i] = 0; pp[i] = 0; dsk[i] = 0.f; dsk_acc[i] = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k) dw_acc[i][k] = 0.f;
    if (c < C) {
      hh[i] = c / p.P; pp[i] = c - hh[i] * p.P;
      load16<T>(w + c, wv[i]);
      if (S) dsk[i] = p.d_skip[hh[i]];
    }
  }
  const unsigned rows = (unsigned)p.batch * (unsigned)p.T;   // < 2^31, checked by the launcher
  uint4 nY[TAIL_VIT], nG[TAIL_VIT], nS[TAIL_VIT], nD[TAIL_VIT];
  auto fetch = [&](unsigned row) {   // raw pieces of the next row, in flight while this one is reduced
    const int t = (int)(row % (unsigned)p.T), b = (int)(row / (unsigned)p.T);
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        const size_t yi = (((size_t)b * p.H + hh[i]) * p.T + t) * p.P + pp[i];
        nY[i] = *reinterpret_cast<const uint4*>(Y + yi);
        nG[i] = *reinterpret_cast<const uint4*>(gate + (size_t)row * p.gs + c);
        nD[i] = *reinterpret_cast<const uint4*>(dn + (size_t)row * C + c);
        if (S) nS[i] = *reinterpret_cast<const uint4*>(S + yi);
      }
    }
  };
  if (blockIdx.x < rows) fetch(blockIdx.x);
  for (unsigned row = blockIdx.x; row < rows; row += gridDim.x) {
    const int t = (int)(row % (unsigned)p.T), b = (int)(row / (unsigned)p.T);
    float pre[TAIL_VIT][V], sv[TAIL_VIT][V], g[TAIL_VIT][V], dnv[TAIL_VIT][V];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        unpack16<T>(nY[i], pre[i]);
        unpack16<T>(nG[i], g[i]);
        unpack16<T>(nD[i], dnv[i]);
        if (S) unpack16<T>(nS[i], sv[i]);
      }
    }
    if (row + gridDim.x < rows) fetch(row + gridDim.x);
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        if (S) {
#pragma unroll
          for (int k = 0; k < V; k += 2) {
            pre[i][k] += sv[i][k] * dsk[i]; pre[i][k + 1] += sv[i][k + 1] * dsk[i];
            round_pair<T>(pre[i][k], pre[i][k + 1]);
          }
        }
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          float h0 = pre[i][k] * silu_f(g[i][k]), h1 = pre[i][k + 1] * silu_f(g[i][k + 1]);
          round_pair<T>(h0, h1);
          ss += h0 * h0 + h1 * h1;
          dot += h0 * dnv[i][k] * wv[i][k] + h1 * dnv[i][k + 1] * wv[i][k + 1];
        }
      }
    }
    ss = block_sum(ss, s_red);
    dot = block_sum(dot, s_red);
    const float rstd = rsqrtf(ss / (float)C + p.eps);
    const float coef = dot * rstd * rstd * rstd / (float)C;
#pragma unroll
    for (int i = 0; i < TAIL_VIT; ++i) {
      const int c = (threadIdx.x + i * TAIL_THREADS) * V;
      if (c < C) {
        const size_t yi = (((size_t)b * p.H + hh[i]) * p.T + t) * p.P + pp[i];
        float o_dy[V], o_dg[V], o_ds[V];
#pragma unroll
        for (int k2 = 0; k2 < V; k2 += 2) {
          float sgv[2], hidv[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            sgv[q] = sigmoid_f(g[i][k2 + q]);
            hidv[q] = pre[i][k2 + q] * (g[i][k2 + q] * sgv[q]);
          }
          round_pair<T>(hidv[0], hidv[1]);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int k = k2 + q;
            const float gg = g[i][k], sg = sgv[q], hid = hidv[q];
            dw_acc[i][k] += dnv[i][k] * hid * rstd;
            const float dh = rstd * dnv[i][k] * wv[i][k] - hid * coef;
            const float dpre = dh * gg * sg;
            o_dg[k] = dh * pre[i][k] * sg * (1.f + gg * (1.f - sg));
            o_dy[k] = dpre;
            if (S) { o_ds[k] = dpre * dsk[i]; dsk_acc[i] += dpre * sv[i][k]; }
          }
        }
        store16<T>(dgate + (size_t)row * C + c, o_dg);
        store16<T>(dY + yi, o_dy);
        if (S && dS) store16<T>(dS + yi, o_ds);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < TAIL_VIT; ++i) {
    const int c = (threadIdx.x + i * TAIL_THREADS) * V;
    if (c < C) {
#pragma unroll
      for (int k = 0; k < V; ++k) atomicAdd(p.d_w + c + k, dw_acc[i][k]);
      if (S && p.d_d_skip) atomicAdd(p.d_d_skip + hh[i], dsk_acc[i]);
    }
  }
}

// The common width (heads * P <= 256 pieces of 16 bytes: one piece per thread) with fewer live registers,
// so that three CTAs stay resident per SM: the row is kept as its four packed pieces and unpacked again
// after the reduction (same operations, same roundings), both row sums travel in one reduction, and its
// shared-memory slots alternate with the row so that one barrier per row is enough.
template <typename T>
__global__ void __launch_bounds__(TAIL_THREADS, 3) tail_bwd_row_kernel(TailParams p) {
  constexpr int V = Vec16<T>::N;
  __shared__ float2 s_red[2][TAIL_THREADS / 32];
  const int C = p.H * p.P;
  const T* Y = reinterpret_cast<const T*>(p.Y);
  const T* S = reinterpret_cast<const T*>(p.skip);
  const T* gate = reinterpret_cast<const T*>(p.gate);
  const T* dn = reinterpret_cast<const T*>(p.dn);
  T* dY = reinterpret_cast<T*>(p.dY);
  T* dgate = reinterpret_cast<T*>(p.dgate);
  T* dS = reinterpret_cast<T*>(p.dskip_in);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = threadIdx.x * V;
  const bool act = c < C;
  const int hh = act ? c / p.P : 0, pp = c - hh * p.P;
  const float dsk = (act && S) ? p.d_skip[hh] : 0.f;
  uint4 wraw = make_uint4(0, 0, 0, 0);
  if (act) wraw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.w) + c);
  float dw_acc[V], dsk_acc = 0.f;
#pragma unroll
  for (int k = 0; k < V; ++k) dw_acc[k] = 0.f;
  const unsigned rows = (unsigned)p.batch * (unsigned)p.T;   // < 2^31, checked by the launcher
  const size_t head_off = (size_t)hh * p.T * p.P + pp, batch_step = (size_t)p.H * p.T * p.P;
  uint4 nY = make_uint4(0, 0, 0, 0), nG = nY, nS = nY, nD = nY;
  auto fetch = [&](unsigned row) {
    if (!act) return;
    const unsigned b = row / (unsigned)p.T, t = row - b * (unsigned)p.T;
    const size_t yi = b * batch_step + head_off + (size_t)t * p.P;
    nY = *reinterpret_cast<const uint4*>(Y + yi);
    nG = *reinterpret_cast<const uint4*>(gate + (size_t)row * p.gs + c);
    nD = *reinterpret_cast<const uint4*>(dn + (size_t)row * C + c);
    if (S) nS = *reinterpret_cast<const uint4*>(S + yi);
  };
  if (blockIdx.x < rows) fetch(blockIdx.x);
  int par = 0;
  for (unsigned row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
    const uint4 cY = nY, cG = nG, cS = nS, cD = nD;
    if (row + gridDim.x < rows) fetch(row + gridDim.x);
    float ss = 0.f, dot = 0.f;
    if (act) {
      float pre[V], g[V], dnv[V], wv[V];
      unpack16<T>(cY, pre); unpack16<T>(cG, g); unpack16<T>(cD, dnv); unpack16<T>(wraw, wv);
      if (S) {
        float sv[V];
        unpack16<T>(cS, sv);
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          pre[k] += sv[k] * dsk; pre[k + 1] += sv[k + 1] * dsk;
          round_pair<T>(pre[k], pre[k + 1]);
        }
      }
#pragma unroll
      for (int k = 0; k < V; k += 2) {
        float h0 = pre[k] * silu_f(g[k]), h1 = pre[k + 1] * silu_f(g[k + 1]);
        round_pair<T>(h0, h1);
        ss += h0 * h0 + h1 * h1;
        dot += h0 * dnv[k] * wv[k] + h1 * dnv[k + 1] * wv[k + 1];
      }
    }
    ss = warp_sum(ss); dot = warp_sum(dot);
    if (lane == 0) s_red[par][warp] = make_float2(ss, dot);
    __syncthreads();
    ss = 0.f; dot = 0.f;
#pragma unroll
    for (int k = 0; k < TAIL_THREADS / 32; ++k) { const float2 v = s_red[par][k]; ss += v.x; dot += v.y; }
    const float rstd = rsqrtf(ss / (float)C + p.eps);
    const float coef = dot * rstd * rstd * rstd / (float)C;
    if (act) {
      const unsigned b = row / (unsigned)p.T, t = row - b * (unsigned)p.T;
      const size_t yi = b * batch_step + head_off + (size_t)t * p.P;
      float pre[V], g[V], dnv[V], wv[V], sv[V];
      unpack16<T>(cY, pre); unpack16<T>(cG, g); unpack16<T>(cD, dnv); unpack16<T>(wraw, wv);
      if (S) {
        unpack16<T>(cS, sv);
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          pre[k] += sv[k] * dsk; pre[k + 1] += sv[k + 1] * dsk;
          round_pair<T>(pre[k], pre[k + 1]);
        }
      }
      float o_dy[V], o_dg[V], o_ds[V];
#pragma unroll
      for (int k2 = 0; k2 < V; k2 += 2) {
        float sgv[2], hidv[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          sgv[q] = sigmoid_f(g[k2 + q]);
          hidv[q] = pre[k2 + q] * silu_f(g[k2 + q]);
        }
        round_pair<T>(hidv[0], hidv[1]);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int k = k2 + q;
          const float gg = g[k], sg = sgv[q], hid = hidv[q];
          dw_acc[k] += dnv[k] * hid * rstd;
          const float dh = rstd * dnv[k] * wv[k] - hid * coef;
          const float dpre = dh * gg * sg;
          o_dg[k] = dh * pre[k] * sg * (1.f + gg * (1.f - sg));
          o_dy[k] = dpre;
          o_ds[k] = 0.f;
          if (S) { o_ds[k] = dpre * dsk; dsk_acc += dpre * sv[k]; }
        }
      }
      store16<T>(dgate + (size_t)row * C + c, o_dg);
      store16<T>(dY + yi, o_dy);
      if (S && dS) store16<T>(dS + yi, o_ds);
    }
  }
  if (act) {
#pragma unroll
    for (int k = 0; k < V; ++k) atomicAdd(p.d_w + c + k, dw_acc[k]);
    if (S && p.d_d_skip) atomicAdd(p.d_d_skip + hh, dsk_acc);
  }
}

template <typename T>
bool tail_vec_ok(const TailParams& p) {
  constexpr int V = Vec16<T>::N;
  const long long C = (long long)p.H * p.P;
  auto al = [](const void* q) { return q == nullptr || aligned(q, 16); };
  return (long long)p.batch * p.T < (1ll << 31) && p.P % V == 0 && p.gs % V == 0 && C <= (long long)TAIL_VIT_MAX * TAIL_THREADS * V && al(p.Y) &&
         al(p.gate) && al(p.skip) && al(p.w) && al(p.dn) && al(p.normed) && al(p.dY) && al(p.dgate) &&
         al(p.dskip_in);
}

int tail_check(const void* Y, const void* gate, const void* skip, const float* d_skip,
               const void* w, int batch, int heads, int T, int P, int io_dtype) {
  if (!Y || !gate || !w) return SL_ERR_NULL_POINTER;
  if ((skip == nullptr) != (d_skip == nullptr)) return SL_ERR_NULL_POINTER;
  if (batch < 1 || heads < 1 || T < 1 || P < 1) return SL_ERR_BAD_SHAPE;
  if ((long long)heads * P > (long long)TAIL_THREADS * TAIL_MAX_PER_THREAD) return SL_ERR_UNSUPPORTED;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  return SL_OK;
}

}  // namespace
}  // namespace sl

extern "C" int sl_mixer_tail_fwd(const void* Y, const void* gate, int64_t gate_row_stride,
                                 const void* skip, const float* d_skip, const void* norm_weight,
                                 float eps, void* normed, int batch, int heads, int T, int P,
                                 int io_dtype, void* stream) {
  using namespace sl;
  if (int e = tail_check(Y, gate, skip, d_skip, norm_weight, batch, heads, T, P, io_dtype)) return e;
  if (!normed) return SL_ERR_NULL_POINTER;
  TailParams p{};
  p.Y = Y; p.gate = gate; p.skip = skip; p.w = norm_weight; p.d_skip = d_skip; p.normed = normed;
  p.gs = gate_row_stride; p.eps = eps; p.batch = batch; p.H = heads; p.T = T; p.P = P;
  const long long rows = (long long)batch * T;
  const unsigned grid = (unsigned)(rows < 148 * 8 ? rows : 148 * 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SL_DISPATCH_DTYPE(io_dtype, Tt, {
    if (tail_vec_ok<Tt>(p)) {
      if ((long long)heads * P <= TAIL_THREADS * Vec16<Tt>::N) tail_fwd_vec_kernel<Tt, 1><<<grid, TAIL_THREADS, 0, st>>>(p);
      else tail_fwd_vec_kernel<Tt, 2><<<grid, TAIL_THREADS, 0, st>>>(p);
    } else tail_fwd_kernel<Tt><<<grid, TAIL_THREADS, 0, st>>>(p);
  });
  note_launches(1);
  return launch_status();
}

extern "C" int sl_mixer_tail_bwd(const void* Y, const void* gate, int64_t gate_row_stride,
                                 const void* skip, const float* d_skip, const void* norm_weight,
                                 float eps, const void* d_normed, void* dY, void* d_gate,
                                 void* d_skip_input, float* d_d_skip, float* d_norm_weight,
                                 int batch, int heads, int T, int P, int io_dtype, void* stream) {
  using namespace sl;
  if (int e = tail_check(Y, gate, skip, d_skip, norm_weight, batch, heads, T, P, io_dtype)) return e;
  if (!d_normed || !dY || !d_gate || !d_norm_weight) return SL_ERR_NULL_POINTER;
  TailParams p{};
  p.Y = Y; p.gate = gate; p.skip = skip; p.w = norm_weight; p.d_skip = d_skip; p.dn = d_normed;
  p.dY = dY; p.dgate = d_gate; p.dskip_in = d_skip_input; p.d_d_skip = d_d_skip;
  p.d_w = d_norm_weight; p.gs = gate_row_stride; p.eps = eps;
  p.batch = batch; p.H = heads; p.T = T; p.P = P;
  const long long rows = (long long)batch * T;
  const unsigned grid = (unsigned)(rows < 148 * 2 ? rows : 148 * 2);   // two resident CTAs per SM
  const unsigned grid3 = (unsigned)(rows < 148 * 3 ? rows : 148 * 3);  // three for the one-piece kernel
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)heads * sizeof(float);
  SL_DISPATCH_DTYPE(io_dtype, Tt, {
    if (tail_vec_ok<Tt>(p)) {
      if ((long long)heads * P <= TAIL_THREADS * Vec16<Tt>::N) tail_bwd_row_kernel<Tt><<<grid3, TAIL_THREADS, 0, st>>>(p);
      else tail_bwd_vec_kernel<Tt, 2><<<grid, TAIL_THREADS, 0, st>>>(p);
    } else tail_bwd_kernel<Tt><<<grid, TAIL_THREADS, smem, st>>>(p);
  });
  note_launches(1);
  return launch_status();
}
