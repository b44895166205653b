// Exact float32 sequential v2x2ssd scan (forward and backward), SIMT.
//
// This is the path taken for float32 inputs (parity to 1e-5 needs float32
// products, which the tensor cores do not offer) and for shapes the tensor-core
// path does not cover.  It evaluates the recurrence token by token exactly as the
// sequential oracle does (reference: slinoss/ops/v2x2ssd/reference.py:815-840):
//
//   z_t = m_t z_{t-1} + u_{t-1} (x) (kp_t b_{t-1}) + u_t (x) (kc_t b_t)
//   y_t[p] = Re sum_n conj(c_t[n]) z_t[p,n]
//
// One CTA owns one (batch, head, 64-row slice of P).  A warp owns 32 rows of P
// (lane = row) and NPT complex columns of the state, kept in registers for the
// whole sequence.  Tokens are staged TB at a time in shared memory, already
// multiplied by their taps, so the inner loop is pure FMA on broadcast operands.
//
// Backward = two more sweeps of the same shape plus two small finishing kernels:
//   sweep A (forward in time)  recomputes z_t and emits dc_t[n] = sum_p dy_t[p] z_t[p,n]
//   sweep B (backward in time) carries G_t = dy_t (x) c_t + conj(m_{t+1}) G_{t+1} and
//           emits dbc_t = sum_p u_t G_t, dbp_t = sum_p u_{t-1} G_t, dU, d_initial
//   finish  dK, dB, dC (group sums), and dM from the identity
//           conj(m_t) dm_t = S_t,  S_t = S_{t+1} + <c_t,dc_t> - conj(kp_t)dkp_t - conj(kc_t)dkc_t,
//           S_T = <d_final, z_final>   (no state history is needed for dM).
#include <algorithm>

#include "common.cuh"

namespace sl {
namespace {

struct SweepParams {
  const void *U, *B, *C, *Bprev, *Uprev, *dY;
  const float *M, *K, *z0, *dfinal;
  void* Y;
  float* zfinal;
  float *dc_head, *dbc_head, *dbp_head;  // (batch, heads, T, 2N) float32
  float* sT;                             // (batch, heads, 2)  <d_final, z_final>
  void *dU, *dUprev;
  float* dinit;
  int batch, heads, groups, T, P, N;
  int NS, PW, TB, ptiles;
};

// Sum V per-lane values over the 32 lanes of a warp, scattering the results:
// V >= 32: lane holds columns lane*(V/32)+i in v[i], i < V/32;
// V == 16: every lane holds column (lane & 15) in v[0].
template <int V, int OFF, int LEN>
struct LaneReduce {
  static __device__ __forceinline__ void run(float (&v)[V], int lane) {
    if constexpr (OFF >= 1) {
      if constexpr (OFF >= V) {
#pragma unroll
        for (int i = 0; i < LEN; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], OFF);
        LaneReduce<V, OFF / 2, LEN>::run(v, lane);
      } else {
        constexpr int H = LEN / 2;
        const bool up = (lane & OFF) != 0;
#pragma unroll
        for (int i = 0; i < H; ++i) {
          const float send = up ? v[i] : v[i + H];
          const float keep = up ? v[i + H] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
        }
        LaneReduce<V, OFF / 2, H>::run(v, lane);
      }
    }
  }
};

template <int V>
__device__ __forceinline__ void lane_reduce_store(float (&v)[V], int lane, float* dst) {
  LaneReduce<V, 16, V>::run(v, lane);
  if constexpr (V >= 32) {
    constexpr int PER = V / 32;
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[lane * PER + i] = v[i];
  } else {
    if (lane < V) dst[lane] = v[0];
  }
}

template <typename T>
__device__ __forceinline__ cf load_c(const T* base, size_t cidx) {
  return {to_f32(base[2 * cidx]), to_f32(base[2 * cidx + 1])};
}

// MODE 0: forward (writes Y, final state).  MODE 1: backward sweep A (writes dc_head, sT).
template <typename TIn, typename TY, int NPT, int MODE>
__global__ void __launch_bounds__(512) sweep_fwd_kernel(SweepParams p) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int NS = p.NS, PW = p.PW, TB = p.TB;
  const int ns = w % NS, pw = w / NS;
  const int Npad = NS * NPT, D2 = 2 * Npad, PT = PW * 32, D = 2 * p.N;
  const int h = blockIdx.x, b = blockIdx.y, pt = blockIdx.z;
  const int g = h / (p.heads / p.groups);
  const int pl = pw * 32 + lane;      // row inside the CTA tile
  const int prow = pt * PT + pl;      // row of P
  const bool pvalid = prow < p.P;
  const int n0 = ns * NPT;
  const int T = p.T, N = p.N, P = p.P;

  float* s_bp = smem;
  float* s_bc = s_bp + TB * D2;
  float* s_c = s_bc + TB * D2;
  float* s_u = s_c + TB * D2;             // (TB+1) x PT
  float* s_m = s_u + (TB + 1) * PT;       // TB x 2
  float* s_dy = s_m + 2 * TB;             // TB x PT       (MODE 1)
  float* s_part = s_dy + TB * PT;         // MODE0: TB x NS x PT ; MODE1: TB x PW x D2

  const TIn* Ub = reinterpret_cast<const TIn*>(p.U) + ((size_t)(b * p.heads + h) * T) * P;
  const TIn* Bb = reinterpret_cast<const TIn*>(p.B) + ((size_t)(b * p.groups + g) * T) * D;
  const TIn* Cb = reinterpret_cast<const TIn*>(p.C) + ((size_t)(b * p.groups + g) * T) * D;
  const float* Mb = p.M + (size_t)(b * p.heads + h) * T * 2;
  const float* Kb = p.K + (size_t)(b * p.heads + h) * T * 4;
  const TIn* Bp = p.Bprev ? reinterpret_cast<const TIn*>(p.Bprev) + (size_t)(b * p.groups + g) * D
                          : nullptr;
  const TIn* Up = p.Uprev ? reinterpret_cast<const TIn*>(p.Uprev) + (size_t)(b * p.heads + h) * P
                          : nullptr;
  const TY* dYb = (MODE == 1 && p.dY)
                       ? reinterpret_cast<const TY*>(p.dY) + ((size_t)(b * p.heads + h) * T) * P
                       : nullptr;

  cf z[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    z[j] = {0.f, 0.f};
    if (p.z0 && pvalid && n0 + j < N) {
      const float* zp = p.z0 + ((size_t)(b * p.heads + h) * P + prow) * D + 2 * (n0 + j);
      z[j] = {zp[0], zp[1]};
    }
  }

  for (int t0 = 0; t0 < T; t0 += TB) {
    const int nb = min(TB, T - t0);
    for (int idx = tid; idx < nb * Npad; idx += blockDim.x) {
      const int tt = idx / Npad, n = idx - tt * Npad, t = t0 + tt;
      cf bt = {0.f, 0.f}, bpv = {0.f, 0.f}, ct = {0.f, 0.f};
      if (n < N) {
        bt = load_c(Bb + (size_t)t * D, n);
        if (MODE == 0) ct = load_c(Cb + (size_t)t * D, n);
        if (t > 0) bpv = load_c(Bb + (size_t)(t - 1) * D, n);
        else if (Bp) bpv = load_c(Bp, n);
      }
      const float4 k4 = *reinterpret_cast<const float4*>(Kb + (size_t)t * 4);
      const cf bp = cmul({k4.x, k4.y}, bpv), bc = cmul({k4.z, k4.w}, bt);
      s_bp[tt * D2 + 2 * n] = bp.re; s_bp[tt * D2 + 2 * n + 1] = bp.im;
      s_bc[tt * D2 + 2 * n] = bc.re; s_bc[tt * D2 + 2 * n + 1] = bc.im;
      if (MODE == 0) { s_c[tt * D2 + 2 * n] = ct.re; s_c[tt * D2 + 2 * n + 1] = ct.im; }
    }
    for (int idx = tid; idx < (nb + 1) * PT; idx += blockDim.x) {
      const int tt = idx / PT, pp = idx - tt * PT, t = t0 + tt - 1, pr = pt * PT + pp;
      float v = 0.f;
      if (pr < P) {
        if (t >= 0) v = to_f32(Ub[(size_t)t * P + pr]);
        else if (Up) v = to_f32(Up[pr]);
      }
      s_u[idx] = v;
    }
    if (MODE == 1) {
      for (int idx = tid; idx < nb * PT; idx += blockDim.x) {
        const int tt = idx / PT, pp = idx - tt * PT, pr = pt * PT + pp;
        s_dy[idx] = (pr < P && dYb) ? to_f32(dYb[(size_t)(t0 + tt) * P + pr]) : 0.f;
      }
    }
    for (int idx = tid; idx < 2 * nb; idx += blockDim.x) s_m[idx] = Mb[(size_t)t0 * 2 + idx];
    __syncthreads();

    for (int tt = 0; tt < nb; ++tt) {
      const float mr = s_m[2 * tt], mi = s_m[2 * tt + 1];
      const float up = s_u[tt * PT + pl], u = s_u[(tt + 1) * PT + pl];
      const float4* bp4 = reinterpret_cast<const float4*>(s_bp + tt * D2 + 2 * n0);
      const float4* bc4 = reinterpret_cast<const float4*>(s_bc + tt * D2 + 2 * n0);
      if (MODE == 0) {
        const float4* c4 = reinterpret_cast<const float4*>(s_c + tt * D2 + 2 * n0);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < NPT; j += 2) {
          const float4 a = bp4[j >> 1], c = bc4[j >> 1], q = c4[j >> 1];
          const float zr0 = mr * z[j].re - mi * z[j].im + up * a.x + u * c.x;
          const float zi0 = mr * z[j].im + mi * z[j].re + up * a.y + u * c.y;
          const float zr1 = mr * z[j + 1].re - mi * z[j + 1].im + up * a.z + u * c.z;
          const float zi1 = mr * z[j + 1].im + mi * z[j + 1].re + up * a.w + u * c.w;
          z[j] = {zr0, zi0};
          z[j + 1] = {zr1, zi1};
          acc += q.x * zr0 + q.y * zi0 + q.z * zr1 + q.w * zi1;
        }
        s_part[(tt * NS + ns) * PT + pl] = acc;
      } else {
        const float dy = s_dy[tt * PT + pl];
        float vals[2 * NPT];
#pragma unroll
        for (int j = 0; j < NPT; j += 2) {
          const float4 a = bp4[j >> 1], c = bc4[j >> 1];
          const float zr0 = mr * z[j].re - mi * z[j].im + up * a.x + u * c.x;
          const float zi0 = mr * z[j].im + mi * z[j].re + up * a.y + u * c.y;
          const float zr1 = mr * z[j + 1].re - mi * z[j + 1].im + up * a.z + u * c.z;
          const float zi1 = mr * z[j + 1].im + mi * z[j + 1].re + up * a.w + u * c.w;
          z[j] = {zr0, zi0};
          z[j + 1] = {zr1, zi1};
          vals[2 * j] = dy * zr0;
          vals[2 * j + 1] = dy * zi0;
          vals[2 * j + 2] = dy * zr1;
          vals[2 * j + 3] = dy * zi1;
        }
        lane_reduce_store<2 * NPT>(vals, lane, s_part + (tt * PW + pw) * D2 + 2 * n0);
      }
    }
    __syncthreads();

    if (MODE == 0) {
      TY* Yb = reinterpret_cast<TY*>(p.Y) + ((size_t)(b * p.heads + h) * T) * P;
      for (int idx = tid; idx < nb * PT; idx += blockDim.x) {
        const int tt = idx / PT, pp = idx - tt * PT, pr = pt * PT + pp;
        if (pr < P) {
          float s = 0.f;
          for (int k = 0; k < NS; ++k) s += s_part[(tt * NS + k) * PT + pp];
          Yb[(size_t)(t0 + tt) * P + pr] = from_f32<TY>(s);
        }
      }
    } else {
      float* dcb = p.dc_head + ((size_t)(b * p.heads + h) * T) * D;
      for (int idx = tid; idx < nb * D2; idx += blockDim.x) {
        const int tt = idx / D2, col = idx - tt * D2;
        if (col < D) {
          float s = 0.f;
          for (int k = 0; k < PW; ++k) s += s_part[(tt * PW + k) * D2 + col];
          float* dst = dcb + (size_t)(t0 + tt) * D + col;
          if (p.ptiles > 1) atomicAdd(dst, s); else *dst = s;
        }
      }
    }
    // the staging of the next block only rewrites arrays last read before the
    // second barrier; s_part is next written after the first barrier of that block.
  }

  if (MODE == 0) {
    if (p.zfinal && pvalid) {
#pragma unroll
      for (int j = 0; j < NPT; ++j)
        if (n0 + j < N) {
          float* zp = p.zfinal + ((size_t)(b * p.heads + h) * P + prow) * D + 2 * (n0 + j);
          zp[0] = z[j].re; zp[1] = z[j].im;
        }
    }
  } else {
    // S_T = sum d_final * conj(z_final)
    float sr = 0.f, si = 0.f;
    if (p.dfinal && pvalid) {
#pragma unroll
      for (int j = 0; j < NPT; ++j)
        if (n0 + j < N) {
          const float* dp = p.dfinal + ((size_t)(b * p.heads + h) * P + prow) * D + 2 * (n0 + j);
          sr += dp[0] * z[j].re + dp[1] * z[j].im;
          si += dp[1] * z[j].re - dp[0] * z[j].im;
        }
    }
    sr = warp_sum(sr); si = warp_sum(si);
    __syncthreads();
    if (lane == 0) { s_part[2 * w] = sr; s_part[2 * w + 1] = si; }
    __syncthreads();
    if (tid == 0) {
      float ar = 0.f, ai = 0.f;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) { ar += s_part[2 * k]; ai += s_part[2 * k + 1]; }
      float* dst = p.sT + (size_t)(b * p.heads + h) * 2;
      if (p.ptiles > 1) { atomicAdd(dst, ar); atomicAdd(dst + 1, ai); }
      else { dst[0] = ar; dst[1] = ai; }
    }
  }
}

// Backward sweep B: reverse in time.
template <typename TIn, typename TY, int NPT>
__global__ void __launch_bounds__(512) sweep_rev_kernel(SweepParams p) {
  extern __shared__ __align__(16) float smem[];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int NS = p.NS, PW = p.PW, TB = p.TB;
  const int ns = w % NS, pw = w / NS;
  const int Npad = NS * NPT, D2 = 2 * Npad, PT = PW * 32, D = 2 * p.N;
  const int h = blockIdx.x, b = blockIdx.y, pt = blockIdx.z;
  const int g = h / (p.heads / p.groups);
  const int pl = pw * 32 + lane, prow = pt * PT + pl;
  const bool pvalid = prow < p.P;
  const int n0 = ns * NPT;
  const int T = p.T, N = p.N, P = p.P;

  float* s_bp = smem;
  float* s_bc = s_bp + TB * D2;
  float* s_c = s_bc + TB * D2;
  float* s_u = s_c + TB * D2;              // (TB+1) x PT
  float* s_mn = s_u + (TB + 1) * PT;       // TB x 2 : m_{t+1}
  float* s_dy = s_mn + 2 * TB;             // TB x PT
  float* s_pc = s_dy + TB * PT;            // TB x PW x D2
  float* s_pp = s_pc + TB * PW * D2;       // TB x PW x D2
  float* s_duc = s_pp + TB * PW * D2;      // TB x NS x PT
  float* s_dup = s_duc + TB * NS * PT;     // TB x NS x PT
  float* s_carry = s_dup + TB * NS * PT;   // PT

  const TIn* Ub = reinterpret_cast<const TIn*>(p.U) + ((size_t)(b * p.heads + h) * T) * P;
  const TIn* Bb = reinterpret_cast<const TIn*>(p.B) + ((size_t)(b * p.groups + g) * T) * D;
  const TIn* Cb = reinterpret_cast<const TIn*>(p.C) + ((size_t)(b * p.groups + g) * T) * D;
  const float* Mb = p.M + (size_t)(b * p.heads + h) * T * 2;
  const float* Kb = p.K + (size_t)(b * p.heads + h) * T * 4;
  const TIn* Bp = p.Bprev ? reinterpret_cast<const TIn*>(p.Bprev) + (size_t)(b * p.groups + g) * D
                          : nullptr;
  const TIn* Up = p.Uprev ? reinterpret_cast<const TIn*>(p.Uprev) + (size_t)(b * p.heads + h) * P
                          : nullptr;
  const TY* dYb = p.dY ? reinterpret_cast<const TY*>(p.dY) + ((size_t)(b * p.heads + h) * T) * P
                       : nullptr;
  TIn* dUb = reinterpret_cast<TIn*>(p.dU) + ((size_t)(b * p.heads + h) * T) * P;
  float* dbcb = p.dbc_head + ((size_t)(b * p.heads + h) * T) * D;
  float* dbpb = p.dbp_head + ((size_t)(b * p.heads + h) * T) * D;

  cf G[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    G[j] = {0.f, 0.f};
    if (p.dfinal && pvalid && n0 + j < N) {
      const float* gp = p.dfinal + ((size_t)(b * p.heads + h) * P + prow) * D + 2 * (n0 + j);
      G[j] = {gp[0], gp[1]};
    }
  }
  for (int idx = tid; idx < PT; idx += blockDim.x) s_carry[idx] = 0.f;

  for (int t0 = ((T - 1) / TB) * TB; t0 >= 0; t0 -= TB) {
    const int nb = min(TB, T - t0);
    for (int idx = tid; idx < nb * Npad; idx += blockDim.x) {
      const int tt = idx / Npad, n = idx - tt * Npad, t = t0 + tt;
      cf bt = {0.f, 0.f}, bpv = {0.f, 0.f}, ct = {0.f, 0.f};
      if (n < N) {
        bt = load_c(Bb + (size_t)t * D, n);
        ct = load_c(Cb + (size_t)t * D, n);
        if (t > 0) bpv = load_c(Bb + (size_t)(t - 1) * D, n);
        else if (Bp) bpv = load_c(Bp, n);
      }
      const float4 k4 = *reinterpret_cast<const float4*>(Kb + (size_t)t * 4);
      const cf bp = cmul({k4.x, k4.y}, bpv), bc = cmul({k4.z, k4.w}, bt);
      s_bp[tt * D2 + 2 * n] = bp.re; s_bp[tt * D2 + 2 * n + 1] = bp.im;
      s_bc[tt * D2 + 2 * n] = bc.re; s_bc[tt * D2 + 2 * n + 1] = bc.im;
      s_c[tt * D2 + 2 * n] = ct.re; s_c[tt * D2 + 2 * n + 1] = ct.im;
    }
    for (int idx = tid; idx < (nb + 1) * PT; idx += blockDim.x) {
      const int tt = idx / PT, pp = idx - tt * PT, t = t0 + tt - 1, pr = pt * PT + pp;
      float v = 0.f;
      if (pr < P) {
        if (t >= 0) v = to_f32(Ub[(size_t)t * P + pr]);
        else if (Up) v = to_f32(Up[pr]);
      }
      s_u[idx] = v;
    }
    for (int idx = tid; idx < nb * PT; idx += blockDim.x) {
      const int tt = idx / PT, pp = idx - tt * PT, pr = pt * PT + pp;
      s_dy[idx] = (pr < P && dYb) ? to_f32(dYb[(size_t)(t0 + tt) * P + pr]) : 0.f;
    }
    for (int idx = tid; idx < nb; idx += blockDim.x) {
      const int t = t0 + idx + 1;
      s_mn[2 * idx] = t < T ? Mb[(size_t)t * 2] : 1.f;
      s_mn[2 * idx + 1] = t < T ? Mb[(size_t)t * 2 + 1] : 0.f;
    }
    __syncthreads();

    for (int tt = nb - 1; tt >= 0; --tt) {
      const float mr = s_mn[2 * tt], mi = s_mn[2 * tt + 1];
      const float dy = s_dy[tt * PT + pl];
      const float up = s_u[tt * PT + pl], u = s_u[(tt + 1) * PT + pl];
      const float2* bp2 = reinterpret_cast<const float2*>(s_bp + tt * D2 + 2 * n0);
      const float2* bc2 = reinterpret_cast<const float2*>(s_bc + tt * D2 + 2 * n0);
      const float2* c2 = reinterpret_cast<const float2*>(s_c + tt * D2 + 2 * n0);
      float duc = 0.f, dup = 0.f;
      float vals[2 * NPT];
#pragma unroll
      for (int j = 0; j < NPT; ++j) {
        const float2 a = bp2[j], c = bc2[j], q = c2[j];
        // G = conj(m_{t+1}) G + dy * c_t
        const float gr = mr * G[j].re + mi * G[j].im + dy * q.x;
        const float gi = mr * G[j].im - mi * G[j].re + dy * q.y;
        G[j] = {gr, gi};
        duc += c.x * gr + c.y * gi;
        dup += a.x * gr + a.y * gi;
        vals[2 * j] = u * gr;
        vals[2 * j + 1] = u * gi;
      }
      lane_reduce_store<2 * NPT>(vals, lane, s_pc + (tt * PW + pw) * D2 + 2 * n0);
#pragma unroll
      for (int j = 0; j < NPT; ++j) {
        vals[2 * j] = up * G[j].re;
        vals[2 * j + 1] = up * G[j].im;
      }
      lane_reduce_store<2 * NPT>(vals, lane, s_pp + (tt * PW + pw) * D2 + 2 * n0);
      s_duc[(tt * NS + ns) * PT + pl] = duc;
      s_dup[(tt * NS + ns) * PT + pl] = dup;
    }
    __syncthreads();

    for (int idx = tid; idx < nb * D2; idx += blockDim.x) {
      const int tt = idx / D2, col = idx - tt * D2;
      if (col < D) {
        float sc = 0.f, sp = 0.f;
        for (int k = 0; k < PW; ++k) {
          sc += s_pc[(tt * PW + k) * D2 + col];
          sp += s_pp[(tt * PW + k) * D2 + col];
        }
        const size_t o = (size_t)(t0 + tt) * D + col;
        if (p.ptiles > 1) { atomicAdd(dbcb + o, sc); atomicAdd(dbpb + o, sp); }
        else { dbcb[o] = sc; dbpb[o] = sp; }
      }
    }
    for (int pp = tid; pp < PT; pp += blockDim.x) {
      const int pr = pt * PT + pp;
      float prevp = s_carry[pp];
      for (int tt = nb - 1; tt >= 0; --tt) {
        float sc = 0.f, sp = 0.f;
        for (int k = 0; k < NS; ++k) {
          sc += s_duc[(tt * NS + k) * PT + pp];
          sp += s_dup[(tt * NS + k) * PT + pp];
        }
        if (pr < P) dUb[(size_t)(t0 + tt) * P + pr] = from_f32<TIn>(sc + prevp);
        prevp = sp;
      }
      s_carry[pp] = prevp;
    }
    // next block's staging is separated from these reads by its first barrier
    // only for s_pc/s_pp/s_duc/s_dup (written after that barrier); s_carry is
    // private to thread pp.  The staging arrays were last read before the
    // second barrier above.
  }
  __syncthreads();
  if (p.dUprev) {
    TIn* dUp = reinterpret_cast<TIn*>(p.dUprev) + (size_t)(b * p.heads + h) * P;
    for (int pp = tid; pp < PT; pp += blockDim.x)
      if (pt * PT + pp < P) dUp[pt * PT + pp] = from_f32<TIn>(s_carry[pp]);
  }
  if (p.dinit && pvalid) {
    const float mr = Mb[0], mi = Mb[1];
#pragma unroll
    for (int j = 0; j < NPT; ++j)
      if (n0 + j < N) {
        float* dp = p.dinit + ((size_t)(b * p.heads + h) * P + prow) * D + 2 * (n0 + j);
        dp[0] = mr * G[j].re + mi * G[j].im;
        dp[1] = mr * G[j].im - mi * G[j].re;
      }
  }
}

// One warp per (batch, group, t): dK and the dM scan terms per head, dB / dC summed
// over the heads of the group.
struct FinishParams {
  const void *B, *C, *Bprev;
  const float *K, *dc_head, *dbc_head, *dbp_head;
  float *dK, *sterm;
  void *dB, *dC, *dBprev;
  int batch, heads, groups, T, N;
};

template <typename TIn>
__global__ void __launch_bounds__(256) bwd_finish_kernel(FinishParams p) {
  constexpr int MAXN = 4;  // N <= 128
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)p.batch * p.groups * p.T;
  if (row >= rows) return;
  const int t = (int)(row % p.T);
  const int bg = (int)(row / p.T);
  const int g = bg % p.groups, b = bg / p.groups;
  const int hpg = p.heads / p.groups, N = p.N, D = 2 * N, T = p.T;
  const TIn* Bb = reinterpret_cast<const TIn*>(p.B) + ((size_t)bg * T) * D;
  const TIn* Cb = reinterpret_cast<const TIn*>(p.C) + ((size_t)bg * T) * D;
  const TIn* Bp = p.Bprev ? reinterpret_cast<const TIn*>(p.Bprev) + (size_t)bg * D : nullptr;

  cf bt[MAXN], bprev[MAXN], ct[MAXN], db[MAXN], dc[MAXN], dbp0[MAXN];
#pragma unroll
  for (int i = 0; i < MAXN; ++i) {
    const int n = lane + 32 * i;
    bt[i] = bprev[i] = ct[i] = db[i] = dc[i] = dbp0[i] = {0.f, 0.f};
    if (n < N) {
      bt[i] = load_c(Bb + (size_t)t * D, n);
      ct[i] = load_c(Cb + (size_t)t * D, n);
      if (t > 0) bprev[i] = load_c(Bb + (size_t)(t - 1) * D, n);
      else if (Bp) bprev[i] = load_c(Bp, n);
    }
  }
  for (int hh = 0; hh < hpg; ++hh) {
    const int h = g * hpg + hh;
    const size_t bh = (size_t)b * p.heads + h;
    const float* Kt = p.K + (bh * T + t) * 4;
    const cf kp = {Kt[0], Kt[1]}, kc = {Kt[2], Kt[3]};
    cf kpn = {0.f, 0.f};
    if (t + 1 < T) kpn = {Kt[4], Kt[5]};
    const float* dch = p.dc_head + (bh * T + t) * D;
    const float* dbch = p.dbc_head + (bh * T + t) * D;
    const float* dbph = p.dbp_head + (bh * T + t) * D;
    float kcr = 0.f, kci = 0.f, kpr = 0.f, kpi = 0.f, sr = 0.f, si = 0.f;
#pragma unroll
    for (int i = 0; i < MAXN; ++i) {
      const int n = lane + 32 * i;
      if (n < N) {
        const cf vdc = {dch[2 * n], dch[2 * n + 1]};
        const cf vbc = {dbch[2 * n], dbch[2 * n + 1]};
        const cf vbp = {dbph[2 * n], dbph[2 * n + 1]};
        // dkc += dbc * conj(b_t); dkp += dbp * conj(b_{t-1}); s += c_t * conj(dc_t)
        kcr += vbc.re * bt[i].re + vbc.im * bt[i].im;
        kci += vbc.im * bt[i].re - vbc.re * bt[i].im;
        kpr += vbp.re * bprev[i].re + vbp.im * bprev[i].im;
        kpi += vbp.im * bprev[i].re - vbp.re * bprev[i].im;
        sr += ct[i].re * vdc.re + ct[i].im * vdc.im;
        si += ct[i].im * vdc.re - ct[i].re * vdc.im;
        db[i] = cadd(db[i], cmul_conj_a(kc, vbc));
        if (t + 1 < T) {
          const cf vbpn = {dbph[D + 2 * n], dbph[D + 2 * n + 1]};
          db[i] = cadd(db[i], cmul_conj_a(kpn, vbpn));
        }
        dc[i] = cadd(dc[i], vdc);
        if (t == 0) dbp0[i] = cadd(dbp0[i], cmul_conj_a(kp, vbp));
      }
    }
    kcr = warp_sum(kcr); kci = warp_sum(kci); kpr = warp_sum(kpr); kpi = warp_sum(kpi);
    sr = warp_sum(sr); si = warp_sum(si);
    if (lane == 0) {
      float* dKt = p.dK + (bh * T + t) * 4;
      dKt[0] = kpr; dKt[1] = kpi; dKt[2] = kcr; dKt[3] = kci;
      // s_t = <c,dc> - conj(kp) dkp - conj(kc) dkc
      const cf a = cmul_conj_a(kp, {kpr, kpi}), c2 = cmul_conj_a(kc, {kcr, kci});
      float* st = p.sterm + (bh * T + t) * 2;
      st[0] = sr - a.re - c2.re;
      st[1] = si - a.im - c2.im;
    }
  }
  TIn* dBo = reinterpret_cast<TIn*>(p.dB) + ((size_t)bg * T + t) * D;
  TIn* dCo = reinterpret_cast<TIn*>(p.dC) + ((size_t)bg * T + t) * D;
#pragma unroll
  for (int i = 0; i < MAXN; ++i) {
    const int n = lane + 32 * i;
    if (n < N) {
      dBo[2 * n] = from_f32<TIn>(db[i].re); dBo[2 * n + 1] = from_f32<TIn>(db[i].im);
      dCo[2 * n] = from_f32<TIn>(dc[i].re); dCo[2 * n + 1] = from_f32<TIn>(dc[i].im);
      if (t == 0 && p.dBprev) {
        TIn* o = reinterpret_cast<TIn*>(p.dBprev) + (size_t)bg * D;
        o[2 * n] = from_f32<TIn>(dbp0[i].re); o[2 * n + 1] = from_f32<TIn>(dbp0[i].im);
      }
    }
  }
}

// One CTA per (batch, head): S_t = S_T + sum_{s >= t} sterm_s ; dM_t = S_t / conj(m_t).
__global__ void __launch_bounds__(256) bwd_dm_scan_kernel(const float* __restrict__ sterm,
                                                          const float* __restrict__ sT,
                                                          const float* __restrict__ M,
                                                          float* __restrict__ dM, int T) {
  __shared__ double s_wr[8], s_wi[8];
  __shared__ double s_carry[2];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const size_t bh = blockIdx.x;
  const float* st = sterm + bh * T * 2;
  const float* Mb = M + bh * T * 2;
  float* dMb = dM + bh * T * 2;
  if (tid == 0) { s_carry[0] = sT[bh * 2]; s_carry[1] = sT[bh * 2 + 1]; }
  __syncthreads();
  for (int hi = T; hi > 0; hi -= 256) {
    const int t = hi - 1 - tid;  // thread 0 owns the latest token of the tile
    double vr = 0.0, vi = 0.0;
    if (t >= 0) { vr = st[2 * t]; vi = st[2 * t + 1]; }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double ar = __shfl_up_sync(0xffffffffu, vr, o), ai = __shfl_up_sync(0xffffffffu, vi, o);
      if (lane >= o) { vr += ar; vi += ai; }
    }
    if (lane == 31) { s_wr[w] = vr; s_wi[w] = vi; }
    __syncthreads();
    double offr = s_carry[0], offi = s_carry[1];
    for (int k = 0; k < w; ++k) { offr += s_wr[k]; offi += s_wi[k]; }
    vr += offr; vi += offi;
    if (t >= 0) {
      const float mr = Mb[2 * t], mi = Mb[2 * t + 1];
      const float den = mr * mr + mi * mi;
      // S / conj(m) = S * m / |m|^2
      float outr = 0.f, outi = 0.f;
      if (den > 0.f) {
        outr = (float)((vr * mr - vi * mi) / den);
        outi = (float)((vr * mi + vi * mr) / den);
      }
      dMb[2 * t] = outr; dMb[2 * t + 1] = outi;
    }
    __syncthreads();
    if (tid == 255) { s_carry[0] = vr; s_carry[1] = vi; }
    __syncthreads();
  }
}

struct SimtConfig {
  int NPT, NS, PW, ptiles, TB, threads;
  size_t smem_fwd, smem_rev;
};

bool make_config(const ScanDims& d, SimtConfig& c) {
  if (d.N < 1 || d.N > 128 || d.P < 1) return false;
  c.NPT = d.N <= 32 ? 8 : 16;
  c.NS = (d.N + c.NPT - 1) / c.NPT;
  c.PW = d.P > 32 ? 2 : 1;
  const int PT = 32 * c.PW;
  c.ptiles = (d.P + PT - 1) / PT;
  c.threads = 32 * c.NS * c.PW;
  const int D2 = 2 * c.NS * c.NPT;
  for (c.TB = 16; c.TB >= 4; c.TB /= 2) {
    const size_t TB = c.TB;
    const size_t part_fwd = TB * (size_t)std::max(c.NS * PT, c.PW * D2);
    c.smem_fwd = 4 * (3 * TB * D2 + (TB + 1) * PT + 2 * TB + TB * PT + part_fwd);
    c.smem_rev = 4 * (3 * TB * D2 + (TB + 1) * PT + 2 * TB + TB * PT + 2 * TB * c.PW * D2 +
                      2 * TB * c.NS * PT + PT);
    if (c.smem_rev <= 200 * 1024) return true;
  }
  return false;
}

template <typename F>
int set_smem(F f, size_t bytes) {
  return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) ==
                 cudaSuccess
             ? SL_OK
             : SL_ERR_LAUNCH_FAILED;
}

SweepParams base_params(const void* U, const float* M, const float* K, const void* B,
                        const void* C, const float* z0, const void* Bprev, const void* Uprev,
                        const ScanDims& d, const SimtConfig& c) {
  SweepParams p{};
  p.U = U; p.B = B; p.C = C; p.Bprev = Bprev; p.Uprev = Uprev; p.M = M; p.K = K; p.z0 = z0;
  p.batch = d.batch; p.heads = d.heads; p.groups = d.groups; p.T = d.T; p.P = d.P; p.N = d.N;
  p.NS = c.NS; p.PW = c.PW; p.TB = c.TB; p.ptiles = c.ptiles;
  return p;
}

template <typename TIn, typename TY, int NPT>
int launch_fwd(const SweepParams& p, const SimtConfig& c, cudaStream_t st) {
  auto k = sweep_fwd_kernel<TIn, TY, NPT, 0>;
  if (int e = set_smem(k, c.smem_fwd)) return e;
  dim3 grid(p.heads, p.batch, c.ptiles);
  k<<<grid, c.threads, c.smem_fwd, st>>>(p);
  note_launches(1);
  return launch_status();
}

template <typename TIn, typename TY, int NPT>
int launch_bwd(const SweepParams& p, const SimtConfig& c, cudaStream_t st) {
  auto ka = sweep_fwd_kernel<TIn, TY, NPT, 1>;
  auto kb = sweep_rev_kernel<TIn, TY, NPT>;
  if (int e = set_smem(ka, c.smem_fwd)) return e;
  if (int e = set_smem(kb, c.smem_rev)) return e;
  dim3 grid(p.heads, p.batch, c.ptiles);
  ka<<<grid, c.threads, c.smem_fwd, st>>>(p);
  kb<<<grid, c.threads, c.smem_rev, st>>>(p);
  note_launches(2);
  return launch_status();
}

}  // namespace

bool scan_simt_supported(const ScanDims& d) {
  SimtConfig c;
  return make_config(d, c);
}

int scan_simt_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                  const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                  const ScanDims& d, int io_dtype, int y_dtype, cudaStream_t st) {
  SimtConfig c;
  if (!make_config(d, c)) return SL_ERR_UNSUPPORTED;
  SweepParams p = base_params(U, M, K, B, C, z0, Bprev, Uprev, d, c);
  p.Y = Y; p.zfinal = zfinal;
  int rc = SL_ERR_UNSUPPORTED;
  SL_DISPATCH_DTYPE(io_dtype, TIn, SL_DISPATCH_DTYPE(y_dtype, TY, {
    rc = c.NPT == 8 ? launch_fwd<TIn, TY, 8>(p, c, st) : launch_fwd<TIn, TY, 16>(p, c, st);
  }));
  return rc;
}

// workspace layout: dc_head | dbc_head | dbp_head (each batch*heads*T*2N floats) |
//                   sterm (batch*heads*T*2) | sT (batch*heads*2)
size_t scan_simt_bwd_workspace(const ScanDims& d) {
  const size_t bht = (size_t)d.batch * d.heads * d.T;
  return round_up(4 * (3 * bht * 2 * d.N + bht * 2 + (size_t)d.batch * d.heads * 2), 256);
}

int scan_simt_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                  const float* z0, const void* Bprev, const void* Uprev, const void* dY,
                  const float* dfinal, void* dU, float* dM, float* dK, void* dB, void* dC,
                  float* dinit, void* dBprev, void* dUprev, const ScanDims& d, int io_dtype,
                  int dy_dtype, void* ws, size_t ws_bytes, cudaStream_t st) {
  SimtConfig c;
  if (!make_config(d, c)) return SL_ERR_UNSUPPORTED;
  const size_t need = scan_simt_bwd_workspace(d);
  if (!ws || ws_bytes < need) return SL_ERR_WORKSPACE_TOO_SMALL;
  const size_t bht = (size_t)d.batch * d.heads * d.T, D = 2 * (size_t)d.N;
  float* dc_head = reinterpret_cast<float*>(ws);
  float* dbc_head = dc_head + bht * D;
  float* dbp_head = dbc_head + bht * D;
  float* sterm = dbp_head + bht * D;
  float* sT = sterm + bht * 2;
  if (c.ptiles > 1) {  // partial sums of the P tiles are accumulated atomically
    if (cudaMemsetAsync(ws, 0, need, st) != cudaSuccess) return SL_ERR_LAUNCH_FAILED;
  }
  SweepParams p = base_params(U, M, K, B, C, z0, Bprev, Uprev, d, c);
  p.dY = dY; p.dfinal = dfinal; p.dc_head = dc_head; p.dbc_head = dbc_head;
  p.dbp_head = dbp_head; p.sT = sT; p.dU = dU; p.dUprev = dUprev; p.dinit = dinit;
  int rc = SL_ERR_UNSUPPORTED;
  SL_DISPATCH_DTYPE(io_dtype, TIn, SL_DISPATCH_DTYPE(dy_dtype, TY, {
    rc = c.NPT == 8 ? launch_bwd<TIn, TY, 8>(p, c, st) : launch_bwd<TIn, TY, 16>(p, c, st);
  }));
  if (rc != SL_OK) return rc;
  FinishParams f{};
  f.B = B; f.C = C; f.Bprev = Bprev; f.K = K; f.dc_head = dc_head; f.dbc_head = dbc_head;
  f.dbp_head = dbp_head; f.dK = dK; f.sterm = sterm; f.dB = dB; f.dC = dC; f.dBprev = dBprev;
  f.batch = d.batch; f.heads = d.heads; f.groups = d.groups; f.T = d.T; f.N = d.N;
  const long long rows = (long long)d.batch * d.groups * d.T;
  const unsigned blocks = (unsigned)((rows + 7) / 8);
  SL_DISPATCH_DTYPE(io_dtype, TIn, { bwd_finish_kernel<TIn><<<blocks, 256, 0, st>>>(f); });
  bwd_dm_scan_kernel<<<d.batch * d.heads, 256, 0, st>>>(sterm, sT, M, dM, d.T);
  note_launches(2);
  return launch_status();
}

}  // namespace sl
