// Chunked v2x2ssd scan on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Supported: P = 64, N = 64 (D = 2N = 128), bf16 or fp16 operands, float32 state.
// Everything else takes the exact SIMT path.
//
// Formulation (per (batch, head); chunk of L = 64 tokens, local index t, s).  The two
// taps are merged into one source coefficient with a one-token look-ahead,
//     g_s = kc_s + kp_{s+1} / m_{s+1},
// and the carried state is W = z + u (x) (kp_next / m_next) b, which obeys the
// single-tap recurrence  W_s = m_s W_{s-1} + u_s (x) (g_s b_s)  with
//     y_t = Re<c_t, W_t> - u_t Re(conj(c_t) (g_t - kc_t) b_t).
// With the in-chunk prefix  Pi_t = prod_{s<=t} m_s = exp(l_t) phi_t  (l = cumulative
// log|m|, |phi| = 1) the chunk is four real GEMMs over the interleaved (re, im) lanes:
//     Q_t   = conj(c_t) phi_t                       (unit rotation of C, in place)
//     K'_s  = conj(phi_s) g_s b_s                   (in place over B, stored conjugated)
//     S     = mask_{s<t}( (Q K'^T) * exp(l_t - l_s) ),  S_tt = Re(conj(c_t) kc_t b_t)
//     Y     = S U + exp(l_t) * (Q Zv^T)             (Zv = conj of the chunk-start state)
//     Zv'   = conj(Pi_end) Zv + U^T K''             (K''_s = exp(l_end - l_s) phi_end K'_s)
// Magnitudes only ever enter as exp(non-positive), exactly like the reference's
// chunk_scan policy (slinoss/ops/v2x2ssd/reference.py:498-523, 1224-1261); phases are
// applied to the 16-bit operands, decays to float32 accumulators.
//
// One CTA (128 threads) walks the chunks of one (batch, head) in order.  U/B/C tiles
// arrive by TMA (128B swizzle, one chunk ahead), the state lives in registers (float32,
// 64 per thread), the MMAs use M = 64 accumulators split into two column halves that
// sit in the two 16-lane halves of every TMEM lane quadrant, so that thread
// (warp j, lane i) owns row 16j + (i & 15) and column half (i >> 4) of every result.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "tc_common.cuh"

namespace sl {
namespace {

using namespace tc;

constexpr int L = 64;
constexpr uint32_t TILE = 8192;           // one [64][128 B] tile
constexpr uint32_t STAGE = 5 * TILE;      // U | B(2) | C(2)
constexpr uint32_t OFF_KPP = 2 * STAGE;   // K'' (2 tiles)
constexpr uint32_t OFF_S = OFF_KPP + 2 * TILE;
constexpr uint32_t OFF_ZV = OFF_S + TILE; // Zv (2 tiles)
constexpr uint32_t OFF_SCAL = OFF_ZV + 2 * TILE;
constexpr int NSCAL = 12;                 // per-token float arrays
constexpr uint32_t SMEM_BYTES = OFF_SCAL + NSCAL * 64 * 4 + 64 + 1024;
constexpr uint32_t TMEM_COLS = 256;       // S 0..31 | Yoff 32..63 | Ydiag 64..95 | Inc 128..191

__device__ int g_tc_status = 0;           // first device-side error (bounded wait expired)

struct alignas(64) TcFwdParams {
  CUtensorMap tmU, tmB, tmC;
  const float* M;
  const float* K;
  const float* z0;
  const void* Bprev;
  const void* Uprev;
  void* Y;
  float* zfinal;
  void* states16;       // optional (batch*heads, nchunks, 64, 128) 16-bit: conjugated start state of every chunk
  int heads, groups, T, nchunks;
};

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static constexpr int fmt = 1;
};
template <> struct Pack2<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static constexpr int fmt = 0;
};

__device__ __forceinline__ void report_timeout(int code) { atomicCAS(&g_tc_status, 0, code); }

// Per-chunk scalars, computed by warp 0 (two tokens per lane) with shuffle scans.
//  sc[0] l_t        sc[1] exp(l_t)     sc[2],sc[3] phi_t
//  sc[4],sc[5] w_t = conj(phi_t) g_t                (K'  = w b)
//  sc[6],sc[7] v_t = exp(l_end - l_t) phi_end w_t   (K'' = v b)
//  sc[8],sc[9] kc_t                                 (diagonal)
//  chunk-level: sc[10][0..1] = Pi_end, sc[10][2..3] = its unit phase
__device__ void chunk_scalars(float* sc, const float* __restrict__ Mb, const float* __restrict__ Kb,
                              int t0, int T, int lane) {
  float mr[3], mi[3], kpr[3], kpi[3], kcr[2], kci[2];
#pragma unroll
  for (int q = 0; q < 3; ++q) {
    const int t = t0 + 2 * lane + q;
    mr[q] = 1.f; mi[q] = 0.f; kpr[q] = 0.f; kpi[q] = 0.f;
    if (t < T) {
      const float2 m = *reinterpret_cast<const float2*>(Mb + 2 * (size_t)t);
      const float4 k = *reinterpret_cast<const float4*>(Kb + 4 * (size_t)t);
      mr[q] = m.x; mi[q] = m.y; kpr[q] = k.x; kpi[q] = k.y;
      if (q < 2) { kcr[q] = k.z; kci[q] = k.w; }
    } else if (q < 2) {
      kcr[q] = 0.f; kci[q] = 0.f;
    }
  }
  // local prefixes over the lane's two tokens
  const float mag0 = sqrtf(mr[0] * mr[0] + mi[0] * mi[0]);
  const float mag1 = sqrtf(mr[1] * mr[1] + mi[1] * mi[1]);
  const float a0 = __logf(mag0), a1 = __logf(mag1);
  const float u0r = mr[0] / mag0, u0i = mi[0] / mag0, u1r = mr[1] / mag1, u1i = mi[1] / mag1;
  float lsum = a0 + a1;                       // inclusive scan of log-magnitudes
  float pr = u0r * u1r - u0i * u1i, pi = u0r * u1i + u0i * u1r;  // and of unit phases
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float ol = __shfl_up_sync(0xffffffffu, lsum, o);
    const float opr = __shfl_up_sync(0xffffffffu, pr, o), opi = __shfl_up_sync(0xffffffffu, pi, o);
    if (lane >= o) {
      lsum += ol;
      const float nr = pr * opr - pi * opi, ni = pr * opi + pi * opr;
      pr = nr; pi = ni;
    }
  }
  float el = __shfl_up_sync(0xffffffffu, lsum, 1);
  float epr = __shfl_up_sync(0xffffffffu, pr, 1), epi = __shfl_up_sync(0xffffffffu, pi, 1);
  if (lane == 0) { el = 0.f; epr = 1.f; epi = 0.f; }
  const float l_end = __shfl_sync(0xffffffffu, lsum, 31);
  float per = __shfl_sync(0xffffffffu, pr, 31), pei = __shfl_sync(0xffffffffu, pi, 31);
  { const float n = rsqrtf(per * per + pei * pei); per *= n; pei *= n; }
  float lt[2], phr[2], phi[2];
  lt[0] = el + a0; lt[1] = el + a0 + a1;
  phr[0] = epr * u0r - epi * u0i; phi[0] = epr * u0i + epi * u0r;
  phr[1] = phr[0] * u1r - phi[0] * u1i; phi[1] = phr[0] * u1i + phi[0] * u1r;
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const float n = rsqrtf(phr[q] * phr[q] + phi[q] * phi[q]);
    phr[q] *= n; phi[q] *= n;
    // g = kc + kp_next / m_next
    const float den = mr[q + 1] * mr[q + 1] + mi[q + 1] * mi[q + 1];
    const float gr = kcr[q] + (kpr[q + 1] * mr[q + 1] + kpi[q + 1] * mi[q + 1]) / den;
    const float gi = kci[q] + (kpi[q + 1] * mr[q + 1] - kpr[q + 1] * mi[q + 1]) / den;
    const float wr = phr[q] * gr + phi[q] * gi, wi = phr[q] * gi - phi[q] * gr;  // conj(phi) g
    const float e = __expf(l_end - lt[q]);
    const float vr = e * (per * wr - pei * wi), vi = e * (per * wi + pei * wr);
    const int i = 2 * lane + q;
    sc[0 * 64 + i] = lt[q];
    sc[1 * 64 + i] = __expf(lt[q]);
    sc[2 * 64 + i] = phr[q]; sc[3 * 64 + i] = phi[q];
    sc[4 * 64 + i] = wr; sc[5 * 64 + i] = wi;
    sc[6 * 64 + i] = vr; sc[7 * 64 + i] = vi;
    sc[8 * 64 + i] = kcr[q]; sc[9 * 64 + i] = kci[q];
  }
  if (lane == 0) {
    const float e = __expf(l_end);
    sc[10 * 64 + 0] = e * per; sc[10 * 64 + 1] = e * pei;
    sc[10 * 64 + 2] = per; sc[10 * 64 + 3] = pei;   // unit phase of Pi_end
  }
}

// STATES_ONLY: the state pre-sweep of the backward pass (no C, no scores, no Y).
template <typename TIn, typename TY, bool STATES_ONLY>
__global__ void __launch_bounds__(128, 1) scan_tc_fwd_kernel(const __grid_constant__ TcFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar_tma[2], bar_mma[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  float* sc = reinterpret_cast<float*>(smem + OFF_SCAL);
  float* s_diag = sc + 11 * 64;
  using PK = Pack2<TIn>;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = 16 * warp + (lane & 15), hf = lane >> 4;   // epilogue identity
  const int rcol = tid & 15, rrow0 = tid >> 4;               // rotation identity
  const int bh = blockIdx.x, b = bh / p.heads, h = bh % p.heads;
  const int bg = b * p.groups + h / (p.heads / p.groups);
  const int T = p.T;
  const float* Mb = p.M + (size_t)bh * T * 2;
  const float* Kb = p.K + (size_t)bh * T * 4;

  if (tid == 0) {
    mbar_init(&bar_tma[0], 1); mbar_init(&bar_tma[1], 1);
    mbar_init(&bar_mma[0], 1); mbar_init(&bar_mma[1], 1);
    fence_barrier_init();
    s_abort = 0;
    tma_prefetch_desc(&p.tmU); tma_prefetch_desc(&p.tmB); tma_prefetch_desc(&p.tmC);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  auto issue_loads = [&](int c) {   // one thread
    uint8_t* st = smem + (c & 1) * STAGE;
    uint64_t* bar = &bar_tma[c & 1];
    mbar_expect_tx(bar, STATES_ONLY ? 3 * TILE : STAGE);
    tma_load_3d(st, &p.tmU, bar, 0, c * L, bh);
    tma_load_3d(st + TILE, &p.tmB, bar, 0, c * L, bg);
    tma_load_3d(st + 2 * TILE, &p.tmB, bar, 64, c * L, bg);
    if (!STATES_ONLY) {
      tma_load_3d(st + 3 * TILE, &p.tmC, bar, 0, c * L, bg);
      tma_load_3d(st + 4 * TILE, &p.tmC, bar, 64, c * L, bg);
    }
  };
  if (tid == 0) issue_loads(0);

  // ---- carried state in conjugated form: zv[2j], zv[2j+1] = (re, -im) of column pair j ------
  float zv[64];
  {
    const TIn* Bp = reinterpret_cast<const TIn*>(p.Bprev);
    const TIn* Up = reinterpret_cast<const TIn*>(p.Uprev);
    float cr = 0.f, ci = 0.f, up = 0.f;
    if (Bp) {  // pending prev-tap of the token before the sequence: u_prev (x) (kp_0 / m_0) b_prev
      const float mr = Mb[0], mi = Mb[1], kr = Kb[0], ki = Kb[1];
      const float den = mr * mr + mi * mi;
      cr = (kr * mr + ki * mi) / den; ci = (ki * mr - kr * mi) / den;
      up = to_f32(Up[(size_t)bh * 64 + row]);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int d = 64 * hf + 2 * j;
      float re = 0.f, im = 0.f;
      if (p.z0) {
        const float2 z = *reinterpret_cast<const float2*>(p.z0 + ((size_t)bh * 64 + row) * 128 + d);
        re = z.x; im = z.y;
      }
      if (Bp) {
        const float br = to_f32(Bp[(size_t)bg * 128 + d]), bi = to_f32(Bp[(size_t)bg * 128 + d + 1]);
        re += up * (cr * br - ci * bi);
        im += up * (cr * bi + ci * br);
      }
      zv[2 * j] = re; zv[2 * j + 1] = -im;
    }
  }
  auto store_zv_tile = [&]() {   // bf16 copy of the state: rows p, K-major along d
    uint8_t* zt = smem + OFF_ZV + hf * TILE;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      uint4 v;
      v.x = PK::pack(zv[8 * ch + 0], zv[8 * ch + 1]); v.y = PK::pack(zv[8 * ch + 2], zv[8 * ch + 3]);
      v.z = PK::pack(zv[8 * ch + 4], zv[8 * ch + 5]); v.w = PK::pack(zv[8 * ch + 6], zv[8 * ch + 7]);
      *reinterpret_cast<uint4*>(zt + sw128(row, ch)) = v;
    }
  };
  auto store_chunk_state = [&](int c) {   // conjugated form, 16-bit, row-major [p][128]
    if (!p.states16) return;
    TIn* dst = reinterpret_cast<TIn*>(p.states16) + (((size_t)bh * p.nchunks + c) * 64 + row) * 128 + 64 * hf;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      uint4 v;
      v.x = PK::pack(zv[8 * ch + 0], zv[8 * ch + 1]); v.y = PK::pack(zv[8 * ch + 2], zv[8 * ch + 3]);
      v.z = PK::pack(zv[8 * ch + 4], zv[8 * ch + 5]); v.w = PK::pack(zv[8 * ch + 6], zv[8 * ch + 7]);
      *reinterpret_cast<uint4*>(dst + 8 * ch) = v;
    }
  };
  store_zv_tile();

  constexpr uint32_t ID_S = make_idesc(64, 32, PK::fmt, 0, 0);     // K-major x K-major
  constexpr uint32_t ID_Y = make_idesc(64, 32, PK::fmt, 0, 1);     // K-major x MN-major
  constexpr uint32_t ID_Z = make_idesc(64, 64, PK::fmt, 1, 1);     // MN-major x MN-major
  const uint32_t aKPP = smem_u32(smem + OFF_KPP), aS = smem_u32(smem + OFF_S),
                 aZV = smem_u32(smem + OFF_ZV);
  bool ok = true;

  for (int c = 0; c < p.nchunks && ok; ++c) {
    const int t0 = c * L;
    uint8_t* st = smem + (c & 1) * STAGE;
    if (tid == 0 && c + 1 < p.nchunks) issue_loads(c + 1);
    if (warp == 0) chunk_scalars(sc, Mb, Kb, t0, T, lane);
    store_chunk_state(c);
    ok = mbar_wait(&bar_tma[c & 1], (c >> 1) & 1);
    if (!ok) { report_timeout(1); s_abort = 1; }
    __syncthreads();
    if (s_abort) { ok = false; break; }

    // ---- rotation: C -> Q, B -> K' (both in place), K'' ; diagonal scores --------------------
    {
      const uint32_t half = rcol >> 3, ch = rcol & 7;
      uint8_t* tB = st + TILE + half * TILE;
      uint8_t* tC = st + 3 * TILE + half * TILE;
      uint8_t* tK = smem + OFF_KPP + half * TILE;
#pragma unroll 2
      for (int k = 0; k < 8; ++k) {
        const int r = rrow0 + 8 * k;
        const uint32_t off = sw128(r, ch);
        const float phr = sc[2 * 64 + r], phi = sc[3 * 64 + r];
        const float wr = sc[4 * 64 + r], wi = sc[5 * 64 + r];
        const float vr = sc[6 * 64 + r], vi = sc[7 * 64 + r];
        const float kr = sc[8 * 64 + r], ki = sc[9 * 64 + r];
        uint4 cv = make_uint4(0u, 0u, 0u, 0u);
        if (!STATES_ONLY) cv = *reinterpret_cast<const uint4*>(tC + off);
        const uint4 bv = *reinterpret_cast<const uint4*>(tB + off);
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t qo[4], ko[4], vo[4];
        float dg = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 cc = PK::unpack(cw[e]), bb = PK::unpack(bw[e]);
          qo[e] = PK::pack(cc.x * phr + cc.y * phi, cc.x * phi - cc.y * phr);     // conj(c) phi
          ko[e] = PK::pack(wr * bb.x - wi * bb.y, -(wr * bb.y + wi * bb.x));      // conj(w b)
          vo[e] = PK::pack(vr * bb.x - vi * bb.y, -(vr * bb.y + vi * bb.x));      // conj(v b)
          const float xr = kr * bb.x - ki * bb.y, xi = kr * bb.y + ki * bb.x;     // kc b
          dg += cc.x * xr + cc.y * xi;                                            // Re(conj(c) kc b)
        }
        *reinterpret_cast<uint4*>(tK + off) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
        if (!STATES_ONLY) {
          *reinterpret_cast<uint4*>(tC + off) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
          *reinterpret_cast<uint4*>(tB + off) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, o);
          if (rcol == 0) s_diag[r] = dg;
        }
      }
    }
    fence_async_smem();
    __syncthreads();

    if (!STATES_ONLY) {
    // ---- MMA group 1: scores and off-term ------------------------------------------------------
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t aB = smem_u32(st + TILE), aC = smem_u32(st + 3 * TILE);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint32_t dS = tmem + ((16u * q) << 16), dO = dS + 32;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t ko = (k >> 2) * TILE + (k & 3) * 32;
          const uint64_t da = make_desc(aC + ko, 16, 1024);
          umma(dS, da, make_desc(aB + 4096 * q + ko, 16, 1024), ID_S, k > 0);
          umma(dO, da, make_desc(aZV + 4096 * q + ko, 16, 1024), ID_S, k > 0);
        }
      }
      umma_commit(&bar_mma[0]);
    }
    ok = mbar_wait(&bar_mma[0], c & 1);
    if (!ok) { report_timeout(2); s_abort = 1; }
    tc_fence_after_sync();

    // ---- scores epilogue: decay, causal mask, diagonal -> 16-bit S tile ----------------------------
    {
      uint32_t r32[32];
      tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 0, r32);
      tmem_ld_wait();
      const float lt = sc[row];
      const float dgv = s_diag[row];
      uint8_t* tS = smem + OFF_S;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v2[2];
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int j = 8 * ch + 2 * e + q, s = 32 * hf + j;
            float v = __uint_as_float(r32[j]) * __expf(fminf(lt - sc[s], 0.f));
            v = s < row ? v : (s == row ? dgv : 0.f);
            v2[q] = v;
          }
          w[e] = PK::pack(v2[0], v2[1]);
        }
        *reinterpret_cast<uint4*>(tS + sw128(row, 4 * hf + ch)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (s_abort) { ok = false; break; }
    }  // !STATES_ONLY

    // ---- MMA group 2: Y_diag = S U, Inc = U^T K'' ------------------------------------------------------
    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t aU = smem_u32(st);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const uint32_t dY = tmem + ((16u * q) << 16) + 64, dZ = tmem + ((16u * q) << 16) + 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (!STATES_ONLY)
            umma(dY, make_desc(aS + 32 * k, 16, 1024), make_desc(aU + 64 * q + 2048 * k, 8192, 1024), ID_Y,
                 k > 0);
          umma(dZ, make_desc(aU + 2048 * k, 8192, 1024), make_desc(aKPP + TILE * q + 2048 * k, 8192, 1024),
               ID_Z, k > 0);
        }
      }
      umma_commit(&bar_mma[1]);
    }
    ok = mbar_wait(&bar_mma[1], c & 1);
    if (!ok) { report_timeout(3); s_abort = 1; }
    tc_fence_after_sync();

    // ---- output epilogue: y = Y_diag + exp(l_t) Y_off ---------------------------------------------------
    if (!STATES_ONLY) {
      uint32_t yd[32], yo[32];
      tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 64, yd);
      tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 32, yo);
      tmem_ld_wait();
      const float et = sc[1 * 64 + row];
      if (t0 + row < T) {
        TY* dst = reinterpret_cast<TY*>(p.Y) + ((size_t)bh * T + t0 + row) * 64 + 32 * hf;
        if constexpr (sizeof(TY) == 2) {
          using PY = Pack2<TY>;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = 8 * v + 2 * e;
              w[e] = PY::pack(__uint_as_float(yd[j]) + et * __uint_as_float(yo[j]),
                              __uint_as_float(yd[j + 1]) + et * __uint_as_float(yo[j + 1]));
            }
            *reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        } else {
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float4 o;
            o.x = __uint_as_float(yd[4 * v]) + et * __uint_as_float(yo[4 * v]);
            o.y = __uint_as_float(yd[4 * v + 1]) + et * __uint_as_float(yo[4 * v + 1]);
            o.z = __uint_as_float(yd[4 * v + 2]) + et * __uint_as_float(yo[4 * v + 2]);
            o.w = __uint_as_float(yd[4 * v + 3]) + et * __uint_as_float(yo[4 * v + 3]);
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + 4 * v) = o;
          }
        }
      }
    }
    // ---- state update: zv = conj(Pi_end) zv + Inc -------------------------------------------------------
    {
      const float pr = sc[10 * 64 + 0], pi = sc[10 * 64 + 1];
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t inc[32];
        tmem_ld32(tmem + ((uint32_t)(32 * warp) << 16) + 128 + 32 * part, inc);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float a = zv[32 * part + 2 * j], bq = zv[32 * part + 2 * j + 1];
          zv[32 * part + 2 * j] = pr * a + pi * bq + __uint_as_float(inc[2 * j]);
          zv[32 * part + 2 * j + 1] = pr * bq - pi * a + __uint_as_float(inc[2 * j + 1]);
        }
      }
      store_zv_tile();
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (s_abort) { ok = false; break; }
  }

  if (ok && p.zfinal) {
    float* dst = p.zfinal + ((size_t)bh * 64 + row) * 128 + 64 * hf;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      *reinterpret_cast<float4*>(dst + 4 * j) =
          make_float4(zv[4 * j], -zv[4 * j + 1], zv[4 * j + 2], -zv[4 * j + 3]);
  }
  // unwind: nothing of ours may still be in flight when shared memory / TMEM are released
  if (!ok && tid == 0) {
    for (int s = 0; s < 2; ++s) mbar_wait(&bar_tma[s], 0);   // bounded; best effort drain
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

#include "scan_tc_bwd.cuh"

}  // namespace

bool scan_tc_supported(const ScanDims& d, int io_dtype) {
  return d.P == 64 && d.N == 64 && (io_dtype == SL_BF16 || io_dtype == SL_F16) && d.T >= 1 &&
         tc::encode_tiled_fn() != nullptr;
}
size_t scan_tc_fwd_workspace(const ScanDims&) { return 0; }
namespace {
struct TcBwdLayout {
  size_t states, zfinal, dg, sterm, dkcd, anchor, total;
};
TcBwdLayout tc_bwd_layout(const ScanDims& d) {
  const size_t BH = (size_t)d.batch * d.heads, nC = (d.T + L - 1) / L;
  TcBwdLayout o{};
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t r = off; off += round_up(bytes, 256); return r; };
  o.states = take(BH * nC * 64 * 128 * 2);
  o.zfinal = take(BH * 64 * 128 * 4);
  o.dg = take(BH * d.T * 8);
  o.sterm = take(BH * d.T * 8);
  o.dkcd = take(BH * d.T * 8);
  o.anchor = take(BH * nC * 8);
  o.total = off;
  return o;
}
}  // namespace

size_t scan_tc_bwd_workspace(const ScanDims& d) {
  return std::max(scan_simt_bwd_workspace(d), tc_bwd_layout(d).total);
}

template <typename TIn, typename TY, bool STATES_ONLY>
static int launch_tc_fwd(const TcFwdParams& p, int grid, cudaStream_t st) {
  auto k = scan_tc_fwd_kernel<TIn, TY, STATES_ONLY>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess)
    return SL_ERR_LAUNCH_FAILED;
  k<<<grid, 128, SMEM_BYTES, st>>>(p);
  note_launches(1);
  return launch_status();
}

// Y == nullptr runs the state pre-sweep only (chunk-start states + final state).
int scan_tc_fwd_impl(const void* U, const float* M, const float* K, const void* B, const void* C,
                     const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                     void* states16, const ScanDims& d, int io_dtype, int y_dtype,
                     cudaStream_t st) {
  TcFwdParams p{};
  const bool bf = io_dtype == SL_BF16;
  const uint64_t BH = (uint64_t)d.batch * d.heads, BG = (uint64_t)d.batch * d.groups;
  if (!tc::make_tmap_3d(&p.tmU, U, 64, d.T, BH, 64, bf) || !tc::make_tmap_3d(&p.tmB, B, 128, d.T, BG, 64, bf) ||
      !tc::make_tmap_3d(&p.tmC, C ? C : B, 128, d.T, BG, 64, bf))
    return SL_ERR_LAUNCH_FAILED;
  p.M = M; p.K = K; p.z0 = z0; p.Bprev = Bprev; p.Uprev = Uprev; p.Y = Y; p.zfinal = zfinal;
  p.states16 = states16;
  p.heads = d.heads; p.groups = d.groups; p.T = d.T; p.nchunks = (d.T + L - 1) / L;
  const int grid = (int)BH;
  int rc = SL_ERR_UNSUPPORTED;
  if (!Y) {
    rc = bf ? launch_tc_fwd<__nv_bfloat16, float, true>(p, grid, st)
            : launch_tc_fwd<__half, float, true>(p, grid, st);
  } else if (bf) {
    SL_DISPATCH_DTYPE(y_dtype, TY, { rc = launch_tc_fwd<__nv_bfloat16, TY, false>(p, grid, st); });
  } else {
    SL_DISPATCH_DTYPE(y_dtype, TY, { rc = launch_tc_fwd<__half, TY, false>(p, grid, st); });
  }
  return rc;
}

int scan_tc_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                const ScanDims& d, int io_dtype, int y_dtype, void*, size_t, cudaStream_t st) {
  return scan_tc_fwd_impl(U, M, K, B, C, z0, Bprev, Uprev, Y, zfinal, nullptr, d, io_dtype, y_dtype, st);
}

// Tensor-core backward: state pre-sweep, reverse sweep, scalar finish.  Cases it does not
// cover (grouped B/C, carried B_prev/U_prev, dY of another dtype or absent) take the exact
// float32 sweeps.
int scan_tc_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, const void* dY,
                const float* dfinal, void* dU, float* dM, float* dK, void* dB, void* dC, float* dinit,
                void* dBprev, void* dUprev, const ScanDims& d, int io_dtype, int dy_dtype, void* ws,
                size_t ws_bytes, cudaStream_t st) {
  if (d.groups != d.heads || Bprev || !dY || dy_dtype != io_dtype)
    return scan_simt_bwd(U, M, K, B, C, z0, Bprev, Uprev, dY, dfinal, dU, dM, dK, dB, dC, dinit, dBprev,
                         dUprev, d, io_dtype, dy_dtype, ws, ws_bytes, st);
  const TcBwdLayout lay = tc_bwd_layout(d);
  if (!ws || ws_bytes < lay.total) return SL_ERR_WORKSPACE_TOO_SMALL;
  uint8_t* w = reinterpret_cast<uint8_t*>(ws);
  const bool bf = io_dtype == SL_BF16;
  const uint64_t BH = (uint64_t)d.batch * d.heads;
  const int nC = (d.T + L - 1) / L;
  float* zfinal = reinterpret_cast<float*>(w + lay.zfinal);
  if (int e = scan_tc_fwd_impl(U, M, K, B, nullptr, z0, nullptr, nullptr, nullptr, zfinal, w + lay.states, d,
                               io_dtype, SL_F32, st))
    return e;
  TcBwdParams p{};
  if (!tc::make_tmap_3d(&p.tmU, U, 64, d.T, BH, 64, bf) || !tc::make_tmap_3d(&p.tmB, B, 128, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmC, C, 128, d.T, BH, 64, bf) || !tc::make_tmap_3d(&p.tmdY, dY, 64, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmZ, w + lay.states, 128, (uint64_t)nC * 64, BH, 64, bf))
    return SL_ERR_LAUNCH_FAILED;
  p.M = M; p.K = K; p.dfinal = dfinal; p.zfinal = zfinal; p.dU = dU; p.dB = dB; p.dC = dC;
  p.dg = reinterpret_cast<float2*>(w + lay.dg); p.sterm = reinterpret_cast<float2*>(w + lay.sterm);
  p.dkcd = reinterpret_cast<float2*>(w + lay.dkcd); p.anchor = reinterpret_cast<float2*>(w + lay.anchor);
  p.dinit = dinit; p.T = d.T; p.nchunks = nC;
  if (bf) {
    auto k = scan_tc_bwd_kernel<__nv_bfloat16>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)B_SMEM_BYTES) != cudaSuccess)
      return SL_ERR_LAUNCH_FAILED;
    k<<<(int)BH, 128, B_SMEM_BYTES, st>>>(p);
  } else {
    auto k = scan_tc_bwd_kernel<__half>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)B_SMEM_BYTES) != cudaSuccess)
      return SL_ERR_LAUNCH_FAILED;
    k<<<(int)BH, 128, B_SMEM_BYTES, st>>>(p);
  }
  scan_tc_bwd_finish_kernel<<<(int)BH, 128, 0, st>>>(M, K, p.dg, p.sterm, p.dkcd, p.anchor, dM, dK, d.T, nC);
  note_launches(2);
  return launch_status();
}

int scan_tc_device_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  return v;
}

}  // namespace sl
