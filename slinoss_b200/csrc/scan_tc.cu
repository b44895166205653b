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
// One CTA of 18 warps walks the chunks of one (batch, head) in order: 16 worker warps (4 TMEM
// lane quadrants x 4 column groups: rotation passes and every epilogue), one warp that computes
// the per-chunk scalars one chunk ahead, and one warp whose lane 0 issues every TMA load / store
// and every tcgen05.mma.  U/B/C tiles arrive by TMA (128B swizzle, one chunk ahead), the state
// lives in the workers' registers (float32), the MMAs have M = 64 (rows in lanes 0..15 of every
// TMEM lane quadrant); scan_tc_fwd.cuh and scan_tc_bwd.cuh describe the thread-to-data mappings.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "tc_common.cuh"

namespace sl {
namespace {

using namespace tc;

constexpr int L = 64;
constexpr uint32_t TILE = 8192;           // one [64][128 B] tile
constexpr uint32_t STAGE = 7 * TILE;      // U | B0 | Zv0 | B1 | Zv1 | C0 | C1  (Zv written by the CTA)
constexpr uint32_t OFF_KPP = 2 * STAGE;   // K'' (2 tiles)
constexpr uint32_t OFF_S = OFF_KPP + 2 * TILE;
constexpr uint32_t OFF_Y = OFF_S + TILE;  // 16-bit Y tile staged for its TMA store
constexpr uint32_t OFF_SCAL = OFF_Y + TILE;
constexpr int NSCAL = 12;                 // per-token float arrays
constexpr uint32_t SMEM_BYTES = OFF_SCAL + 2 * NSCAL * 64 * 4 + 64 + 1024;
// TMEM columns: [S | Yoff] 0..127 and 128..255 (chunk parity) | Ydiag 256..319 and 320..383 | Inc 384..511
constexpr uint32_t TMEM_COLS = 512;

__device__ int g_tc_status = 0;

struct alignas(64) TcFwdParams {
  CUtensorMap tmU, tmB, tmC;
  CUtensorMap tmY, tmS;   // 16-bit output and chunk-state tensors (TMA stores); unused ones stay zero
  const float* M;
  const float* K;
  const float* z0;
  const void* Bprev;
  const void* Uprev;
  void* Y;
  const float* Yadd;    // optional float32 (batch*heads, T, 64): added to the output before it is rounded
  float* zfinal;
  void* states16;       // optional (batch*heads, nchunks, 64, 128) 16-bit: conjugated start state of every chunk
  int heads, groups, T, nchunks;
  long long wait_limit;  // SM clocks a wait of the main loop may take before the kernel gives up
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

// Limit of the kernels' bounded waits in SM clocks: about a second by default; the environment
// variable SLINOSS_B200_WAIT_CLOCKS (read at every launch) overrides it, which is how the test of
// the unwind path makes a wait expire without anything being wrong.
static long long wait_limit_clocks() {
  if (const char* e = getenv("SLINOSS_B200_WAIT_CLOCKS")) {
    const long long v = atoll(e);
    if (v > 0) return v;
  }
  return tc::WAIT_CLOCKS_DEFAULT;
}

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

#include "scan_tc_fwd.cuh"
#include "scan_tc_bwd.cuh"

}  // namespace

// The kernels hold 64 complex state columns per (batch, head).  The recurrence does not couple state
// columns (z[:, n] sees b[n] only, and y sums c[n] z[:, n] over n), so N = 128 runs as two passes over the
// column blocks 0..63 and 64..127 of B and C, addressed in place through tensor maps with the full row
// pitch; the passes' Y, dU, dM, dK and dU_prev add, everything else is per column block.
bool scan_tc_supported(const ScanDims& d, int io_dtype) {
  return d.P == 64 && (d.N == 64 || d.N == 128) && (io_dtype == SL_BF16 || io_dtype == SL_F16) && d.T >= 1 &&
         tc::encode_tiled_fn() != nullptr;
}
namespace {
inline ScanDims one_block(const ScanDims& d) { ScanDims o = d; o.N = 64; return o; }
// forward workspace of the two-pass form: start state, final state and B_prev of one column block (dense),
// and the float32 output of the first pass
struct TcFwdSplitLayout { size_t z0, zf, bprev, ypart, total; };
TcFwdSplitLayout tc_fwd_split_layout(const ScanDims& d) {
  const size_t BH = (size_t)d.batch * d.heads, BG = (size_t)d.batch * d.groups;
  TcFwdSplitLayout o{};
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t r = off; off += round_up(bytes, 256); return r; };
  o.z0 = take(BH * 64 * 128 * 4);
  o.zf = take(BH * 64 * 128 * 4);
  o.bprev = take(BG * 128 * 2);
  o.ypart = take(BH * (size_t)d.T * 64 * 4);
  o.total = off;
  return o;
}
}  // namespace
size_t scan_tc_fwd_workspace(const ScanDims& d) { return d.N == 128 ? tc_fwd_split_layout(d).total : 0; }
namespace {
struct TcBwdLayout {
  size_t states, zfinal, dg, sterm, dkcd, anchor, dbh, dch, dstart, dgb, total;
};
// (the carried-tap regions are always reserved: the workspace query does not know whether the call
// will carry B_prev / U_prev)
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
  if (d.groups != d.heads) {   // per-head dB / dC (16-bit) before the reduction over the heads of a group
    o.dbh = take(BH * d.T * 128 * 2);
    o.dch = take(BH * d.T * 128 * 2);
  }
  o.dstart = take(BH * 64 * 128 * 4);   // adjoint of the start state when the caller wants no d_initial
  o.dgb = take(BH * 8);                 // gradient of the pending tap's coefficient
  o.total = off;
  return o;
}
}  // namespace

// backward workspace of the two-pass form: the one-block workspace (reused by both passes), dense copies
// of the per-block inputs, dense per-block outputs, and the second pass' summands
struct TcBwdSplitLayout {
  size_t inner, z0, zf, dfin, dinit, bprev, dbprev, du, dm, dk, duprev, total;
};
TcBwdSplitLayout tc_bwd_split_layout(const ScanDims& d) {
  const size_t BH = (size_t)d.batch * d.heads, BG = (size_t)d.batch * d.groups;
  TcBwdSplitLayout o{};
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t r = off; off += round_up(bytes, 256); return r; };
  o.inner = take(tc_bwd_layout(one_block(d)).total);
  o.z0 = take(BH * 64 * 128 * 4);
  o.zf = take(BH * 64 * 128 * 4);
  o.dfin = take(BH * 64 * 128 * 4);
  o.dinit = take(BH * 64 * 128 * 4);
  o.bprev = take(BG * 128 * 2);
  o.dbprev = take(BG * 128 * 2);
  o.du = take(BH * (size_t)d.T * 64 * 2);
  o.dm = take(BH * (size_t)d.T * 2 * 4);
  o.dk = take(BH * (size_t)d.T * 4 * 4);
  o.duprev = take(BH * 64 * 2);
  o.total = off;
  return o;
}

size_t scan_tc_bwd_workspace(const ScanDims& d) {
  const size_t tcw = d.N == 128 ? tc_bwd_split_layout(d).total : tc_bwd_layout(d).total;
  return std::max(scan_simt_bwd_workspace(d), tcw);
}

constexpr int NW = 4;   // worker warps per TMEM lane quadrant

template <typename TIn, typename TY, bool STATES_ONLY>
static int launch_tc_fwd(const TcFwdParams& p, int grid, cudaStream_t st) {
  auto k = scan_tc_fwd_kernel<TIn, TY, STATES_ONLY, NW>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) != cudaSuccess)
    return SL_ERR_LAUNCH_FAILED;
  k<<<grid, 128 * NW + 64, SMEM_BYTES, st>>>(p);
  note_launches(1);
  return launch_status();
}

// Y == nullptr runs the state pre-sweep only (chunk-start states + final state).
// ``bc_pitch`` = elements per row of B and C (128, or 256 when B / C point at one column block of
// N = 128 rows); everything else is dense with 64 state columns.  ``Yadd`` (float32, or null) is added to
// the output before it is rounded: the first pass' output in the two-pass form.
int scan_tc_fwd_impl(const void* U, const float* M, const float* K, const void* B, const void* C,
                     const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                     void* states16, const ScanDims& d, int io_dtype, int y_dtype,
                     cudaStream_t st, int bc_pitch = 128, const float* Yadd = nullptr) {
  TcFwdParams p{};
  const bool bf = io_dtype == SL_BF16;
  const uint64_t BH = (uint64_t)d.batch * d.heads, BG = (uint64_t)d.batch * d.groups;
  if (!tc::make_tmap_3d(&p.tmU, U, 64, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmB, B, 128, d.T, BG, 64, bf, bc_pitch) ||
      !tc::make_tmap_3d(&p.tmC, C ? C : B, 128, d.T, BG, 64, bf, bc_pitch))
    return SL_ERR_LAUNCH_FAILED;
  p.M = M; p.K = K; p.z0 = z0; p.Bprev = Bprev; p.Uprev = Uprev; p.Y = Y; p.zfinal = zfinal; p.Yadd = Yadd;
  p.states16 = states16;
  p.heads = d.heads; p.groups = d.groups; p.T = d.T; p.nchunks = (d.T + L - 1) / L;
  p.wait_limit = wait_limit_clocks();
  if (Y && y_dtype != SL_F32 && !tc::make_tmap_3d(&p.tmY, Y, 64, d.T, BH, 64, y_dtype == SL_BF16))
    return SL_ERR_LAUNCH_FAILED;
  if (states16 && !tc::make_tmap_3d(&p.tmS, states16, 128, (uint64_t)p.nchunks * 64, BH, 64, bf))
    return SL_ERR_LAUNCH_FAILED;
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

size_t scan_tc_states_bytes(const ScanDims& d) {   // N = 128: the two column blocks one after the other
  return (size_t)d.batch * d.heads * ((d.T + L - 1) / L) * 64 * 128 * 2 * (d.N / 64);
}

namespace {
// column block ``blk`` (128 values of 256) of a (rows, 256) tensor <-> a dense (rows, 128) one
inline bool copy_block_in(void* dense, const void* wide, int blk, size_t rows, size_t esize, cudaStream_t st) {
  return cudaMemcpy2DAsync(dense, 128 * esize, reinterpret_cast<const uint8_t*>(wide) + blk * 128 * esize,
                           256 * esize, 128 * esize, rows, cudaMemcpyDeviceToDevice, st) == cudaSuccess;
}
inline bool copy_block_out(void* wide, const void* dense, int blk, size_t rows, size_t esize, cudaStream_t st) {
  return cudaMemcpy2DAsync(reinterpret_cast<uint8_t*>(wide) + blk * 128 * esize, 256 * esize, dense,
                           128 * esize, 128 * esize, rows, cudaMemcpyDeviceToDevice, st) == cudaSuccess;
}
inline const void* block_of(const void* wide, int blk) {   // 16-bit rows of 256: start of a column block
  return wide ? reinterpret_cast<const uint8_t*>(wide) + blk * 256 : nullptr;
}

// a += b over n 16-bit values (summed in float32) or float32 values; 16 bytes per thread, the last
// thread takes what is left of a length that is no multiple of that
template <typename T>
__global__ void __launch_bounds__(256) add_into_kernel(T* __restrict__ a, const T* __restrict__ b, size_t n) {
  constexpr int V = Vec16<T>::N;
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (i >= n) return;
  if (i + V <= n) {
    float x[V], y[V];
    load16<T>(a + i, x);
    load16<T>(b + i, y);
#pragma unroll
    for (int k = 0; k < V; ++k) x[k] += y[k];
    store16<T>(a + i, x);
  } else {
    for (size_t j = i; j < n; ++j) a[j] = from_f32<T>(to_f32(a[j]) + to_f32(b[j]));
  }
}
template <typename T>
void add_into(void* a, const void* b, size_t n, cudaStream_t st) {
  const size_t pieces = (n + Vec16<T>::N - 1) / Vec16<T>::N;
  add_into_kernel<T><<<(unsigned)((pieces + 255) / 256), 256, 0, st>>>(reinterpret_cast<T*>(a),
                                                                      reinterpret_cast<const T*>(b), n);
  note_launches(1);
}
}  // namespace

int scan_tc_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                void* states_out, const ScanDims& d, int io_dtype, int y_dtype, void* ws, size_t ws_bytes,
                cudaStream_t st) {
  if (d.N == 64)
    return scan_tc_fwd_impl(U, M, K, B, C, z0, Bprev, Uprev, Y, zfinal, states_out, d, io_dtype, y_dtype, st);
  // N = 128: two passes over the column blocks; the second adds the first's float32 output
  const TcFwdSplitLayout lay = tc_fwd_split_layout(d);
  if (!ws || ws_bytes < lay.total) return SL_ERR_WORKSPACE_TOO_SMALL;
  uint8_t* w = reinterpret_cast<uint8_t*>(ws);
  const ScanDims d1 = one_block(d);
  const size_t BH = (size_t)d.batch * d.heads, BG = (size_t)d.batch * d.groups;
  const size_t st_bytes = scan_tc_states_bytes(d1);
  float* ypart = reinterpret_cast<float*>(w + lay.ypart);
  for (int blk = 0; blk < 2; ++blk) {
    float* z0b = z0 ? reinterpret_cast<float*>(w + lay.z0) : nullptr;
    float* zfb = zfinal ? reinterpret_cast<float*>(w + lay.zf) : nullptr;
    void* bpb = Bprev ? (void*)(w + lay.bprev) : nullptr;
    if (z0 && !copy_block_in(z0b, z0, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
    if (Bprev && !copy_block_in(bpb, Bprev, blk, BG, 2, st)) return SL_ERR_LAUNCH_FAILED;
    void* st_out = states_out ? reinterpret_cast<uint8_t*>(states_out) + blk * st_bytes : nullptr;
    const int rc = scan_tc_fwd_impl(U, M, K, block_of(B, blk), block_of(C, blk), z0b, bpb, Uprev,
                                    blk == 0 ? (void*)ypart : Y, zfb, st_out, d1, io_dtype,
                                    blk == 0 ? (int)SL_F32 : y_dtype, st, 256, blk == 0 ? nullptr : ypart);
    if (rc != SL_OK) return rc;
    if (zfinal && !copy_block_out(zfinal, zfb, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
  }
  return launch_status();
}

template <typename TIn>
static int launch_tc_bwd(const TcBwdParams& p, int grid, cudaStream_t st) {
  auto k = scan_tc_bwd_kernel<TIn, NW>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)B_SMEM_BYTES) != cudaSuccess)
    return SL_ERR_LAUNCH_FAILED;
  k<<<grid, 128 * NW + 64, B_SMEM_BYTES, st>>>(p);
  return launch_status();
}

// Tensor-core backward: state pre-sweep (unless the forward saved its chunk states), reverse sweep,
// the boundary terms of carried B_prev / U_prev, scalar finish and, for grouped B/C, the reduction of
// dB / dC over the heads of a group.  A dY of another dtype (or none) takes the exact float32 sweeps.
//
// One block of 64 state columns: ``d.N`` is 64; B, C, dB, dC have ``bc_pitch`` elements per row (128, or 256
// when they point at one column block of N = 128 rows); every other tensor is dense.
static int scan_tc_bwd_block(const void* U, const float* M, const float* K, const void* B, const void* C,
                             const float* z0, const void* Bprev, const void* Uprev, const void* states_in,
                             const float* zfinal_in, const void* dY, const float* dfinal, void* dU, float* dM,
                             float* dK, void* dB, void* dC, float* dinit, void* dBprev, void* dUprev,
                             const ScanDims& d, int io_dtype, void* ws, size_t ws_bytes, cudaStream_t st,
                             int bc_pitch) {
  const TcBwdLayout lay = tc_bwd_layout(d);
  if (!ws || ws_bytes < lay.total) return SL_ERR_WORKSPACE_TOO_SMALL;
  uint8_t* w = reinterpret_cast<uint8_t*>(ws);
  const bool bf = io_dtype == SL_BF16;
  const uint64_t BH = (uint64_t)d.batch * d.heads, BG = (uint64_t)d.batch * d.groups;
  const bool grouped = d.groups != d.heads;
  void* dBh = grouped ? (void*)(w + lay.dbh) : dB;   // where the sweep stores dB / dC (per head)
  void* dCh = grouped ? (void*)(w + lay.dch) : dC;
  const int nC = (d.T + L - 1) / L;
  const float* zfinal = zfinal_in;
  const void* states = states_in;
  if (!states || !zfinal) {   // nothing saved by the forward: recompute with the state pre-sweep
    float* zf = reinterpret_cast<float*>(w + lay.zfinal);
    if (int e = scan_tc_fwd_impl(U, M, K, B, nullptr, z0, Bprev, Uprev, nullptr, zf, w + lay.states, d,
                                 io_dtype, SL_F32, st, bc_pitch))
      return e;
    zfinal = zf;
    states = w + lay.states;
  }
  TcBwdParams p{};
  const uint64_t out_pitch = grouped ? 128 : bc_pitch;   // the per-head workspace is dense
  if (!tc::make_tmap_3d(&p.tmU, U, 64, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmB, B, 128, d.T, BG, 64, bf, bc_pitch) ||
      !tc::make_tmap_3d(&p.tmC, C, 128, d.T, BG, 64, bf, bc_pitch) ||
      !tc::make_tmap_3d(&p.tmdY, dY, 64, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmZ, states, 128, (uint64_t)nC * 64, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmdU, dU, 64, d.T, BH, 64, bf) ||
      !tc::make_tmap_3d(&p.tmdB, dBh, 128, d.T, BH, 64, bf, out_pitch) ||
      !tc::make_tmap_3d(&p.tmdC, dCh, 128, d.T, BH, 64, bf, out_pitch))
    return SL_ERR_LAUNCH_FAILED;
  p.M = M; p.K = K; p.dfinal = dfinal; p.zfinal = zfinal;
  p.dg = reinterpret_cast<float2*>(w + lay.dg); p.sterm = reinterpret_cast<float2*>(w + lay.sterm);
  p.dkcd = reinterpret_cast<float2*>(w + lay.dkcd); p.anchor = reinterpret_cast<float2*>(w + lay.anchor);
  // with carried taps the adjoint of the start state is needed even when the caller asks for no d_initial
  float* dstart = dinit ? dinit : (Bprev ? reinterpret_cast<float*>(w + lay.dstart) : nullptr);
  float2* dgb = Bprev ? reinterpret_cast<float2*>(w + lay.dgb) : nullptr;
  p.dinit = dstart; p.T = d.T; p.nchunks = nC; p.heads = d.heads; p.groups = d.groups;
  p.wait_limit = wait_limit_clocks();
  int rc = SL_ERR_UNSUPPORTED;
  rc = bf ? launch_tc_bwd<__nv_bfloat16>(p, (int)BH, st) : launch_tc_bwd<__half>(p, (int)BH, st);
  if (rc != SL_OK) return rc;
  if (Bprev) {
    if (bf)
      scan_tc_bwd_boundary_kernel<__nv_bfloat16><<<(unsigned)BG, 128, 0, st>>>(
          dstart, (const __nv_bfloat16*)Bprev, (const __nv_bfloat16*)Uprev, M, K, (__nv_bfloat16*)dBprev,
          (__nv_bfloat16*)dUprev, dgb, d.heads, d.groups, d.T);
    else
      scan_tc_bwd_boundary_kernel<__half><<<(unsigned)BG, 128, 0, st>>>(dstart, (const __half*)Bprev,
                                                                       (const __half*)Uprev, M, K, (__half*)dBprev,
                                                                       (__half*)dUprev, dgb, d.heads, d.groups, d.T);
    note_launches(1);
  }
  scan_tc_bwd_finish_kernel<<<dim3((unsigned)BH, (unsigned)((nC + 3) / 4)), 128, 0, st>>>(M, K, p.dg, p.sterm, p.dkcd, p.anchor, dgb, dM, dK, d.T, nC);
  note_launches(2);
  if (grouped) {
    const size_t pieces = BG * (size_t)d.T * 16;
    const unsigned blocks = (unsigned)((pieces + 255) / 256);
    if (bf)
      scan_tc_group_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(
          (const __nv_bfloat16*)dBh, (const __nv_bfloat16*)dCh, (__nv_bfloat16*)dB, (__nv_bfloat16*)dC, d.heads,
          d.groups, d.T, pieces, bc_pitch);
    else
      scan_tc_group_reduce_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)dBh, (const __half*)dCh, (__half*)dB,
                                                                 (__half*)dC, d.heads, d.groups, d.T, pieces,
                                                                 bc_pitch);
    note_launches(1);
  }
  return launch_status();
}


int scan_tc_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, const void* states_in,
                const float* zfinal_in, const void* dY,
                const float* dfinal, void* dU, float* dM, float* dK, void* dB, void* dC, float* dinit,
                void* dBprev, void* dUprev, const ScanDims& d, int io_dtype, int dy_dtype, void* ws,
                size_t ws_bytes, cudaStream_t st) {
  if (!dY || dy_dtype != io_dtype)
    return scan_simt_bwd(U, M, K, B, C, z0, Bprev, Uprev, dY, dfinal, dU, dM, dK, dB, dC, dinit, dBprev,
                         dUprev, d, io_dtype, dy_dtype, ws, ws_bytes, st);
  if (d.N == 64)
    return scan_tc_bwd_block(U, M, K, B, C, z0, Bprev, Uprev, states_in, zfinal_in, dY, dfinal, dU, dM, dK, dB,
                             dC, dinit, dBprev, dUprev, d, io_dtype, ws, ws_bytes, st, 128);
  // N = 128: one pass per column block.  dB, dC, d_initial and dB_prev are per block; dU, dM, dK and
  // dU_prev are the sums of the passes (the second pass writes into the workspace and is added).
  const TcBwdSplitLayout lay = tc_bwd_split_layout(d);
  if (!ws || ws_bytes < lay.total) return SL_ERR_WORKSPACE_TOO_SMALL;
  uint8_t* w = reinterpret_cast<uint8_t*>(ws);
  const ScanDims d1 = one_block(d);
  const size_t BH = (size_t)d.batch * d.heads, BG = (size_t)d.batch * d.groups;
  const size_t st_bytes = scan_tc_states_bytes(d1), inner_bytes = tc_bwd_layout(d1).total;
  const bool saved = states_in && zfinal_in;
  for (int blk = 0; blk < 2; ++blk) {
    float* z0b = z0 ? reinterpret_cast<float*>(w + lay.z0) : nullptr;
    float* zfb = saved ? reinterpret_cast<float*>(w + lay.zf) : nullptr;
    float* dfb = dfinal ? reinterpret_cast<float*>(w + lay.dfin) : nullptr;
    float* dib = dinit ? reinterpret_cast<float*>(w + lay.dinit) : nullptr;
    void* bpb = Bprev ? (void*)(w + lay.bprev) : nullptr;
    void* dbpb = Bprev ? (void*)(w + lay.dbprev) : nullptr;
    if (z0 && !copy_block_in(z0b, z0, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
    if (saved && !copy_block_in(zfb, zfinal_in, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
    if (dfinal && !copy_block_in(dfb, dfinal, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
    if (Bprev && !copy_block_in(bpb, Bprev, blk, BG, 2, st)) return SL_ERR_LAUNCH_FAILED;
    const void* stb = saved ? reinterpret_cast<const uint8_t*>(states_in) + blk * st_bytes : nullptr;
    void* dUb = blk == 0 ? dU : (void*)(w + lay.du);
    float* dMb = blk == 0 ? dM : reinterpret_cast<float*>(w + lay.dm);
    float* dKb = blk == 0 ? dK : reinterpret_cast<float*>(w + lay.dk);
    void* dUpb = !Uprev ? nullptr : (blk == 0 ? dUprev : (void*)(w + lay.duprev));
    const int rc = scan_tc_bwd_block(U, M, K, block_of(B, blk), block_of(C, blk), z0b, bpb, Uprev, stb, zfb, dY, dfb,
                                     dUb, dMb, dKb, const_cast<void*>(block_of(dB, blk)),
                                     const_cast<void*>(block_of(dC, blk)), dib, dbpb, dUpb, d1, io_dtype,
                                     w + lay.inner, inner_bytes, st, 256);
    if (rc != SL_OK) return rc;
    if (dinit && !copy_block_out(dinit, dib, blk, BH * 64, 4, st)) return SL_ERR_LAUNCH_FAILED;
    if (Bprev && dBprev && !copy_block_out(dBprev, dbpb, blk, BG, 2, st)) return SL_ERR_LAUNCH_FAILED;
  }
  const bool bf = io_dtype == SL_BF16;
  if (bf) add_into<__nv_bfloat16>(dU, w + lay.du, BH * (size_t)d.T * 64, st);
  else add_into<__half>(dU, w + lay.du, BH * (size_t)d.T * 64, st);
  add_into<float>(dM, w + lay.dm, BH * (size_t)d.T * 2, st);
  add_into<float>(dK, w + lay.dk, BH * (size_t)d.T * 4, st);
  if (Uprev && dUprev) {
    if (bf) add_into<__nv_bfloat16>(dUprev, w + lay.duprev, BH * 64, st);
    else add_into<__half>(dUprev, w + lay.duprev, BH * 64, st);
  }
  return launch_status();
}

// The site code of the first expired wait on the current device since the last reset (0 = none).
int scan_tc_device_status(bool reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (reset && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace sl
