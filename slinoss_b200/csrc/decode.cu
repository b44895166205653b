// One-token decode of the v2x2ssd scan over the carried float32 state.
//
//   z' = m z + u_prev (x) (kp b_prev) + u (x) (kc b),   y[p] = Re sum_n conj(c[n]) z'[p,n]
//
// (the T = 1 case of the sequential scan, slinoss/ops/v2x2ssd/reference.py:815-840,
// which is what the reference's decode step evaluates, slinoss/ops/mixer/step.py:231).
// The kernel is bandwidth bound: every state element is read once and written
// once with 16-byte accesses; one CTA owns one (batch, head), a warp owns one row
// of P at a time and its lanes stride over the 2N columns.
#include "common.cuh"

namespace sl {
namespace {

// State update and read-out of a warp's rows when a state row is KQ float4 per lane (2N = 128 KQ): 8 / KQ rows
// at a time, all loads first.
template <int KQ, typename TIn, typename TY>
__device__ __forceinline__ void decode_rows(const TIn* __restrict__ U, const TIn* __restrict__ Uprev,
                                            const float* state_in, float* state_out, TY* __restrict__ Y,
                                            const float* s_bp, const float* s_bc, const float* s_c, float mr,
                                            float mi, size_t bh, int P, int lane, int w, int nw) {
  constexpr int R = 8 / KQ;
  constexpr int D = 128 * KQ;
  float4 a[KQ], c[KQ], cc[KQ];
#pragma unroll
  for (int q = 0; q < KQ; ++q) {
    a[q] = reinterpret_cast<const float4*>(s_bp)[lane + 32 * q];
    c[q] = reinterpret_cast<const float4*>(s_bc)[lane + 32 * q];
    cc[q] = reinterpret_cast<const float4*>(s_c)[lane + 32 * q];
  }
  for (int p0 = R * w; p0 < P; p0 += R * nw) {
    float4 z[R][KQ];
    float u[R], up[R];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int q = 0; q < KQ; ++q)
        z[r][q] = reinterpret_cast<const float4*>(state_in + (bh * P + p0 + r) * D)[lane + 32 * q];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      u[r] = to_f32(U[bh * P + p0 + r]);
      up[r] = Uprev ? to_f32(Uprev[bh * P + p0 + r]) : 0.f;
    }
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      acc[r] = 0.f;
#pragma unroll
      for (int q = 0; q < KQ; ++q) {
        const float4 zz = z[r][q];
        float4 o;
        o.x = mr * zz.x - mi * zz.y + up[r] * a[q].x + u[r] * c[q].x;
        o.y = mr * zz.y + mi * zz.x + up[r] * a[q].y + u[r] * c[q].y;
        o.z = mr * zz.z - mi * zz.w + up[r] * a[q].z + u[r] * c[q].z;
        o.w = mr * zz.w + mi * zz.z + up[r] * a[q].w + u[r] * c[q].w;
        reinterpret_cast<float4*>(state_out + (bh * P + p0 + r) * D)[lane + 32 * q] = o;
        acc[r] += cc[q].x * o.x + cc[q].y * o.y + cc[q].z * o.z + cc[q].w * o.w;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    if (lane < R) {
      float v = acc[0];
#pragma unroll
      for (int r = 1; r < R; ++r) v = lane == r ? acc[r] : v;
      Y[bh * P + p0 + lane] = from_f32<TY>(v);
    }
  }
}

template <typename TIn, typename TY>
__global__ void __launch_bounds__(256) decode_kernel(
    const TIn* __restrict__ U, const float* __restrict__ M, const float* __restrict__ K,
    const TIn* __restrict__ B, const TIn* __restrict__ C, const float* state_in,
    const TIn* __restrict__ Bprev, const TIn* __restrict__ Uprev, TY* __restrict__ Y,
    float* state_out, int heads, int groups, int P, int N) {
  extern __shared__ __align__(16) float smem[];
  const int D = 2 * N;
  float* s_bp = smem;
  float* s_bc = smem + D;
  float* s_c = smem + 2 * D;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  const size_t bh = blockIdx.x;
  const int b = (int)(bh / heads), h = (int)(bh % heads);
  const size_t bg = (size_t)b * groups + h / (heads / groups);
  const float4 k4 = *reinterpret_cast<const float4*>(K + bh * 4);
  for (int n = tid; n < N; n += blockDim.x) {
    const cf bt = {to_f32(B[bg * D + 2 * n]), to_f32(B[bg * D + 2 * n + 1])};
    cf bp = {0.f, 0.f};
    if (Bprev) bp = {to_f32(Bprev[bg * D + 2 * n]), to_f32(Bprev[bg * D + 2 * n + 1])};
    const cf a = cmul({k4.x, k4.y}, bp), c = cmul({k4.z, k4.w}, bt);
    s_bp[2 * n] = a.re; s_bp[2 * n + 1] = a.im;
    s_bc[2 * n] = c.re; s_bc[2 * n + 1] = c.im;
    s_c[2 * n] = to_f32(C[bg * D + 2 * n]); s_c[2 * n + 1] = to_f32(C[bg * D + 2 * n + 1]);
  }
  __syncthreads();
  const float mr = M[bh * 2], mi = M[bh * 2 + 1];
  const bool vec4 = (N % 2) == 0;
  // N = 64 / N = 128: a state row is one / two float4 per lane.  A warp takes 8 / 4 consecutive rows at a
  // time and issues all 8 loads before any arithmetic, so 4 KB per warp are in flight.  (Measured and not
  // kept, both because the extra registers cost the third resident CTA per SM: requesting the first rows
  // ahead of the staging above, 96 -> 124 us; two streams per CTA at N = 64, 96 -> 114 us.)
  if (D == 128 && (P % (8 * nw)) == 0) {
    decode_rows<1>(U, Uprev, state_in, state_out, Y, s_bp, s_bc, s_c, mr, mi, bh, P, lane, w, nw);
    return;
  }
  if (D == 256 && (P % (4 * nw)) == 0) {
    decode_rows<2>(U, Uprev, state_in, state_out, Y, s_bp, s_bc, s_c, mr, mi, bh, P, lane, w, nw);
    return;
  }
#pragma unroll 2
  for (int p = w; p < P; p += nw) {
    const float u = to_f32(U[bh * P + p]);
    const float up = Uprev ? to_f32(Uprev[bh * P + p]) : 0.f;
    const float* zi = state_in + (bh * P + p) * D;
    float* zo = state_out + (bh * P + p) * D;
    float acc = 0.f;
    if (vec4) {
      for (int q = lane; q < D / 4; q += 32) {
        const float4 z = reinterpret_cast<const float4*>(zi)[q];
        const float4 a = reinterpret_cast<const float4*>(s_bp)[q];
        const float4 c = reinterpret_cast<const float4*>(s_bc)[q];
        const float4 cc = reinterpret_cast<const float4*>(s_c)[q];
        float4 o;
        o.x = mr * z.x - mi * z.y + up * a.x + u * c.x;
        o.y = mr * z.y + mi * z.x + up * a.y + u * c.y;
        o.z = mr * z.z - mi * z.w + up * a.z + u * c.z;
        o.w = mr * z.w + mi * z.z + up * a.w + u * c.w;
        reinterpret_cast<float4*>(zo)[q] = o;
        acc += cc.x * o.x + cc.y * o.y + cc.z * o.z + cc.w * o.w;
      }
    } else {
      for (int n = lane; n < N; n += 32) {
        const float2 z = reinterpret_cast<const float2*>(zi)[n];
        float2 o;
        o.x = mr * z.x - mi * z.y + up * s_bp[2 * n] + u * s_bc[2 * n];
        o.y = mr * z.y + mi * z.x + up * s_bp[2 * n + 1] + u * s_bc[2 * n + 1];
        reinterpret_cast<float2*>(zo)[n] = o;
        acc += s_c[2 * n] * o.x + s_c[2 * n + 1] * o.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) Y[bh * P + p] = from_f32<TY>(acc);
  }
}

}  // namespace
}  // namespace sl

extern "C" int sl_v2x2ssd_decode(const void* U, const float* M, const float* K, const void* B,
                                 const void* C, const float* state_in, const void* B_prev,
                                 const void* U_prev, void* Y, float* state_out, int batch,
                                 int heads, int groups, int P, int N, int io_dtype,
                                 int y_dtype, void* stream) {
  using namespace sl;
  if (!U || !M || !K || !B || !C || !state_in || !Y || !state_out) return SL_ERR_NULL_POINTER;
  if ((B_prev == nullptr) != (U_prev == nullptr)) return SL_ERR_NULL_POINTER;
  if (batch < 1 || heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1)
    return SL_ERR_BAD_SHAPE;
  if (!dtype_ok(io_dtype) || !dtype_ok(y_dtype)) return SL_ERR_UNSUPPORTED;
  if (!aligned(K, 16) || !aligned(state_in, 16) || !aligned(state_out, 16) || !aligned(M, 8))
    return SL_ERR_BAD_ALIGNMENT;
  const size_t smem = 3 * 2 * (size_t)N * sizeof(float);
  if (smem > 48 * 1024) return SL_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)batch * heads;
  SL_DISPATCH_DTYPE(io_dtype, TIn, SL_DISPATCH_DTYPE(y_dtype, TY, {
    decode_kernel<TIn, TY><<<grid, 256, smem, st>>>(
        reinterpret_cast<const TIn*>(U), M, K, reinterpret_cast<const TIn*>(B),
        reinterpret_cast<const TIn*>(C), state_in, reinterpret_cast<const TIn*>(B_prev),
        reinterpret_cast<const TIn*>(U_prev), reinterpret_cast<TY*>(Y), state_out, heads,
        groups, P, N);
  }));
  note_launches(1);
  return launch_status();
}
