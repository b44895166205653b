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
  if (D == 128 && (P % (8 * nw)) == 0) {
    // N = 64: a state row is one float4 per lane.  A warp takes 8 consecutive rows at a time and
    // issues all 8 loads before any arithmetic, so 4 KB per warp are in flight.
    const float4 a = reinterpret_cast<const float4*>(s_bp)[lane];
    const float4 c = reinterpret_cast<const float4*>(s_bc)[lane];
    const float4 cc = reinterpret_cast<const float4*>(s_c)[lane];
    for (int p0 = 8 * w; p0 < P; p0 += 8 * nw) {
      float4 z[8];
      float u[8], up[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        z[r] = reinterpret_cast<const float4*>(state_in + (bh * P + p0 + r) * D)[lane];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        u[r] = to_f32(U[bh * P + p0 + r]);
        up[r] = Uprev ? to_f32(Uprev[bh * P + p0 + r]) : 0.f;
      }
      float acc[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        float4 o;
        o.x = mr * z[r].x - mi * z[r].y + up[r] * a.x + u[r] * c.x;
        o.y = mr * z[r].y + mi * z[r].x + up[r] * a.y + u[r] * c.y;
        o.z = mr * z[r].z - mi * z[r].w + up[r] * a.z + u[r] * c.z;
        o.w = mr * z[r].w + mi * z[r].z + up[r] * a.w + u[r] * c.w;
        reinterpret_cast<float4*>(state_out + (bh * P + p0 + r) * D)[lane] = o;
        acc[r] = cc.x * o.x + cc.y * o.y + cc.z * o.z + cc.w * o.w;
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[r] = warp_sum(acc[r]);
      if (lane < 8) {
        float v = acc[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) v = lane == r ? acc[r] : v;
        Y[bh * P + p0 + lane] = from_f32<TY>(v);
      }
    }
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
