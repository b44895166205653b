// One decode token of the whole mixer between in_proj and out_proj, in ONE launch:
//
//   causal conv update + bias + SiLU  ->  u          (per channel, carried conv window)
//   scan preparation of the token     ->  m, kp, kc  (per head)   and  b, c  (per group)
//   state update + read-out            z' = m z + u_prev (x) (kp b_prev) + u (x) (kc b),  y = Re<c, z'>
//   skip + gate                        hid = (y + d_skip u) SiLU(gate)
//   RMSNorm over the inner width       normed = hid * rsqrt(mean hid^2 + eps) * w
//
// (what run_reference_decode_step evaluates with separate torch ops, slinoss/ops/mixer/step.py:201-258 and
// 323-429, and what mixer_decode_step_cute fuses for d_skip-free mixers only,
// slinoss/ops/v2x2ssd/cute/step.py:224-627; out_proj stays a library GEMM in the caller.)
//
// One CTA per (batch, head).  The RMSNorm needs the sum of squares over ALL heads of a batch row: every
// CTA writes its 64 gated values to a scratch row and adds its partial sum to a per-row accumulator; the
// CTA that takes the last ticket of the row (an atomic counter, no waiting on other CTAs) normalises the
// whole row and puts accumulator and counter back to zero for the next call.  The state is updated in
// place, 16 bytes per lane, every element read once and written once: the kernel is bound by that traffic.
//
// Values are rounded to the io dtype where the sequence kernels round them (u, b, c, y, the skip sum, the
// gated value), so that a decoded token equals the same token of a forward pass.
#include "common.cuh"

namespace sl {
namespace {

#include "scanprep_math.cuh"

template <typename T> __device__ __forceinline__ float round_io(float v) { return to_f32(from_f32<T>(v)); }

struct StepParams {
  const void *gate, *value;          // (batch, C) with row strides (column slices of the in_proj output)
  long long gate_stride, value_stride;
  const void *params, *bc;           // (batch, 3H), (batch, G, 4, N)
  const void *conv_w, *conv_b;       // (C, W), (C)
  void* conv_state;                  // (batch, C, W-1), updated in place
  const float *dt_bias, *alpha_bias, *theta_mod_bias, *theta_bias, *theta_sign, *d_skip;
  const void* norm_w;                // (C)
  sl_scanprep_config cfg;
  float norm_eps;
  float* state;                      // (batch, H, P, 2N), updated in place
  const void* b_prev_in;             // (batch, G, 2N)
  void* b_prev_out;                  // (batch, G, 2N): this token's b (a buffer of its own: heads of a group race otherwise)
  void* u_prev;                      // (batch, H, P), updated in place
  void* normed;                      // (batch, C)
  float* hid;                        // scratch (batch, C)
  float* sumsq;                      // scratch (batch), zero between calls
  unsigned* tickets;                 // scratch (batch), zero between calls
  int batch, H, G, P, N, W;
};

template <typename T>
__global__ void __launch_bounds__(256, 4) mixer_step_kernel(StepParams p) {
  extern __shared__ __align__(16) float smem[];
  const int D = 2 * p.N, C = p.H * p.P;
  float* s_bp = smem;            // kp * b_prev
  float* s_bc = smem + D;        // kc * b
  float* s_c = smem + 2 * D;     // c
  float* s_b = smem + 3 * D;     // b (rounded)
  float* s_u = smem + 4 * D;     // [P] u, then [P] u_prev, then [P] y
  float* s_up = s_u + p.P;
  float* s_y = s_up + p.P;
  __shared__ float s_coef[6];    // m, kp, kc
  __shared__ float s_red[8];
  __shared__ unsigned s_ticket;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, nw = blockDim.x >> 5;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int g = h / (p.H / p.G);
  const size_t bg = (size_t)b * p.G + g;

  // ---- requests.  Nothing below depends on anything but the inputs until phase D, so every global value
  // the phases A, C, D, E and F read is requested here, ahead of any arithmetic: the CTA then pays for one
  // round trip to memory instead of one per phase (the phases are separated by barriers, and a CTA per
  // (batch, head) has too little work to hide five of them).
  float* state = p.state + (size_t)bh * p.P * D;
  const bool rows8 = D == 128 && (p.P % (8 * nw)) == 0;   // N = 64: a state row is one float4 per lane
  float4 z[8];
  if (rows8) {
#pragma unroll
    for (int r = 0; r < 8; ++r) z[r] = reinterpret_cast<const float4*>(state + (size_t)(8 * w + r) * D)[lane];
  }
  const bool one_pass = p.P <= (int)blockDim.x && p.N <= 64;   // one channel / one b pair per thread
  const T* convw = reinterpret_cast<const T*>(p.conv_w);
  float r_x = 0.f, r_bias = 0.f, r_win[3] = {0.f, 0.f, 0.f}, r_wgt[4] = {0.f, 0.f, 0.f, 0.f};
  float r_up = 0.f, r_gate = 0.f, r_dsk = 0.f, r_bp[2] = {0.f, 0.f}, r_bc[4] = {0.f, 0.f, 0.f, 0.f};
  if (one_pass) {
    if (tid < p.P) {
      const int c = h * p.P + tid;
      r_x = to_f32(reinterpret_cast<const T*>(p.value)[(size_t)b * p.value_stride + c]);
      r_gate = to_f32(reinterpret_cast<const T*>(p.gate)[(size_t)b * p.gate_stride + c]);
      r_up = to_f32(reinterpret_cast<const T*>(p.u_prev)[(size_t)bh * p.P + tid]);
      if (p.d_skip) r_dsk = p.d_skip[h];
      if (convw) {
        const T* st = reinterpret_cast<const T*>(p.conv_state) + ((size_t)b * C + c) * (p.W - 1);
        if (p.conv_b) r_bias = to_f32(reinterpret_cast<const T*>(p.conv_b)[c]);
        for (int j = 0; j < p.W - 1; ++j) r_win[j] = to_f32(st[j]);
        for (int j = 0; j < p.W; ++j) r_wgt[j] = to_f32(convw[(size_t)c * p.W + j]);
      }
    }
    if (w == 2 || w == 3) {
      const T* src = reinterpret_cast<const T*>(p.bc) + bg * 4 * p.N + (size_t)(2 * (w - 2)) * p.N;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int n = lane + 32 * q;
        if (n < p.N) { r_bc[2 * q] = to_f32(src[n]); r_bc[2 * q + 1] = to_f32(src[p.N + n]); }
      }
    }
    if (tid >= 128 && tid < 128 + p.N && p.b_prev_in) {   // (warps 4, 5: not the ones busy with b and c)
      const T* bpin = reinterpret_cast<const T*>(p.b_prev_in) + bg * D + 2 * (tid - 128);
      r_bp[0] = to_f32(bpin[0]); r_bp[1] = to_f32(bpin[1]);
    }
  }

  // ---- A. conv update of this head's channels ------------------------------------------------
  if (one_pass) {
    if (tid < p.P) {
      const int c = h * p.P + tid;
      float u = r_x;
      if (convw) {
        T* st = reinterpret_cast<T*>(p.conv_state) + ((size_t)b * C + c) * (p.W - 1);
        float a = r_bias;
        for (int j = 0; j < p.W - 1; ++j) a += r_wgt[j] * r_win[j];
        a += r_wgt[p.W - 1] * r_x;
        u = round_io<T>(silu_f(a));
        for (int j = 0; j + 1 < p.W - 1; ++j) st[j] = from_f32<T>(r_win[j + 1]);
        if (p.W > 1) st[p.W - 2] = from_f32<T>(r_x);
      }
      s_u[tid] = u;
      s_up[tid] = r_up;
      reinterpret_cast<T*>(p.u_prev)[(size_t)bh * p.P + tid] = from_f32<T>(u);
    }
  } else {
    for (int pp = tid; pp < p.P; pp += blockDim.x) {
      const int c = h * p.P + pp;
      T* st = reinterpret_cast<T*>(p.conv_state) + ((size_t)b * C + c) * (p.W - 1);
      const float x = to_f32(reinterpret_cast<const T*>(p.value)[(size_t)b * p.value_stride + c]);
      float u = x;
      if (convw) {
        float a = p.conv_b ? to_f32(reinterpret_cast<const T*>(p.conv_b)[c]) : 0.f;
        float win[4] = {0.f, 0.f, 0.f, 0.f};      // the carried inputs, oldest first
        for (int j = 0; j < p.W - 1; ++j) { win[j] = to_f32(st[j]); a += to_f32(convw[(size_t)c * p.W + j]) * win[j]; }
        a += to_f32(convw[(size_t)c * p.W + p.W - 1]) * x;
        u = round_io<T>(silu_f(a));
        for (int j = 0; j + 1 < p.W - 1; ++j) st[j] = from_f32<T>(win[j + 1]);
        if (p.W > 1) st[p.W - 2] = from_f32<T>(x);
      }
      T* up = reinterpret_cast<T*>(p.u_prev) + (size_t)bh * p.P + pp;
      s_u[pp] = u;
      s_up[pp] = to_f32(*up);
      *up = from_f32<T>(u);
    }
  }
  // ---- B. transition and taps of this head (one thread; float64 inside) ------------------------
  if (tid == blockDim.x - 1) {
    const T* pr = reinterpret_cast<const T*>(p.params) + (size_t)b * 3 * p.H + 3 * h;
    const CoeffOut o = coeff_eval<false>(to_f32(pr[0]) + p.dt_bias[h], to_f32(pr[1]) + p.alpha_bias[h],
                                  to_f32(pr[2]) + p.theta_mod_bias[h], p.theta_bias[h], p.theta_sign[h], p.cfg);
    const zc kp = {o.dt * o.k2.re, o.dt * o.k2.im};
    s_coef[0] = (float)o.rho.re; s_coef[1] = (float)o.rho.im;
    s_coef[2] = (float)kp.re; s_coef[3] = (float)kp.im;
    s_coef[4] = (float)(o.dt * o.k1.re - kp.re); s_coef[5] = (float)(o.dt * o.k1.im - kp.im);
  }
  // ---- C. b and c of this head's group (warps 2, 3: one each) ------------------------------------
  if (w == 2 || w == 3) {
    const int which = w - 2;      // 0: b (rows 0, 1 of bc), 1: c (rows 2, 3)
    const T* src = reinterpret_cast<const T*>(p.bc) + bg * 4 * p.N + (size_t)(2 * which) * p.N;
    float* dst = which ? s_c : s_b;
    float ss = 0.f;
    if (one_pass) {
      float amp[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        amp[q] = lane + 32 * q < p.N ? softplus_f(r_bc[2 * q]) : 0.f;
        ss += amp[q] * amp[q];
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(fmaxf(ss / (float)p.N, p.cfg.eps));
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int n = lane + 32 * q;
        if (n < p.N) {
          float sn, cs;
          sincosf(3.14159265358979323846f * tanhf(r_bc[2 * q + 1]), &sn, &cs);
          dst[2 * n] = round_io<T>(amp[q] * inv * cs);
          dst[2 * n + 1] = round_io<T>(amp[q] * inv * sn);
        }
      }
    } else {
      for (int n = lane; n < p.N; n += 32) { const float a = softplus_f(to_f32(src[n])); ss += a * a; }
      ss = warp_sum(ss);
      const float inv = rsqrtf(fmaxf(ss / (float)p.N, p.cfg.eps));
      for (int n = lane; n < p.N; n += 32) {
        const float a = softplus_f(to_f32(src[n])) * inv;
        const float ph = 3.14159265358979323846f * tanhf(to_f32(src[p.N + n]));
        float sn, cs;
        sincosf(ph, &sn, &cs);
        dst[2 * n] = round_io<T>(a * cs);
        dst[2 * n + 1] = round_io<T>(a * sn);
      }
    }
  }
  __syncthreads();
  // ---- D. tap-weighted b vectors; the group's first head hands b on as the next token's b_prev ----
  {
    const cf kp = {s_coef[2], s_coef[3]}, kc = {s_coef[4], s_coef[5]};
    const T* bpin = reinterpret_cast<const T*>(p.b_prev_in);
    T* bpout = reinterpret_cast<T*>(p.b_prev_out);
    const bool hand_on = h % (p.H / p.G) == 0;
    auto taps = [&](int n, cf bp) {
      const cf bt = {s_b[2 * n], s_b[2 * n + 1]};
      const cf a = cmul(kp, bp), c2 = cmul(kc, bt);
      s_bp[2 * n] = a.re; s_bp[2 * n + 1] = a.im;
      s_bc[2 * n] = c2.re; s_bc[2 * n + 1] = c2.im;
      if (hand_on) { bpout[bg * D + 2 * n] = from_f32<T>(bt.re); bpout[bg * D + 2 * n + 1] = from_f32<T>(bt.im); }
    };
    if (one_pass) {
      if (tid >= 128 && tid < 128 + p.N) taps(tid - 128, cf{r_bp[0], r_bp[1]});
    } else {
      for (int n = tid; n < p.N; n += blockDim.x) {
        cf bp = {0.f, 0.f};
        if (bpin) bp = {to_f32(bpin[bg * D + 2 * n]), to_f32(bpin[bg * D + 2 * n + 1])};
        taps(n, bp);
      }
    }
  }
  __syncthreads();
  // ---- E. state update and read-out --------------------------------------------------------------
  const float mr = s_coef[0], mi = s_coef[1];
  if (rows8) {
    // a warp takes 8 rows at a time, all loads first (the first 8 were requested at the top)
    const float4 a = reinterpret_cast<const float4*>(s_bp)[lane];
    const float4 c = reinterpret_cast<const float4*>(s_bc)[lane];
    const float4 cc = reinterpret_cast<const float4*>(s_c)[lane];
    for (int p0 = 8 * w; p0 < p.P; p0 += 8 * nw) {
      if (p0 != 8 * w) {
#pragma unroll
        for (int r = 0; r < 8; ++r) z[r] = reinterpret_cast<const float4*>(state + (size_t)(p0 + r) * D)[lane];
      }
      float acc[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float u = s_u[p0 + r], up = s_up[p0 + r];
        float4 o;
        o.x = mr * z[r].x - mi * z[r].y + up * a.x + u * c.x;
        o.y = mr * z[r].y + mi * z[r].x + up * a.y + u * c.y;
        o.z = mr * z[r].z - mi * z[r].w + up * a.z + u * c.z;
        o.w = mr * z[r].w + mi * z[r].z + up * a.w + u * c.w;
        reinterpret_cast<float4*>(state + (size_t)(p0 + r) * D)[lane] = o;
        acc[r] = cc.x * o.x + cc.y * o.y + cc.z * o.z + cc.w * o.w;
      }
#pragma unroll
      for (int r = 0; r < 8; ++r) acc[r] = warp_sum(acc[r]);
      if (lane < 8) {
        float v = acc[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) v = lane == r ? acc[r] : v;
        s_y[p0 + lane] = round_io<T>(v);
      }
    }
  } else {
    for (int pp = w; pp < p.P; pp += nw) {
      const float u = s_u[pp], up = s_up[pp];
      float* zr = state + (size_t)pp * D;
      float acc = 0.f;
      for (int n = lane; n < p.N; n += 32) {
        const float2 z = reinterpret_cast<const float2*>(zr)[n];
        float2 o;
        o.x = mr * z.x - mi * z.y + up * s_bp[2 * n] + u * s_bc[2 * n];
        o.y = mr * z.y + mi * z.x + up * s_bp[2 * n + 1] + u * s_bc[2 * n + 1];
        reinterpret_cast<float2*>(zr)[n] = o;
        acc += s_c[2 * n] * o.x + s_c[2 * n + 1] * o.y;
      }
      acc = warp_sum(acc);
      if (lane == 0) s_y[pp] = round_io<T>(acc);
    }
  }
  __syncthreads();
  // ---- F. skip, gate, partial sum of squares ------------------------------------------------------
  float ss = 0.f;
  for (int pp = tid; pp < p.P; pp += blockDim.x) {
    const int c = h * p.P + pp;
    float pre = s_y[pp];
    if (p.d_skip) pre = round_io<T>(pre + s_u[pp] * (one_pass ? r_dsk : p.d_skip[h]));
    const float gt = one_pass ? r_gate : to_f32(reinterpret_cast<const T*>(p.gate)[(size_t)b * p.gate_stride + c]);
    const float hv = round_io<T>(pre * silu_f(gt));
    p.hid[(size_t)b * C + c] = hv;
    ss += hv * hv;
  }
  ss = warp_sum(ss);
  if (lane == 0) s_red[w] = ss;
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int k = 0; k < nw; ++k) tot += s_red[k];
    atomicAdd(p.sumsq + b, tot);
    __threadfence();                                   // hid and the sum before the ticket
    s_ticket = atomicAdd(p.tickets + b, 1u);
  }
  __syncthreads();
  // ---- G. the CTA with the row's last ticket normalises the row ------------------------------------
  if (s_ticket == (unsigned)p.H - 1) {
    __threadfence();
    const float total = atomicAdd(p.sumsq + b, 0.f);   // (an atomic read: the other CTAs' adds are in L2)
    const float rstd = rsqrtf(total / (float)C + p.norm_eps);
    const T* wn = reinterpret_cast<const T*>(p.norm_w);
    T* out = reinterpret_cast<T*>(p.normed) + (size_t)b * C;
    const volatile float* hid = p.hid + (size_t)b * C;
    for (int c = tid; c < C; c += blockDim.x) out[c] = from_f32<T>(hid[c] * rstd * to_f32(wn[c]));
    __syncthreads();
    if (tid == 0) { p.sumsq[b] = 0.f; p.tickets[b] = 0u; }
  }
}

}  // namespace

size_t mixer_step_workspace(int batch, int heads, int P) {
  return round_up((size_t)batch * heads * P * 4, 256) + round_up((size_t)batch * 4, 256) +
         round_up((size_t)batch * 4, 256);
}

}  // namespace sl

extern "C" size_t sl_mixer_decode_step_workspace_bytes(int batch, int heads, int P) {
  if (batch < 1 || heads < 1 || P < 1) return 0;
  return sl::mixer_step_workspace(batch, heads, P);
}

extern "C" int sl_mixer_decode_step(const void* gate, int64_t gate_row_stride, const void* value,
                                    int64_t value_row_stride, const void* params, const void* bc,
                                    const void* conv_weight, const void* conv_bias, void* conv_state,
                                    int d_conv, const float* dt_bias, const float* alpha_bias,
                                    const float* theta_mod_bias, const float* theta_bias,
                                    const float* theta_sign, const sl_scanprep_config* cfg,
                                    const float* d_skip, const void* norm_weight, float norm_eps,
                                    float* state, const void* b_prev_in, void* b_prev_out, void* u_prev,
                                    void* normed, void* workspace, size_t workspace_bytes, int batch,
                                    int heads, int groups, int P, int N, int io_dtype, void* stream) {
  using namespace sl;
  if (!gate || !value || !params || !bc || !dt_bias || !alpha_bias || !theta_mod_bias || !theta_bias ||
      !theta_sign || !cfg || !norm_weight || !state || !b_prev_out || !u_prev || !normed)
    return SL_ERR_NULL_POINTER;
  if (conv_weight && d_conv > 1 && !conv_state) return SL_ERR_NULL_POINTER;
  if (batch < 1 || heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1 || d_conv < 1 || d_conv > 4)
    return SL_ERR_BAD_SHAPE;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  if (!aligned(state, 16)) return SL_ERR_BAD_ALIGNMENT;
  if (!workspace || workspace_bytes < mixer_step_workspace(batch, heads, P)) return SL_ERR_WORKSPACE_TOO_SMALL;
  const size_t smem = ((size_t)4 * 2 * N + 3 * (size_t)P) * sizeof(float);
  if (smem > 48 * 1024) return SL_ERR_UNSUPPORTED;
  StepParams p{};
  p.gate = gate; p.value = value; p.gate_stride = gate_row_stride; p.value_stride = value_row_stride;
  p.params = params; p.bc = bc; p.conv_w = conv_weight; p.conv_b = conv_bias; p.conv_state = conv_state;
  p.dt_bias = dt_bias; p.alpha_bias = alpha_bias; p.theta_mod_bias = theta_mod_bias; p.theta_bias = theta_bias;
  p.theta_sign = theta_sign; p.d_skip = d_skip; p.norm_w = norm_weight; p.cfg = *cfg; p.norm_eps = norm_eps;
  p.state = state; p.b_prev_in = b_prev_in; p.b_prev_out = b_prev_out; p.u_prev = u_prev; p.normed = normed;
  uint8_t* w = reinterpret_cast<uint8_t*>(workspace);
  p.hid = reinterpret_cast<float*>(w);
  p.sumsq = reinterpret_cast<float*>(w + round_up((size_t)batch * heads * P * 4, 256));
  p.tickets = reinterpret_cast<unsigned*>(w + round_up((size_t)batch * heads * P * 4, 256) + round_up((size_t)batch * 4, 256));
  p.batch = batch; p.H = heads; p.G = groups; p.P = P; p.N = N; p.W = conv_weight ? d_conv : 1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)batch * heads;
  SL_DISPATCH_DTYPE(io_dtype, T, { mixer_step_kernel<T><<<grid, 256, smem, st>>>(p); });
  note_launches(1);
  return launch_status();
}
