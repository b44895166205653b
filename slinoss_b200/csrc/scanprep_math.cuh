// Scan-preparation arithmetic shared by the sequence kernels (scanprep_conv.cu) and the fused decode
// step (mixer_step.cu); included inside their namespaces.
//
// Bounded per-token maps and exact first-order-hold taps (slinoss/layers/scanprep.py:237-283,
// slinoss/ops/scanprep/reference.py:25-56): the bounded maps are evaluated in float32 like the
// reference, the tap quotients kappa1 = (rho - 1)/z and kappa2 = (rho (z - 1) + 1)/z^2, which cancel
// in float32 for small |z|, in float64.
#pragma once

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct zc { double re, im; };
__device__ __forceinline__ zc zmul(zc a, zc b) { return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re}; }
__device__ __forceinline__ zc zdiv(zc a, zc b) {
  const double d = b.re * b.re + b.im * b.im;
  return {(a.re * b.re + a.im * b.im) / d, (a.im * b.re - a.re * b.im) / d};
}
__device__ __forceinline__ zc zconj_mul(zc a, zc b) {  // conj(a) * b
  return {a.re * b.re + a.im * b.im, a.re * b.im - a.im * b.re};
}

struct CoeffOut {
  double dt, r, theta, ea;          // ea = exp(-alpha)
  double dsg_dt, dsg_al, dsg_thu, tanh2; // sigmoid derivatives etc. for the backward
  zc rho, k1, k2, dk1, dk2;         // kappa1, kappa2 and their z-derivatives
};

__device__ __forceinline__ float wrap_angle_f(float theta) {
  // remainder(theta + pi, 2 pi) - pi evaluated in float32 like the reference
  const float pi = 3.14159265358979323846f, two_pi = 6.28318530717958647692f;
  float r = fmodf(theta + pi, two_pi);
  if (r < 0.f) r += two_pi;
  return r - pi;
}

// WITH_DERIVS = false leaves the derivative fields (dsg_*, tanh2, dk1, dk2) unset: the forward kernels
// do not pay for the backward's float64 exponentials and quotients.
template <bool WITH_DERIVS = true>
__device__ __forceinline__ CoeffOut coeff_eval(float p0, float p1, float p2, float th_bias,
                                               float th_sign, const sl_scanprep_config& c) {
  CoeffOut o;
  // bounded maps in float32 (as the reference), then float64 for the taps
  const float sdt = 1.f / (1.f + expf(-p0));
  const float sal = 1.f / (1.f + expf(-p1));
  const float th = tanhf(p2);
  const float thu = 1.f / (1.f + expf(-(th_bias + c.theta_mod_scale * th)));
  const float span = fmaxf(c.theta_init_max - c.theta_init_min, 1.0e-6f);
  const float dt = c.dt_min + (c.dt_max - c.dt_min) * sdt;
  const float alpha = c.alpha_min + (c.alpha_max - c.alpha_min) * sal;
  const float theta = wrap_angle_f(th_sign * (c.theta_init_min + span * thu));
  const float ea = expf(-alpha);
  const float r = c.r_min + (c.r_max - c.r_min) * ea;
  o.dt = dt; o.r = r; o.theta = theta; o.ea = ea;
  // sigma'(x) = sigma(x) sigma(-x) = e / (1 + e)^2 with e = exp(-|x|): exact even where
  // the sigmoid saturates (1 - sigma(x) would cancel in float32)
  if constexpr (WITH_DERIVS) {
    auto dsig = [](double x) { const double e = exp(-fabs(x)); return e / ((1.0 + e) * (1.0 + e)); };
    o.dsg_dt = dsig((double)p0); o.dsg_al = dsig((double)p1);
    o.dsg_thu = dsig((double)th_bias + (double)c.theta_mod_scale * (double)th);
    o.tanh2 = (double)th * th;
  }
  const double a = log((double)r);
  double sn, cs;
  sincos((double)theta, &sn, &cs);
  o.rho = {(double)r * cs, (double)r * sn};
  const zc z = {a, (double)theta};
  const float lr = logf(r);
  const double thr = fmax(1.0e-4, sqrt(fmax((double)c.eps, 1.0e-12)));
  const bool small = (double)(lr * lr + theta * theta) < thr * thr;
  if (small) {
    const zc z2 = zmul(z, z), z3 = zmul(z2, z);
    o.k1 = {1.0 + 0.5 * z.re + z2.re / 6.0 + z3.re / 24.0, 0.5 * z.im + z2.im / 6.0 + z3.im / 24.0};
    o.k2 = {0.5 + z.re / 3.0 + z2.re / 8.0 + z3.re / 30.0, z.im / 3.0 + z2.im / 8.0 + z3.im / 30.0};
    if constexpr (WITH_DERIVS) {
      o.dk1 = {0.5 + z.re / 3.0 + z2.re / 8.0, z.im / 3.0 + z2.im / 8.0};
      o.dk2 = {1.0 / 3.0 + z.re / 4.0 + z2.re / 10.0, z.im / 4.0 + z2.im / 10.0};
    }
  } else {
    const zc rm1 = {o.rho.re - 1.0, o.rho.im};
    o.k1 = zdiv(rm1, z);
    const zc zm1 = {z.re - 1.0, z.im};
    zc num = zmul(o.rho, zm1);
    num.re += 1.0;
    o.k2 = zdiv(num, zmul(z, z));
    if constexpr (WITH_DERIVS) {
      // kappa1' = (rho - kappa1)/z ; kappa2' = (rho - 2 kappa2)/z
      o.dk1 = zdiv({o.rho.re - o.k1.re, o.rho.im - o.k1.im}, z);
      o.dk2 = zdiv({o.rho.re - 2.0 * o.k2.re, o.rho.im - 2.0 * o.k2.im}, z);
    }
  }
  return o;
}

