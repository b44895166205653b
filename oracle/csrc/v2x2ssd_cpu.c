/*
 * C / OpenMP port of the v2x2ssd scan, forward and backward, in float32.
 *
 * TEST / BASELINE INFRASTRUCTURE ONLY: used to time the CPU path on the host
 * cores of the GPU box and as a second checker.  It restates the sequential
 * scan of the reference (slinoss/ops/v2x2ssd/reference.py:815-840):
 *
 *   z_t = m_t z_{t-1} + u_{t-1} (x) (kp_t b_{t-1}) + u_t (x) (kc_t b_t)
 *   y_t[p] = Re sum_n conj(c_t[n]) z_t[p,n]
 *
 * and its adjoint (the gradients the reference gets from autograd).  The
 * backward keeps every z_t of one (batch, head) stream in memory and walks it
 * in reverse, exactly like reverse-mode autodiff of the loop; (batch, head)
 * streams are distributed over the OpenMP threads.  Grouped B/C gradients are
 * summed over the heads of a group.
 *
 * Layouts: U (b,h,T,P), M (b,h,T,2), K (b,h,T,2,2), B,C (b,g,T,2N), state (b,h,P,2N).
 */
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* torchrun exports OMP_NUM_THREADS=1: callers that want all cores say so explicitly */
void oracle_set_num_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* one step of the recurrence on a (P, N) complex state stored interleaved */
static void step(float* z, const float* u, const float* up, const float* b, const float* bp,
                 const float* m, const float* k, int P, int N) {
  const float mr = m[0], mi = m[1];
  for (int p = 0; p < P; ++p) {
    float* zp = z + (size_t)p * 2 * N;
    const float uc = u[p], upv = up ? up[p] : 0.f;
    for (int n = 0; n < N; ++n) {
      const float br = b[2 * n], bi = b[2 * n + 1];
      const float pr = bp ? bp[2 * n] : 0.f, pi = bp ? bp[2 * n + 1] : 0.f;
      const float bcr = k[2] * br - k[3] * bi, bci = k[2] * bi + k[3] * br;
      const float bpr = k[0] * pr - k[1] * pi, bpi = k[0] * pi + k[1] * pr;
      const float zr = zp[2 * n], zi = zp[2 * n + 1];
      zp[2 * n] = mr * zr - mi * zi + upv * bpr + uc * bcr;
      zp[2 * n + 1] = mr * zi + mi * zr + upv * bpi + uc * bci;
    }
  }
}

void oracle_v2x2ssd_fwd(const float* U, const float* M, const float* K, const float* B,
                        const float* C, const float* z0, const float* Bprev, const float* Uprev,
                        float* Y, float* zfinal, int batch, int heads, int groups, int T, int P,
                        int N) {
  const int D = 2 * N, hpg = heads / groups;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < batch * heads; ++bh) {
    const int b = bh / heads, h = bh % heads, bg = b * groups + h / hpg;
    float* z = (float*)calloc((size_t)P * D, sizeof(float));
    if (z0) memcpy(z, z0 + (size_t)bh * P * D, sizeof(float) * P * D);
    for (int t = 0; t < T; ++t) {
      const float* u = U + ((size_t)bh * T + t) * P;
      const float* up = t > 0 ? u - P : (Uprev ? Uprev + (size_t)bh * P : NULL);
      const float* bt = B + ((size_t)bg * T + t) * D;
      const float* bp = t > 0 ? bt - D : (Bprev ? Bprev + (size_t)bg * D : NULL);
      const float* ct = C + ((size_t)bg * T + t) * D;
      step(z, u, up, bt, bp, M + ((size_t)bh * T + t) * 2, K + ((size_t)bh * T + t) * 4, P, N);
      float* y = Y + ((size_t)bh * T + t) * P;
      for (int p = 0; p < P; ++p) {
        const float* zp = z + (size_t)p * D;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) acc += ct[d] * zp[d];
        y[p] = acc;
      }
    }
    if (zfinal) memcpy(zfinal + (size_t)bh * P * D, z, sizeof(float) * P * D);
    free(z);
  }
}

/* Gradients.  dB, dC, dBprev must be zero-initialised by the caller (group sums are
 * accumulated with atomics); every other output is fully written. */
void oracle_v2x2ssd_bwd(const float* U, const float* M, const float* K, const float* B,
                        const float* C, const float* z0, const float* Bprev, const float* Uprev,
                        const float* dY, const float* dfinal, float* dU, float* dM, float* dK,
                        float* dB, float* dC, float* dinit, float* dBprev, float* dUprev,
                        int batch, int heads, int groups, int T, int P, int N) {
  const int D = 2 * N, hpg = heads / groups;
  const size_t S = (size_t)P * D;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < batch * heads; ++bh) {
    const int b = bh / heads, h = bh % heads, bg = b * groups + h / hpg;
    float* zs = (float*)malloc(sizeof(float) * S * ((size_t)T + 1)); /* z_{-1} .. z_{T-1} */
    float* G = (float*)calloc(S, sizeof(float));
    float* dbc = (float*)malloc(sizeof(float) * D);
    float* dbp = (float*)malloc(sizeof(float) * D);
    if (z0) memcpy(zs, z0 + (size_t)bh * S, sizeof(float) * S);
    else memset(zs, 0, sizeof(float) * S);
    for (int t = 0; t < T; ++t) {
      memcpy(zs + S * (t + 1), zs + S * t, sizeof(float) * S);
      const float* u = U + ((size_t)bh * T + t) * P;
      const float* up = t > 0 ? u - P : (Uprev ? Uprev + (size_t)bh * P : NULL);
      const float* bt = B + ((size_t)bg * T + t) * D;
      const float* bp = t > 0 ? bt - D : (Bprev ? Bprev + (size_t)bg * D : NULL);
      step(zs + S * (t + 1), u, up, bt, bp, M + ((size_t)bh * T + t) * 2,
           K + ((size_t)bh * T + t) * 4, P, N);
    }
    if (dfinal) memcpy(G, dfinal + (size_t)bh * S, sizeof(float) * S);
    float mnr = 1.f, mni = 0.f; /* m_{t+1}; the final state is z_{T-1} itself */
    for (int t = T - 1; t >= 0; --t) {
      const float* u = U + ((size_t)bh * T + t) * P;
      const float* up = t > 0 ? u - P : (Uprev ? Uprev + (size_t)bh * P : NULL);
      const float* bt = B + ((size_t)bg * T + t) * D;
      const float* bp = t > 0 ? bt - D : (Bprev ? Bprev + (size_t)bg * D : NULL);
      const float* ct = C + ((size_t)bg * T + t) * D;
      const float* k = K + ((size_t)bh * T + t) * 4;
      const float* dy = dY + ((size_t)bh * T + t) * P;
      const float* zt = zs + S * (t + 1);
      const float* zprev = zs + S * t;
      float* dct = dC + ((size_t)bg * T + t) * D;
      float dmr = 0.f, dmi = 0.f;
      memset(dbc, 0, sizeof(float) * D);
      memset(dbp, 0, sizeof(float) * D);
      float* dut = dU + ((size_t)bh * T + t) * P;
      for (int p = 0; p < P; ++p) {
        float* Gp = G + (size_t)p * D;
        const float* zp = zt + (size_t)p * D;
        const float* zq = zprev + (size_t)p * D;
        const float upv = up ? up[p] : 0.f;
        float duc = 0.f, dup = 0.f;
        for (int n = 0; n < N; ++n) {
          /* G = conj(m_{t+1}) G + dy c */
          const float gr0 = Gp[2 * n], gi0 = Gp[2 * n + 1];
          const float gr = mnr * gr0 + mni * gi0 + dy[p] * ct[2 * n];
          const float gi = mnr * gi0 - mni * gr0 + dy[p] * ct[2 * n + 1];
          Gp[2 * n] = gr; Gp[2 * n + 1] = gi;
#pragma omp atomic
          dct[2 * n] += dy[p] * zp[2 * n];
#pragma omp atomic
          dct[2 * n + 1] += dy[p] * zp[2 * n + 1];
          /* dm += G conj(z_{t-1}) */
          dmr += gr * zq[2 * n] + gi * zq[2 * n + 1];
          dmi += gi * zq[2 * n] - gr * zq[2 * n + 1];
          dbc[2 * n] += u[p] * gr; dbc[2 * n + 1] += u[p] * gi;
          dbp[2 * n] += upv * gr; dbp[2 * n + 1] += upv * gi;
          const float br = bt[2 * n], bi = bt[2 * n + 1];
          const float pr = bp ? bp[2 * n] : 0.f, pi = bp ? bp[2 * n + 1] : 0.f;
          const float bcr = k[2] * br - k[3] * bi, bci = k[2] * bi + k[3] * br;
          const float bpr = k[0] * pr - k[1] * pi, bpi = k[0] * pi + k[1] * pr;
          duc += bcr * gr + bci * gi;
          dup += bpr * gr + bpi * gi;
        }
        if (t == T - 1) dut[p] = duc; else dut[p] += duc;
        if (t > 0) dut[p - P] = dup;      /* first write of row t-1; += duc follows */
        else if (dUprev) dUprev[(size_t)bh * P + p] = dup;
      }
      dM[((size_t)bh * T + t) * 2] = dmr;
      dM[((size_t)bh * T + t) * 2 + 1] = dmi;
      float kcr = 0.f, kci = 0.f, kpr = 0.f, kpi = 0.f;
      float* dbt = dB + ((size_t)bg * T + t) * D;
      float* dbq = t > 0 ? dbt - D : (dBprev ? dBprev + (size_t)bg * D : NULL);
      for (int n = 0; n < N; ++n) {
        const float br = bt[2 * n], bi = bt[2 * n + 1];
        const float pr = bp ? bp[2 * n] : 0.f, pi = bp ? bp[2 * n + 1] : 0.f;
        kcr += dbc[2 * n] * br + dbc[2 * n + 1] * bi;
        kci += dbc[2 * n + 1] * br - dbc[2 * n] * bi;
        kpr += dbp[2 * n] * pr + dbp[2 * n + 1] * pi;
        kpi += dbp[2 * n + 1] * pr - dbp[2 * n] * pi;
        /* db_t += conj(kc) dbc ; db_{t-1} += conj(kp) dbp */
#pragma omp atomic
        dbt[2 * n] += k[2] * dbc[2 * n] + k[3] * dbc[2 * n + 1];
#pragma omp atomic
        dbt[2 * n + 1] += k[2] * dbc[2 * n + 1] - k[3] * dbc[2 * n];
        if (dbq) {
#pragma omp atomic
          dbq[2 * n] += k[0] * dbp[2 * n] + k[1] * dbp[2 * n + 1];
#pragma omp atomic
          dbq[2 * n + 1] += k[0] * dbp[2 * n + 1] - k[1] * dbp[2 * n];
        }
      }
      float* dk = dK + ((size_t)bh * T + t) * 4;
      dk[0] = kpr; dk[1] = kpi; dk[2] = kcr; dk[3] = kci;
      mnr = M[((size_t)bh * T + t) * 2]; mni = M[((size_t)bh * T + t) * 2 + 1];
    }
    if (dinit) {
      for (size_t i = 0; i < S; i += 2) {
        dinit[(size_t)bh * S + i] = mnr * G[i] + mni * G[i + 1];
        dinit[(size_t)bh * S + i + 1] = mnr * G[i + 1] - mni * G[i];
      }
    }
    free(zs); free(G); free(dbc); free(dbp);
  }
}
