// Backward of the chunked scan on tcgen05 (included by scan_tc.cu inside its namespaces).
//
// With V_t = m_t W_{t-1} (state after the decay, before the injection of token t):
//     y_t = Re<c_t, V_t> + u_t Re(conj(c_t) kc_t b_t),      W_t = V_t + u_t (x) (g_t b_t).
// One CTA walks the chunks of one (batch, head) in REVERSE order carrying
// dz = adjoint of the chunk-end state (conjugated pairs, float32, in registers).
// Per chunk, with the same rotated operands as the forward (unit phases on the 16-bit
// operands, decays exp(<=0) on float32 accumulators):
//     P~ = Q K'^T,  dS = dY U^T      -> Pdec = mask_{s<t} e^{l_t-l_s} P~ ,  dP = mask_{s<t} e^{l_t-l_s} dS
//     dQ = dP K' + e^{l_t} (dY Zv)                     -> dC  (un-rotate, + diagonal term)
//     dX = dP^T Q + (e^{l_end-l_s} U) dWv              -> dB, dg   (dWv = dz rotated by the unit phase of Pi_end;
//                                                        the decay is folded into the 16-bit rows of U)
//     dU = Pdec^T dY + e^{l_end-l_s} (K' dWv^T)        (+ dy_s diag_s)
//     dz <- e^{l_end} dWv + (e^{l_t} dY)^T Q           (adjoint of the chunk-start state)
// Per-token scalars for dM / dK go to the workspace and are finished by
// scan_tc_bwd_finish_kernel using
//     conj(m_t) dm_t = S_t,   S_t = S_{t+1} + <q_t, dq_t> - conj(g_t) dg_t,
// anchored at every chunk end by S = <dZ, Z> of the state carried across that boundary.

constexpr uint32_t B_STAGE = 8 * TILE;                 // U | B(2) | C(2) | dY | Zv(2)
constexpr uint32_t B_OFF_Q = 2 * B_STAGE;              // Q (2)
constexpr uint32_t B_OFF_KP = B_OFF_Q + 2 * TILE;      // K' (2)
constexpr uint32_t B_OFF_DYO = B_OFF_KP + 2 * TILE;    // e^{l_t} dY (1)
constexpr uint32_t B_OFF_PD = B_OFF_DYO + TILE;        // Pdec (1)
constexpr uint32_t B_OFF_DP = B_OFF_PD + TILE;         // dP (1)
constexpr uint32_t B_OFF_DW = B_OFF_DP + TILE;         // dWv (2)
constexpr uint32_t B_OFF_UE = B_OFF_DW + 2 * TILE;      // e^{l_end-l_s} U (1)
constexpr uint32_t B_OFF_SCAL = B_OFF_UE + TILE;
constexpr int B_NSCAL = 2 * 11 + 5 + 32;   // 2 x 11 look-ahead rows, 5 worker rows, 4 x 8 partial sums
constexpr uint32_t B_SMEM_BYTES = B_OFF_SCAL + B_NSCAL * 64 * 4 + 1024;
// TMEM columns: P~ then dUa 0 | dS then dUb 64 | dQ 128..255 | dX 256..383 | dZ 384..511.  All products have
// M = 64 (rows in lanes 0..15 of a quadrant).  P~, dS, dUa and dUb are N = 64 and read with the 16x256b load
// shape; dQ, dX and dZ are N = 128 products (each the sum of two operand pairs but for dZ) read with the
// 16x32bx2 shape (thread t: row t % 16 of column half t / 16).  dUa and dUb reuse the columns of P~ and dS,
// which are dead after epilogue 1.
constexpr uint32_t B_TMEM_COLS = 512;

struct alignas(64) TcBwdParams {
  CUtensorMap tmU, tmB, tmC, tmdY, tmZ;
  CUtensorMap tmdU, tmdB, tmdC;   // outputs, written with TMA stores from shared memory
  const float* M;
  const float* K;
  const float* dfinal;   // (BH, 64, 128) or null
  const float* zfinal;   // forward final state (pre-sweep), read when dfinal is given
  float2 *dg, *sterm, *dkcd, *anchor;   // per token / per chunk scalars (workspace)
  float* dinit;          // (BH, 64, 128) adjoint of the carried start state, or null
  int T, nchunks;
  int heads, groups;     // B and C are shared by the heads of a group; dB / dC leave per head
  long long wait_limit;  // SM clocks a wait of the main loop may take before the kernel gives up
};

// Per-token table: rows 0..10 as written by chunk_scalars, then
//  11 e^{l_end-l_t}   12 sigma_t = <dy_t,u_t>   13 diag_t   14,15 sum_n c conj(b)
//  s_acc (after row 15): partial sums per (column group, half): re/im of <q,dq>, re/im of sum conj(b) dX
// NW = warps per TMEM lane quadrant (same thread-to-data mapping as the forward kernel).
template <typename TIn, int NW>
__global__ void __launch_bounds__(128 * NW + 64, 1) scan_tc_bwd_kernel(const __grid_constant__ TcBwdParams p) {
  constexpr int NT = 128 * NW;               // worker threads; two more warps: scalars, TMA + MMA issue
  constexpr int ZC = 64 / NW;                // columns per thread of a 64-wide accumulator half
  constexpr int SC = 32 / NW;                // columns per thread of a 32-wide accumulator half
  constexpr int PC = ZC > 32 ? 32 : ZC;      // columns handled per TMEM load in the wide epilogues
  constexpr int RSTEP = NT / 16;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar_tma[2], bar_mma[5];   // bar_mma: P~,dS | dX | dQ | dU | dZ (all earlier MMAs)
  __shared__ uint64_t bar_st[3], bar_drain;    // output tiles staged in shared memory: dB | dC | dU
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ float s_red[8 * NW + 2];
  float* sc_tab = reinterpret_cast<float*>(smem + B_OFF_SCAL);   // two tables of 11 rows (chunk parity)
  float* sw = sc_tab + 22 * 64;  // rows written by the workers: e^{l_end-l_t}, sigma, diag, c conj(b)
  float* s_acc = sw + 5 * 64;    // [4 quantities][8 = column group x half][64 rows]
  using PK = Pack2<TIn>;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool worker = warp < 4 * NW;
  const int quad = warp & 3, cg = worker ? (warp >> 2) : 0;
  const int row = 16 * quad + (lane & 15), hf = lane >> 4;
  const int rowA = 16 * quad + (lane >> 2), rowB = rowA + 8, cq = lane & 3;   // identity for the 16x256b loads
  constexpr int WC = 64 / NW, WB = WC / 8;   // columns / 8-column blocks per warp of a 64-wide accumulator
  static_assert(NW == 2 || NW == 4, "one to four 8-column blocks per warp");
  const int rcol = tid & 15, rrow0 = tid >> 4;
  const int d0 = cg * ZC;                    // first column (inside the half) of this thread
  const int bh = blockIdx.x;
  const int bg = (bh / p.heads) * p.groups + (bh % p.heads) / (p.heads / p.groups);   // row of B and C
  const int T = p.T, nC = p.nchunks;
  const float* Mb = p.M + (size_t)bh * T * 2;
  const float* Kb = p.K + (size_t)bh * T * 4;
  const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
  const long long wl = p.wait_limit;   // limit of the main loop's waits (the drain waits keep the default)

  if (tid == 0) {
    mbar_init(&bar_tma[0], 1); mbar_init(&bar_tma[1], 1);
    for (int i = 0; i < 5; ++i) mbar_init(&bar_mma[i], 1);
    for (int i = 0; i < 3; ++i) mbar_init(&bar_st[i], 4 * NW);   // one arrival per worker warp
    mbar_init(&bar_drain, 1);
    fence_barrier_init();
    s_abort = 0;
    tma_prefetch_desc(&p.tmU); tma_prefetch_desc(&p.tmB); tma_prefetch_desc(&p.tmC);
    tma_prefetch_desc(&p.tmdY); tma_prefetch_desc(&p.tmZ);
    tma_prefetch_desc(&p.tmdU); tma_prefetch_desc(&p.tmdB); tma_prefetch_desc(&p.tmdC);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, B_TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  // The stage of chunk c is requested at the top of the previous iteration, as soon as the output stores of
  // the chunk that used the stage before have read it (half an iteration ahead was not enough any more: the
  // workers were seen waiting 1000+ clk for the data).  That chunk's deferred epilogue 5 works on a register
  // copy of its Zv cells.
  auto issue_loads_inputs = [&](int c, int it) {   // one thread; also arms the barrier for the whole stage
    uint8_t* st = smem + (it & 1) * B_STAGE;
    uint64_t* bar = &bar_tma[it & 1];
    mbar_expect_tx(bar, B_STAGE);
    tma_load_3d(st, &p.tmU, bar, 0, c * L, bh);
    tma_load_3d(st + TILE, &p.tmB, bar, 0, c * L, bg);
    tma_load_3d(st + 2 * TILE, &p.tmB, bar, 64, c * L, bg);
    tma_load_3d(st + 3 * TILE, &p.tmC, bar, 0, c * L, bg);
    tma_load_3d(st + 4 * TILE, &p.tmC, bar, 64, c * L, bg);
    tma_load_3d(st + 5 * TILE, &p.tmdY, bar, 0, c * L, bh);
  };
  auto issue_loads_states = [&](int c, int it) {   // one thread
    uint8_t* st = smem + (it & 1) * B_STAGE;
    uint64_t* bar = &bar_tma[it & 1];
    tma_load_3d(st + 6 * TILE, &p.tmZ, bar, 0, c * 64, bh);
    tma_load_3d(st + 7 * TILE, &p.tmZ, bar, 64, c * 64, bh);
  };
  if (tid == 0) { issue_loads_inputs(nC - 1, 0); issue_loads_states(nC - 1, 0); }

  auto block_sum2 = [&](float a, float b, float& oa, float& ob) {
    a = warp_sum(a); b = warp_sum(b);   // workers only
    bar_sync(1, NT);
    if (lane == 0) { s_red[2 * warp] = a; s_red[2 * warp + 1] = b; }
    bar_sync(1, NT);
    oa = 0.f; ob = 0.f;
#pragma unroll
    for (int k = 0; k < 4 * NW; ++k) { oa += s_red[2 * k]; ob += s_red[2 * k + 1]; }
  };

  // adjoint state, conjugated pairs (da, db):  dz = da - i db
  float dz[ZC];
  {
    float ar = 0.f, ai = 0.f;
#pragma unroll
    for (int j = 0; j < ZC / 2; ++j) {
      float re = 0.f, im = 0.f;
      if (p.dfinal && worker) {
        const size_t o = ((size_t)bh * 64 + row) * 128 + 64 * hf + d0 + 2 * j;
        const float2 g = *reinterpret_cast<const float2*>(p.dfinal + o);
        const float2 z = *reinterpret_cast<const float2*>(p.zfinal + o);
        re = g.x; im = g.y;
        ar += re * z.x + im * z.y;   // d_final * conj(z_final)
        ai += im * z.x - re * z.y;
      }
      dz[2 * j] = re; dz[2 * j + 1] = -im;
    }
    if (worker) {
      float sr, si;
      block_sum2(ar, ai, sr, si);
      if (tid == 0) p.anchor[(size_t)bh * nC + nC - 1] = make_float2(sr, si);
    }
  }
  if (warp == 4 * NW) chunk_scalars(sc_tab, Mb, Kb, (nC - 1) * L, T, lane);
  __syncthreads();

  constexpr uint32_t ID_KK32 = make_idesc(64, 32, PK::fmt, 0, 0);
  constexpr uint32_t ID_KK64 = make_idesc(64, 64, PK::fmt, 0, 0);
  constexpr uint32_t ID_KM64 = make_idesc(64, 64, PK::fmt, 0, 1);
  constexpr uint32_t ID_MM64 = make_idesc(64, 64, PK::fmt, 1, 1);
  constexpr uint32_t ID_MM32 = make_idesc(64, 32, PK::fmt, 1, 1);
  constexpr uint32_t ID_KM128 = make_idesc(64, 128, PK::fmt, 0, 1);
  constexpr uint32_t ID_MM128 = make_idesc(64, 128, PK::fmt, 1, 1);
  const uint32_t aQ = smem_u32(smem + B_OFF_Q), aKP = smem_u32(smem + B_OFF_KP),
                 aDYO = smem_u32(smem + B_OFF_DYO), aPD = smem_u32(smem + B_OFF_PD),
                 aDP = smem_u32(smem + B_OFF_DP), aDW = smem_u32(smem + B_OFF_DW),
                 aUE = smem_u32(smem + B_OFF_UE);
  bool ok = true;
  int issued_it = 0;   // issue lane: the last iteration whose loads were requested (iteration 0 by thread 0 above)

  // ---- epilogue 5 of the chunk of iteration itp (run one iteration late): dz <- e^{l_end} dWv + dZ,
  // and the anchor S = <dz, z> of the boundary below that chunk ------------------------------------------
  float em_keep = 0.f;   // e^{l_end} of the chunk whose epilogue 5 is pending
  uint4 zv_keep[ZC / 8];  // and this thread's cells of its Zv tiles
#pragma unroll
  for (int ch = 0; ch < ZC / 8; ++ch) zv_keep[ch] = make_uint4(0u, 0u, 0u, 0u);
  auto epilogue5 = [&](int itp, bool live) {
    const int cp = nC - 1 - itp;
    // (this thread's cells of that chunk's Zv tiles were copied to zv_keep at the end of its iteration, so
    // that the whole stage can be refilled at the top of the next one)
    if (live && !mbar_wait(&bar_mma[4], itp & 1, wl)) { report_timeout(16); s_abort = 1; live = false; }
    tc_fence_after_sync();
    const float em = em_keep;
    float ar = 0.f, ai = 0.f;
    if (live) {
#pragma unroll
      for (int part = 0; part < ZC / PC; ++part) {
        uint32_t zi[PC];
        tmem_ld_16x32bx2<PC, 64>(tmem + lane_base + 384 + d0 + PC * part, zi);
        tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < PC / 8; ++ch) {
          const uint4 zv4 = zv_keep[(PC / 8) * part + ch];
          const uint32_t zw[4] = {zv4.x, zv4.y, zv4.z, zv4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = 8 * ch + 2 * e, jj = PC * part + j;
            const float da = em * dz[jj] + __uint_as_float(zi[j]);
            const float db = em * dz[jj + 1] + __uint_as_float(zi[j + 1]);
            dz[jj] = da; dz[jj + 1] = db;
            const float2 z = PK::unpack(zw[e]);   // (a, b): z = a - i b ; dz = da - i db
            ar += da * z.x + db * z.y;            // dz conj(z)
            ai += da * z.y - db * z.x;
          }
        }
      }
    }
    // per-warp partial sums of the anchor; they are added up by finish_anchor() on the scalar warp after
    // named barrier 7 (no CTA-wide reduction here)
    ar = warp_sum(ar); ai = warp_sum(ai);
    if (lane == 0) { s_red[2 * warp] = live ? ar : 0.f; s_red[2 * warp + 1] = live ? ai : 0.f; }
  };
  auto finish_anchor = [&](int itp) {   // one thread of the scalar warp, after the barrier that follows epilogue5(itp)
    const int cp = nC - 1 - itp;
    if (cp <= 0) return;
    float sr = 0.f, si = 0.f;
#pragma unroll
    for (int k = 0; k < 4 * NW; ++k) { sr += s_red[2 * k]; si += s_red[2 * k + 1]; }
    p.anchor[(size_t)bh * nC + cp - 1] = make_float2(sr, si);
  };
  // ---- dWv tile of a chunk: dz rotated by the unit phase of Pi_end: (a,b) -> (ur a - ui b, ui a + ur b),
  // and the row e^{l_end - l_t} of that chunk ------------------------------------------------------------------
  auto make_dwv = [&](const float* sc) {
    const float ur = sc[10 * 64 + 2], ui = sc[10 * 64 + 3];
    if (tid < 64) sw[0 * 64 + tid] = __expf(fminf(sc[63] - sc[tid], 0.f));
    uint8_t* dw = smem + B_OFF_DW + hf * TILE;
#pragma unroll
    for (int ch = 0; ch < ZC / 8; ++ch) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = dz[8 * ch + 2 * e], bq = dz[8 * ch + 2 * e + 1];
        const float na = ur * a - ui * bq, nb = ui * a + ur * bq;
        dz[8 * ch + 2 * e] = na; dz[8 * ch + 2 * e + 1] = nb;
        w[e] = PK::pack(na, nb);
      }
      *reinterpret_cast<uint4*>(dw + sw128(row, d0 / 8 + ch)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  };

  for (int it = 0; it < nC && ok; ++it) {
    const int c = nC - 1 - it, t0 = c * L;
    uint8_t* st = smem + (it & 1) * B_STAGE;
    uint8_t *tU = st, *tB = st + TILE, *tC = st + 3 * TILE, *tDY = st + 5 * TILE, *tZ = st + 6 * TILE;
    float* sc = sc_tab + (it & 1) * (11 * 64);
    if (warp == 4 * NW) {
      // scalars of the next (earlier) chunk; this warp meets the others only at the barrier that
      // ends the iteration
      // (it starts after the workers' first passes: global loads issued while every worker warp
      // bursts shared-memory traffic at the top of the iteration stalled the whole SM for about a
      // DRAM round trip)
      bar_sync(2, NT + 64);   // the workers only arrive here (bar_arrive): they never wait for this warp
      if (it + 1 < nC) chunk_scalars(sc_tab + ((it + 1) & 1) * (11 * 64), Mb, Kb, t0 - L, T, lane);
      // the anchor of the previous chunk: a global store by a worker thread here would make that
      // thread's next proxy fence (epilogue 1) wait for the store, and every worker for that thread
      bar_sync(7, NT + 32);
      if (lane == 0 && it > 0 && s_abort == 0) finish_anchor(it - 1);
      __syncwarp();
    } else if (!worker) {
      // Issue warp (one lane): every MMA of this chunk, the TMA loads of the next (earlier) chunk and
      // the TMA stores of this chunk's outputs.  The workers never wait for this warp, only for the
      // commit barriers of the products they read: they arrive on named barriers 2 ("passes done")
      // and 4 ("epilogue 1 done") without waiting and move on.
      // K-major (kX) and MN-major (mX) base descriptors of every operand tile of this chunk
      const uint64_t kQ = make_desc(aQ, 16, 1024), mQ = make_desc(aQ, 8192, 1024);
      const uint64_t kKP = make_desc(aKP, 16, 1024), mKP = make_desc(aKP, 8192, 1024);
      const uint64_t kU = make_desc(smem_u32(tU), 16, 1024);
      const uint64_t kDY = make_desc(smem_u32(tDY), 16, 1024), mDY = make_desc(smem_u32(tDY), 8192, 1024);
      const uint64_t mZ = make_desc(smem_u32(tZ), 8192, 1024);
      const uint64_t kDP = make_desc(aDP, 16, 1024), mDP = make_desc(aDP, 8192, 1024);
      const uint64_t mPD = make_desc(aPD, 8192, 1024), mDYO = make_desc(aDYO, 8192, 1024), kDYO = make_desc(aDYO, 16, 1024);
      const uint64_t kDW = make_desc(aDW, 16, 1024), mDW = make_desc(aDW, 8192, 1024);
      const uint64_t kUE = make_desc(aUE, 16, 1024);
      bool go = lane == 0 && s_abort == 0;
      if (go) do {
        // (1) products of raw tiles, as soon as the stage has landed
        if (!mbar_wait(&bar_tma[it & 1], (it >> 1) & 1, wl)) { report_timeout(20); s_abort = 1; go = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dS[t][s] = sum_p dY[t][p] U[s][p]            A: dY K-major, B: U K-major rows s
          umma(tmem + 64, desc_adv(kDY, 32 * k), desc_adv(kU, 32 * k), ID_KK64, k > 0);
        if (it + 1 < nC) {   // next chunk's input tiles
          tma_store_wait_read();   // the stores of the previous chunk read the stage being refilled
          issue_loads_inputs(c - 1, it + 1);
          issue_loads_states(c - 1, it + 1);
          issued_it = it + 1;
        }
      } while (false);
      __syncwarp();
      // (1b) the first four k-steps of P~, once the first column halves of Q and K' are rotated
      bar_sync(5, NT + 32);
      if (go && s_abort == 0) {
        tc_fence_after_sync();
        // P~[t][s] = sum_d Q[t][d] K'[s][d]              A: Q K-major, B: K' K-major rows s
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma(tmem + 0, desc_adv(kQ, k * 32), desc_adv(kKP, k * 32), ID_KK64, k > 0);
      }
      __syncwarp();
      // (2) products of rotated tiles, once the workers' passes are done (Q, K', dYoff written)
      bar_sync(2, NT + 64);
      if (go && s_abort == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 4; k < 8; ++k) {
          const uint32_t ko = TILE + (k & 3) * 32;
          umma(tmem + 0, desc_adv(kQ, ko), desc_adv(kKP, ko), ID_KK64, 1);
        }
        umma_commit(&bar_mma[0]);   // P~ and dS: epilogue 1 may start
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dQ[t][d] = sum_p dYoff[t][p] Zv[p][d] (+ dP K' below)   A: dYoff K-major, B: Zv MN-major (rows = p)
          umma(tmem + 128, desc_adv(kDYO, 32 * k), desc_adv(mZ, 2048 * k), ID_KM128, k > 0);
      }
      __syncwarp();
      // (2b) once the workers have finished epilogue 5 of the previous chunk (the Zv tiles of the other
      // stage are free) and written this chunk's dWv
      bar_sync(6, NT + 32);
      if (go && s_abort == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dX[s][d] = sum_p (e^{l_end-l_s} U[s][p]) dWv[p][d] (+ dP^T Q below)   A: Uee K-major, B: dWv MN-major
          umma(tmem + 256, desc_adv(kUE, 32 * k), desc_adv(mDW, 2048 * k), ID_KM128, k > 0);
      }
      __syncwarp();
      // (3) products of the masked tiles, once epilogue 1 has written Pdec and dP; ordered by the
      // epilogue that consumes them (dX, dQ, dU, dZ)
      bar_sync(4, NT + 32);
      if (go && s_abort == 0) do {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dX[s][d] += sum_t dP[t][s] Q[t][d]         A: dP MN-major (rows = t), B: Q MN-major
          umma(tmem + 256, desc_adv(mDP, 2048 * k), desc_adv(mQ, 2048 * k), ID_MM128, 1);
        umma_commit(&bar_mma[1]);   // dX
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dQa[t][d] = sum_s dP[t][s] K'[s][d]        A: dP K-major, B: K' MN-major (rows = s)
          umma(tmem + 128, desc_adv(kDP, 32 * k), desc_adv(mKP, 2048 * k), ID_KM128, 1);
        umma_commit(&bar_mma[2]);   // dQ
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dUa[s][p] = sum_t Pdec[t][s] dY[t][p]        A: Pdec MN-major, B: dY MN-major
          umma(tmem + 0, desc_adv(mPD, 2048 * k), desc_adv(mDY, 2048 * k), ID_MM64, k > 0);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // dUb[s][p] = sum_d K'[s][d] dWv[p][d]         A: K' K-major, B: dWv K-major rows p
          const uint32_t ko = (k >> 2) * TILE + (k & 3) * 32;
          umma(tmem + 64, desc_adv(kKP, ko), desc_adv(kDW, ko), ID_KK64, k > 0);
        }
        umma_commit(&bar_mma[3]);   // dU
#pragma unroll
        for (int k = 0; k < 4; ++k)
          // dZ[p][d]  = sum_t dYoff[t][p] Q[t][d]      A: dYoff MN-major, B: Q MN-major
          umma(tmem + 384, desc_adv(mDYO, 2048 * k), desc_adv(mQ, 2048 * k), ID_MM128, k > 0);
        umma_commit(&bar_mma[4]);   // dZ
        // (4) output tiles: the workers overwrite dead operand tiles of this stage in place (C with dB,
        // B with dC, dY with dU) and signal; one TMA store per tile writes full 128-byte rows.
        if (!mbar_wait(&bar_st[0], it & 1, wl)) { report_timeout(17); s_abort = 1; break; }
        tma_store_3d(&p.tmdB, tC, 0, t0, bh); tma_store_3d(&p.tmdB, tC + TILE, 64, t0, bh);
        tma_store_commit();
        if (!mbar_wait(&bar_st[1], it & 1, wl)) { report_timeout(18); s_abort = 1; break; }
        tma_store_3d(&p.tmdC, tB, 0, t0, bh); tma_store_3d(&p.tmdC, tB + TILE, 64, t0, bh);
        tma_store_commit();
        if (!mbar_wait(&bar_st[2], it & 1, wl)) { report_timeout(19); s_abort = 1; break; }
        tma_store_3d(&p.tmdU, tDY, 0, t0, bh);
        tma_store_commit();
        // The next iteration's passes overwrite the dYoff and Q tiles that the dZ products (issued after
        // everything the workers wait for in this iteration) read: this lane sees them complete before it
        // joins the barrier that ends the iteration.
        if (!mbar_wait(&bar_mma[4], it & 1, wl)) { report_timeout(21); s_abort = 1; break; }
      } while (false);
      __syncwarp();
    } else {
    bool live = true;   // cleared when a bounded wait expired: the rest of the chunk is skipped
    if (!mbar_wait(&bar_tma[it & 1], (it >> 1) & 1, wl)) { report_timeout(11); s_abort = 1; live = false; }

    // ---- pass 1 over dY, U: sigma_t = <dy_t, u_t>, dYoff = e^{l_t} dY -------------------------------
    if (live) {
#pragma unroll
    for (int k = 0; k < 512 / NT; ++k) {
      const int item = tid + NT * k, r = item >> 3, ch = item & 7;
      const uint32_t off = sw128(r, ch);
      const uint4 dv = *reinterpret_cast<const uint4*>(tDY + off);
      const uint4 uv = *reinterpret_cast<const uint4*>(tU + off);
      const uint32_t dw_[4] = {dv.x, dv.y, dv.z, dv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
      const float et = sc[1 * 64 + r];
      const float ee = __expf(fminf(sc[63] - sc[r], 0.f));   // e^{l_end - l_s}
      uint32_t o[4], ue[4];
      float sg = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d2 = PK::unpack(dw_[e]), u2 = PK::unpack(uw[e]);
        sg += d2.x * u2.x + d2.y * u2.y;
        o[e] = PK::pack(et * d2.x, et * d2.y);
        ue[e] = PK::pack(ee * u2.x, ee * u2.y);
      }
      *reinterpret_cast<uint4*>(smem + B_OFF_DYO + off) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(smem + B_OFF_UE + off) = make_uint4(ue[0], ue[1], ue[2], ue[3]);
      sg += __shfl_xor_sync(0xffffffffu, sg, 4);
      sg += __shfl_xor_sync(0xffffffffu, sg, 2);
      sg += __shfl_xor_sync(0xffffffffu, sg, 1);
      if (ch == 0) sw[1 * 64 + r] = sg;
    }
    }
    // ---- pass 2 over B, C: Q, K', diagonal pieces ------------------------------------------------------
    // Two phases, one per 64-column half of the state dimension: P~ accumulates over that dimension, so
    // the issue warp starts its first four k-steps (named barrier 5) while the workers rotate the second
    // half.  A thread keeps its rows in both phases (8 threads per row), so the row sums stay in registers.
    {
      constexpr int IPT = 512 / NT;   // (row, piece) items per thread and phase
      float cbrk[IPT], cbik[IPT];
#pragma unroll
      for (int j = 0; j < IPT; ++j) { cbrk[j] = 0.f; cbik[j] = 0.f; }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (live) {
#pragma unroll
          for (int j = 0; j < IPT; ++j) {
            const int item = tid + NT * j, r = item >> 3;
            const uint32_t off = half * TILE + sw128(r, item & 7);
            const float phr = sc[2 * 64 + r], phi = sc[3 * 64 + r];
            const float wr = sc[4 * 64 + r], wi = sc[5 * 64 + r];
            const uint4 cv = *reinterpret_cast<const uint4*>(tC + off);
            const uint4 bv = *reinterpret_cast<const uint4*>(tB + off);
            const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
            uint32_t qo[4], ko[4];
            float cbr = 0.f, cbi = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 cc = PK::unpack(cw[e]), bb = PK::unpack(bw[e]);
              qo[e] = PK::pack(cc.x * phr + cc.y * phi, cc.x * phi - cc.y * phr);     // conj(c) phi
              ko[e] = PK::pack(wr * bb.x - wi * bb.y, -(wr * bb.y + wi * bb.x));      // conj(w b)
              cbr += cc.x * bb.x + cc.y * bb.y;                                       // c conj(b)
              cbi += cc.y * bb.x - cc.x * bb.y;
            }
            cbrk[j] += cbr; cbik[j] += cbi;
            *reinterpret_cast<uint4*>(smem + B_OFF_Q + off) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
            *reinterpret_cast<uint4*>(smem + B_OFF_KP + off) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
          }
        }
        if (half == 0) {   // first halves of Q and K' are complete: P~ may start
          fence_async_smem();
          tc_fence_before_sync();
          bar_arrive(5, NT + 32);
        }
      }
      if (live) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
#pragma unroll
          for (int j = 0; j < IPT; ++j) {
            cbrk[j] += __shfl_xor_sync(0xffffffffu, cbrk[j], o);
            cbik[j] += __shfl_xor_sync(0xffffffffu, cbik[j], o);
          }
        }
        if ((tid & 7) == 0) {
#pragma unroll
          for (int j = 0; j < IPT; ++j) {
            const int r = (tid + NT * j) >> 3;
            // diagonal term Re sum conj(c) kc b = Re(kc conj(sum c conj(b)))
            sw[2 * 64 + r] = sc[8 * 64 + r] * cbrk[j] + sc[9 * 64 + r] * cbik[j];
            sw[3 * 64 + r] = cbrk[j]; sw[4 * 64 + r] = cbik[j];
          }
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    // no barrier among the workers here or at the end of the gap below: what a warp does next (epilogue 5
    // of the previous chunk, dWv, the decay factors) touches nothing the passes of another warp read or
    // write; the workers meet at the end of epilogue 1
    bar_arrive(2, NT + 64);      // the scalar and issue warps are told without being waited for
    live = s_abort == 0;
    // ---- in the shadow of the P~ MMAs: epilogue 5 of the previous iteration, then this chunk's dWv ------
    if (it > 0) epilogue5(it - 1, live);
    live = live && s_abort == 0;
    if (live) make_dwv(sc);
    em_keep = sc[1 * 64 + 63];
    fence_async_smem();
    tc_fence_before_sync();
    bar_arrive(6, NT + 32);      // dWv written, the previous dZ accumulator and Zv tiles released
    bar_arrive(7, NT + 32);      // anchor partial sums written: the scalar warp adds them up and stores

    // ---- MMA group 1 (issued by the look-ahead warp): P~ = Q K'^T, dS = dY U^T ------------------------
    // The waits and TMEM loads below are compiler barriers, so everything an epilogue reads from shared
    // memory is fetched by hand BEFORE the wait it would otherwise queue behind.
    float dec[4 * WB];   // causal decay factors of this thread's (row, column) cells, [hh][i][0..1]
    {
      // loads and exponentials are unconditional (a load under a condition is not speculated by the
      // compiler: eight serial branches, each with its own load-to-exp latency); the mask is a select
      float ls[2 * WB];
#pragma unroll
      for (int i = 0; i < WB; ++i) {
        const float2 l2 = *reinterpret_cast<const float2*>(sc + cg * WC + 8 * i + 2 * cq);
        ls[2 * i] = l2.x; ls[2 * i + 1] = l2.y;
      }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int R = hh ? rowB : rowA;
        const float lt = sc[R];
#pragma unroll
        for (int i = 0; i < WB; ++i) {
          const int s0 = cg * WC + 8 * i + 2 * cq;
          const float e0 = __expf(fminf(lt - ls[2 * i], 0.f)), e1 = __expf(fminf(lt - ls[2 * i + 1], 0.f));
          dec[(hh * WB + i) * 2 + 0] = s0 < R ? e0 : 0.f;
          dec[(hh * WB + i) * 2 + 1] = s0 + 1 < R ? e1 : 0.f;
        }
      }
    }
    if (live && !mbar_wait(&bar_mma[0], it & 1, wl)) { report_timeout(12); s_abort = 1; live = false; }
    tc_fence_after_sync();

    // ---- epilogue 1: decayed, strictly causal Pdec and dP as 16-bit tiles -------------------------------
    if (live) {
      uint32_t pr[4 * WB], ds[4 * WB];
      tmem_ld_16x256<WB>(tmem + lane_base + 0 + cg * WC, pr);
      tmem_ld_16x256<WB>(tmem + lane_base + 64 + cg * WC, ds);
      tmem_ld_wait();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int R = hh ? rowB : rowA;
#pragma unroll
        for (int i = 0; i < WB; ++i) {
          const float dec0 = dec[(hh * WB + i) * 2 + 0], dec1 = dec[(hh * WB + i) * 2 + 1];
          const uint32_t off = sw128(R, cg * WB + i) + 4 * cq;
          *reinterpret_cast<uint32_t*>(smem + B_OFF_PD + off) =
              PK::pack(dec0 * __uint_as_float(pr[4 * i + 2 * hh]), dec1 * __uint_as_float(pr[4 * i + 2 * hh + 1]));
          *reinterpret_cast<uint32_t*>(smem + B_OFF_DP + off) =
              PK::pack(dec0 * __uint_as_float(ds[4 * i + 2 * hh]), dec1 * __uint_as_float(ds[4 * i + 2 * hh + 1]));
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    bar_sync(3, NT);
    bar_arrive(4, NT + 32);
    live = s_abort == 0;

    // ---- MMA group 2 (issued by the look-ahead warp, one commit per accumulator set) ------------------
    // operands of epilogues 3 and 2 (this thread's cells of the C, B and Q tiles and its row's scalars),
    // fetched while the products are still running
    uint4 cvv[ZC / 8], bvv[ZC / 8], qvv[ZC / 8];
#pragma unroll
    for (int ch = 0; ch < ZC / 8; ++ch) {
      const uint32_t off = hf * TILE + sw128(row, d0 / 8 + ch);
      cvv[ch] = *reinterpret_cast<const uint4*>(tC + off);
      bvv[ch] = *reinterpret_cast<const uint4*>(tB + off);
      qvv[ch] = *reinterpret_cast<const uint4*>(smem + B_OFF_Q + off);
    }
    const float sig = sw[1 * 64 + row];
    const float wr = sc[4 * 64 + row], wi = sc[5 * 64 + row];
    const float phr = sc[2 * 64 + row], phi = sc[3 * 64 + row];
    const float skr = sig * sc[8 * 64 + row], ski = sig * sc[9 * 64 + row];   // sigma kc
    if (live && !mbar_wait(&bar_mma[1], it & 1, wl)) { report_timeout(13); s_abort = 1; live = false; }
    tc_fence_after_sync();

    // ---- epilogue 3 (first): dX -> dB, R = sum conj(b) dX ---------------------------------------------------------
    if (live) {
      float rr = 0.f, ri = 0.f;
      uint32_t xall[ZC];
      tmem_ld_16x32bx2<ZC, 64>(tmem + lane_base + 256 + d0, xall);
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < ZC / 8; ++ch) {
        const uint32_t* xa = xall + 8 * ch;
        const uint32_t off = hf * TILE + sw128(row, d0 / 8 + ch);
        const uint4 cv = cvv[ch], bv = bvv[ch];
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 2 * e;
          const float ga = __uint_as_float(xa[j]), gb = __uint_as_float(xa[j + 1]);
          const float2 cc = PK::unpack(cw[e]), bb = PK::unpack(bw[e]);
          // dX = ga - i gb ; R += conj(b) dX
          rr += bb.x * ga - bb.y * gb;
          ri += -bb.x * gb - bb.y * ga;
          // db = conj(w) dX + sigma conj(kc) c
          const float dbr = wr * ga - wi * gb + (skr * cc.x + ski * cc.y);
          const float dbi = -wr * gb - wi * ga + (skr * cc.y - ski * cc.x);
          o[e] = PK::pack(dbr, dbi);
        }
        *reinterpret_cast<uint4*>(tC + off) = make_uint4(o[0], o[1], o[2], o[3]);   // dB over C, in place
      }
      s_acc[(2 * 8 + 2 * cg + hf) * 64 + row] = rr;
      s_acc[(3 * 8 + 2 * cg + hf) * 64 + row] = ri;
    }
    // the tile is complete once every worker warp has arrived; the issue warp then stores it
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_st[0]);
    if (live && !mbar_wait(&bar_mma[2], it & 1, wl)) { report_timeout(14); s_abort = 1; live = false; }
    tc_fence_after_sync();
    // ---- epilogue 2: dQ -> dC, <q,dq> ------------------------------------------------------------------
    if (live) {
      float ar = 0.f, ai = 0.f;
      uint32_t qall[ZC];
      tmem_ld_16x32bx2<ZC, 64>(tmem + lane_base + 128 + d0, qall);
      tmem_ld_wait();
#pragma unroll
      for (int ch = 0; ch < ZC / 8; ++ch) {
        const uint32_t* qa = qall + 8 * ch;
        const uint32_t off = hf * TILE + sw128(row, d0 / 8 + ch);
        const uint4 qv = qvv[ch], bv = bvv[ch];
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 2 * e;
          const float dqr = __uint_as_float(qa[j]), dqi = __uint_as_float(qa[j + 1]);
          const float2 q = PK::unpack(qw[e]), bb = PK::unpack(bw[e]);
          ar += q.x * dqr + q.y * dqi;          // conj(q) dq
          ai += q.x * dqi - q.y * dqr;
          // dc = conj(dq) phi + sigma kc b
          const float dcr = dqr * phr + dqi * phi + (skr * bb.x - ski * bb.y);
          const float dci = dqr * phi - dqi * phr + (skr * bb.y + ski * bb.x);
          o[e] = PK::pack(dcr, dci);
        }
        *reinterpret_cast<uint4*>(tB + off) = make_uint4(o[0], o[1], o[2], o[3]);   // dC over B, in place
      }
      s_acc[(0 * 8 + 2 * cg + hf) * 64 + row] = ar;
      s_acc[(1 * 8 + 2 * cg + hf) * 64 + row] = ai;
    }
    // the tile is complete once every worker warp has arrived; the issue warp then stores it
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_st[1]);
    // operands of epilogue 4: this thread's cells of the dY tile and its rows' scalars
    uint32_t dyc[2 * WB];
    float e4s[4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int R = hh ? rowB : rowA;
      e4s[2 * hh] = sw[0 * 64 + R]; e4s[2 * hh + 1] = sw[2 * 64 + R];
#pragma unroll
      for (int i = 0; i < WB; ++i)
        dyc[hh * WB + i] = *reinterpret_cast<const uint32_t*>(tDY + sw128(R, cg * WB + i) + 4 * cq);
    }
    if (live && !mbar_wait(&bar_mma[3], it & 1, wl)) { report_timeout(15); s_abort = 1; live = false; }
    tc_fence_after_sync();
    // ---- epilogue 4: dU ---------------------------------------------------------------------------------------
    if (live) {
      uint32_t ua[4 * WB], ub[4 * WB];
      tmem_ld_16x256<WB>(tmem + lane_base + 0 + cg * WC, ua);
      tmem_ld_16x256<WB>(tmem + lane_base + 64 + cg * WC, ub);
      tmem_ld_wait();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int R = hh ? rowB : rowA;
        const float ee = e4s[2 * hh], dgv = e4s[2 * hh + 1];
#pragma unroll
        for (int i = 0; i < WB; ++i) {
          uint32_t* cell = reinterpret_cast<uint32_t*>(tDY + sw128(R, cg * WB + i) + 4 * cq);
          const float2 d2 = PK::unpack(dyc[hh * WB + i]);
          *cell = PK::pack(__uint_as_float(ua[4 * i + 2 * hh]) + ee * __uint_as_float(ub[4 * i + 2 * hh]) + dgv * d2.x,
                           __uint_as_float(ua[4 * i + 2 * hh + 1]) + ee * __uint_as_float(ub[4 * i + 2 * hh + 1]) + dgv * d2.y);   // dU over dY, in place
        }
      }
    }
    // the tile is complete once every worker warp has arrived; the issue warp then stores it
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_st[2]);
    // (epilogue 5 of this chunk - the update of dz - runs in the next iteration, in the shadow of the
    // P~ MMAs; its inputs, the dZ accumulator and the Zv tiles of this stage, stay untouched until then)
#pragma unroll
    for (int ch = 0; ch < ZC / 8; ++ch)   // for the deferred epilogue 5 of this chunk
      zv_keep[ch] = *reinterpret_cast<const uint4*>(tZ + hf * TILE + sw128(row, d0 / 8 + ch));
    bar_sync(1, NT);   // the partial sums written by epilogues 2 and 3 are read by other threads below
    // the proxy fence for this iteration's shared-memory accesses goes BEFORE the global stores
    // below (the code after them touches no tile)
    fence_async_smem();
    // ---- per-token scalars of this chunk ---------------------------------------------------------------------
    if (live && tid < 64 && t0 + tid < T) {
      const int t = tid;
      float Ar = 0.f, Ai = 0.f, Rr = 0.f, Ri = 0.f;
#pragma unroll
      for (int k = 0; k < 2 * NW; ++k) {
        Ar += s_acc[(0 * 8 + k) * 64 + t]; Ai += s_acc[(1 * 8 + k) * 64 + t];
        Rr += s_acc[(2 * 8 + k) * 64 + t]; Ri += s_acc[(3 * 8 + k) * 64 + t];
      }
      const float phr = sc[2 * 64 + t], phi = sc[3 * 64 + t], wr = sc[4 * 64 + t], wi = sc[5 * 64 + t];
      const size_t o = (size_t)bh * T + t0 + t;
      p.dg[o] = make_float2(phr * Rr - phi * Ri, phr * Ri + phi * Rr);                 // phi R
      p.sterm[o] = make_float2(Ar - (wr * Rr + wi * Ri), Ai - (wr * Ri - wi * Rr));   // A - conj(w) R
      const float sg = sw[1 * 64 + t];
      p.dkcd[o] = make_float2(sg * sw[3 * 64 + t], sg * sw[4 * 64 + t]);
    }
    tc_fence_before_sync();
    }  // worker
    __syncthreads();
    if (s_abort) { ok = false; break; }
  }

  if (ok && worker) epilogue5(nC - 1, true);
  ok = ok && s_abort == 0;
  if (ok && p.dinit && worker) {
    float* dst = p.dinit + ((size_t)bh * 64 + row) * 128 + 64 * hf + d0;
#pragma unroll
    for (int j = 0; j < ZC / 4; ++j)
      *reinterpret_cast<float4*>(dst + 4 * j) =
          make_float4(dz[4 * j], -dz[4 * j + 1], dz[4 * j + 2], -dz[4 * j + 3]);
  }
  // Unwind: nothing of this CTA may still be in flight when shared memory and TMEM are released.  The
  // issue lane started every asynchronous operation (but for the loads of the first iteration), so it
  // drains them: after an expired wait the loads of the last two requested iterations (their barriers,
  // default long limit) and, always, every tcgen05.mma issued so far (one more commit) and its TMA stores.
  if (warp == 4 * NW + 1 && lane == 0) {
    if (s_abort)
      for (int ii = issued_it > 0 ? issued_it - 1 : 0; ii <= issued_it; ++ii) mbar_wait(&bar_tma[ii & 1], (ii >> 1) & 1);
    umma_commit(&bar_drain);
    mbar_wait(&bar_drain, 0);
    tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, B_TMEM_COLS);
}

// dM and dK from the per-token scalars.  One warp per chunk (two tokens per lane); chunks are
// independent given the anchors, so the grid is (batch*heads, chunks / 4).
__global__ void __launch_bounds__(128) scan_tc_bwd_finish_kernel(const float* __restrict__ M,
                                                                 const float* __restrict__ K,
                                                                 const float2* __restrict__ dg,
                                                                 const float2* __restrict__ sterm,
                                                                 const float2* __restrict__ dkcd,
                                                                 const float2* __restrict__ anchor,
                                                                 const float2* __restrict__ dg_boundary,
                                                                 float* __restrict__ dM,
                                                                 float* __restrict__ dK, int T, int nC) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t bh = blockIdx.x;
  // grid.y covers the chunks four at a time: every warp of the grid owns exactly one chunk
  for (int c = blockIdx.y * 4 + warp; c < nC; c += 4 * gridDim.y) {
    const int tA = c * 64 + 2 * lane, tB = tA + 1;
    float2 sA = make_float2(0.f, 0.f), sB = sA;
    if (tA < T) sA = sterm[bh * T + tA];
    if (tB < T) sB = sterm[bh * T + tB];
    // inclusive suffix sums over the chunk
    float xr = sA.x + sB.x, xi = sA.y + sB.y;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float yr = __shfl_down_sync(0xffffffffu, xr, o), yi = __shfl_down_sync(0xffffffffu, xi, o);
      if (lane + o < 32) { xr += yr; xi += yi; }
    }
    const float2 an = anchor[bh * nC + c];
    const float SAr = an.x + xr, SAi = an.y + xi;            // S at token tA
    const float SBr = SAr - sA.x, SBi = SAi - sA.y;          // S at token tB
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int t = q ? tB : tA;
      if (t >= T) continue;
      const float Sr = q ? SBr : SAr, Si = q ? SBi : SAi;
      const float mr = M[(bh * T + t) * 2], mi = M[(bh * T + t) * 2 + 1];
      const float den = mr * mr + mi * mi;
      const float4 k4 = *reinterpret_cast<const float4*>(K + (bh * T + t) * 4);
      float2 gp = make_float2(0.f, 0.f);
      // the prev-tap of token t belongs to the merged coefficient of token t-1; for t = 0 that is the
      // pending tap of the token before the sequence (carried B_prev / U_prev), if there is one
      if (t > 0) gp = dg[bh * T + t - 1];
      else if (dg_boundary) gp = dg_boundary[bh];
      const float2 gc = dg[bh * T + t], kd = dkcd[bh * T + t];
      // x / conj(m) = x m / |m|^2
      const float dmr = (Sr * mr - Si * mi) / den, dmi = (Sr * mi + Si * mr) / den;
      const float dkpr = (gp.x * mr - gp.y * mi) / den, dkpi = (gp.x * mi + gp.y * mr) / den;
      // q = kp / m ; dm -= conj(q) dkp
      const float qr = (k4.x * mr + k4.y * mi) / den, qi = (k4.y * mr - k4.x * mi) / den;
      float2* dMo = reinterpret_cast<float2*>(dM) + bh * T + t;
      *dMo = make_float2(dmr - (qr * dkpr + qi * dkpi), dmi - (qr * dkpi - qi * dkpr));
      *reinterpret_cast<float4*>(dK + (bh * T + t) * 4) = make_float4(dkpr, dkpi, gc.x + kd.x, gc.y + kd.y);
    }
  }
}

// Grouped B / C: the sweep leaves dB and dC per head (16-bit); here the heads of a group are added up in
// float32 and cast once (the reference reduces in float32 as well:
// slinoss/ops/v2x2ssd/cute/kernels/bwd/__init__.py:548-563).  One thread per 16-byte piece of an output row.
template <typename TIn>
__global__ void __launch_bounds__(256) scan_tc_group_reduce_kernel(const TIn* __restrict__ per_head_b,
                                                                   const TIn* __restrict__ per_head_c,
                                                                   TIn* __restrict__ dB, TIn* __restrict__ dC,
                                                                   int heads, int groups, int T, size_t pieces,
                                                                   int out_pitch) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // piece index over (batch*groups, T, 16)
  if (i >= pieces) return;
  const int hpg = heads / groups;
  const size_t row = i >> 4, piece = i & 15;
  const size_t bgi = row / T, t = row % T;
  const size_t b = bgi / groups, g = bgi % groups;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const TIn* src = which ? per_head_c : per_head_b;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int hh = 0; hh < hpg; ++hh) {
      const size_t bh = b * heads + g * hpg + hh;
      float v[8];
      load16<TIn>(src + (bh * T + t) * 128 + piece * 8, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
    store16<TIn>((which ? dC : dB) + (bgi * T + t) * out_pitch + piece * 8, acc);
  }
}

// Carried taps: the sequence starts from  W_{-1} = z_{-1} + u_prev (x) (X b_prev),  X = kp_0 / m_0.  Given
// D = the adjoint of W_{-1} (what the sweep leaves as d_initial), per (batch, head):
//     v[n]      = sum_p u_prev[p] D[p,n]
//     dB_prev  += conj(X) v            (summed over the heads of a group, float32, cast once)
//     dU_prev[p] = Re sum_n conj(X b_prev[n]) D[p,n]
//     dX        = sum_n conj(b_prev[n]) v[n]     -> scan_tc_bwd_finish_kernel turns it into dkp_0 and its part of dm_0
// (reference: slinoss/ops/v2x2ssd/cute/autograd.py:269-276 returns these as dB_prev / dU_prev).
// One CTA of 128 threads per (batch, group); thread j owns the interleaved lane j of B_prev.
template <typename TIn>
__global__ void __launch_bounds__(128) scan_tc_bwd_boundary_kernel(const float* __restrict__ D,
                                                                   const TIn* __restrict__ Bprev,
                                                                   const TIn* __restrict__ Uprev,
                                                                   const float* __restrict__ M,
                                                                   const float* __restrict__ K,
                                                                   TIn* __restrict__ dBprev, TIn* __restrict__ dUprev,
                                                                   float2* __restrict__ dg_boundary, int heads,
                                                                   int groups, int T) {
  __shared__ float s_v[128], s_b[128], s_u[64], s_red[8];
  const int bg = blockIdx.x, b = bg / groups, g = bg % groups, hpg = heads / groups;
  const int j = threadIdx.x, lane = j & 31, warp = j >> 5;
  s_b[j] = to_f32(Bprev[(size_t)bg * 128 + j]);
  float acc_db = 0.f;   // this lane of dB_prev, summed over the heads of the group
  for (int hh = 0; hh < hpg; ++hh) {
    const size_t bh = (size_t)b * heads + g * hpg + hh;
    const float* Dh = D + bh * 64 * 128;
    const float mr = M[bh * T * 2], mi = M[bh * T * 2 + 1];
    const float kr = K[bh * T * 4], ki = K[bh * T * 4 + 1];
    const float den = mr * mr + mi * mi;
    const float xr = (kr * mr + ki * mi) / den, xi = (ki * mr - kr * mi) / den;   // X = kp_0 / m_0
    __syncthreads();   // s_u, s_v of the previous head are no longer read
    if (j < 64) s_u[j] = to_f32(Uprev[bh * 64 + j]);
    __syncthreads();
    float v = 0.f;
#pragma unroll 8
    for (int p = 0; p < 64; ++p) v += s_u[p] * Dh[p * 128 + j];
    s_v[j] = v;
    __syncthreads();
    // conj(X) v on the (re, im) pair this lane belongs to
    const float vr = s_v[j & ~1], vi = s_v[j | 1];
    acc_db += (j & 1) ? (xr * vi - xi * vr) : (xr * vr + xi * vi);
    // dX = sum_n conj(b[n]) v[n]: lane pairs contribute (re: br vr + bi vi, im: br vi - bi vr)
    float cr = 0.f, ci = 0.f;
    if (!(j & 1)) {
      const float br = s_b[j], bi = s_b[j + 1];
      cr = br * vr + bi * vi;
      ci = br * vi - bi * vr;
    }
    cr = warp_sum(cr); ci = warp_sum(ci);
    if (lane == 0) { s_red[2 * warp] = cr; s_red[2 * warp + 1] = ci; }
    // dU_prev[p] = Re sum_n conj(X b[n]) D[p,n]   (threads 0..63: one row each)
    if (j < 64 && dUprev) {
      float du = 0.f;
      for (int n = 0; n < 64; ++n) {
        const float yr = xr * s_b[2 * n] - xi * s_b[2 * n + 1], yi = xr * s_b[2 * n + 1] + xi * s_b[2 * n];   // X b
        const float2 d2 = *reinterpret_cast<const float2*>(Dh + j * 128 + 2 * n);
        du += yr * d2.x + yi * d2.y;
      }
      dUprev[bh * 64 + j] = from_f32<TIn>(du);
    }
    __syncthreads();
    if (j == 0)
      dg_boundary[bh] = make_float2(s_red[0] + s_red[2] + s_red[4] + s_red[6], s_red[1] + s_red[3] + s_red[5] + s_red[7]);
  }
  if (dBprev) dBprev[(size_t)bg * 128 + j] = from_f32<TIn>(acc_db);
}
