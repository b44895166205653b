// Forward kernel of the chunked scan on tcgen05 (included by scan_tc.cu inside its namespaces).
//
// NW = warps per TMEM lane quadrant (2 or 4).  The CTA has 4*NW worker warps; warp w reads TMEM
// lanes 32*(w & 3) .. +31 (a hardware rule) and, inside every accumulator, the column group
// (w >> 2) of NW.  All MMAs have M = 64, whose rows live in lanes 0..15 of every quadrant.  The
// epilogues read them with the 16x256b shape of tcgen05.ld, which spreads those 16 lanes over all
// 32 threads of the warp: thread t owns rows 16*quad + t/4 and + 8 and, in every block of 8
// columns, the column pair 2*(t%4), 2*(t%4)+1 - a complex pair stays inside one thread.  Every
// tcgen05.mma costs the tensor pipe >= 44 cycles whatever its N, so operands are laid out for few,
// wide instructions: [K' ; Zv] is one 128-row B operand (scores and off-term in one MMA per
// k-step) and K'' is one 128-column MN-major operand.
//
// STATES_ONLY: the state pre-sweep of the backward pass (no C, no scores, no Y).
template <typename TIn, typename TY, bool STATES_ONLY, int NW>
__global__ void __launch_bounds__(128 * NW + 64, 1) scan_tc_fwd_kernel(const __grid_constant__ TcFwdParams p) {
  constexpr int NT = 128 * NW;  // worker threads; two more warps: per-chunk scalars, TMA + MMA issue
  constexpr int ZC = 128 / NW;  // state columns per warp
  constexpr int SC = 64 / NW;   // score / output columns per warp
  constexpr int SB = SC / 8;    // 8-column blocks of a score / output group
  constexpr int ZB = ZC / 8;    // 8-column blocks of a state group: 2 ZB state values per thread and row
  constexpr int RSTEP = NT / 16;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar_tma[2], bar_mma[3], bar_drain;   // bar_mma: [S|Yoff] | Inc | Ydiag
  __shared__ uint64_t bar_st;                  // Y tile staged in shared memory (16-bit outputs)
  constexpr bool Y_TMA = !STATES_ONLY && sizeof(TY) == 2;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  float* sc_tab = reinterpret_cast<float*>(smem + OFF_SCAL);   // two tables: chunk parity
  using PK = Pack2<TIn>;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool worker = warp < 4 * NW;     // warp 4 NW runs chunk_scalars one chunk ahead, warp 4 NW + 1 issues
  const int quad = warp & 3, cg = worker ? (warp >> 2) : 0;
  const int rowA = 16 * quad + (lane >> 2), rowB = rowA + 8;  // epilogue identity: two rows ...
  const int cq = lane & 3;                                    // ... and one column pair per 8-column block
  const int rcol = tid & 15, rrow0 = tid >> 4;               // rotation identity
  const uint32_t lane_base = (uint32_t)(32 * quad) << 16;
  const int bh = blockIdx.x, b = bh / p.heads, h = bh % p.heads;
  const int bg = b * p.groups + h / (p.heads / p.groups);
  const int T = p.T;
  const float* Mb = p.M + (size_t)bh * T * 2;
  const float* Kb = p.K + (size_t)bh * T * 4;
  const long long wl = p.wait_limit;   // limit of the main loop's waits (the drain waits keep the default)

  if (tid == 0) {
    mbar_init(&bar_tma[0], 1); mbar_init(&bar_tma[1], 1);
    for (int i = 0; i < 3; ++i) mbar_init(&bar_mma[i], 1);
    mbar_init(&bar_st, 4 * NW);   // one arrival per worker warp
    mbar_init(&bar_drain, 1);
    fence_barrier_init();
    s_abort = 0;
    tma_prefetch_desc(&p.tmU); tma_prefetch_desc(&p.tmB); tma_prefetch_desc(&p.tmC);
    if (Y_TMA) tma_prefetch_desc(&p.tmY);
    if (p.states16) tma_prefetch_desc(&p.tmS);
  }
  if (warp == 0) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  auto issue_loads = [&](int c) {   // one thread
    uint8_t* st = smem + (c & 1) * STAGE;
    uint64_t* bar = &bar_tma[c & 1];
    mbar_expect_tx(bar, (STATES_ONLY ? 3 : 5) * TILE);
    tma_load_3d(st, &p.tmU, bar, 0, c * L, bh);
    tma_load_3d(st + TILE, &p.tmB, bar, 0, c * L, bg);
    tma_load_3d(st + 3 * TILE, &p.tmB, bar, 64, c * L, bg);
    if (!STATES_ONLY) {
      tma_load_3d(st + 5 * TILE, &p.tmC, bar, 0, c * L, bg);
      tma_load_3d(st + 6 * TILE, &p.tmC, bar, 64, c * L, bg);
    }
  };
  if (tid == 0) issue_loads(0);

  // ---- carried state, conjugated: zv[2j], zv[2j+1] = (re, -im) of column pair j of this thread ----
  const int d0 = cg * ZC;             // first state column (0..127) of this warp
  // zv[4 i + 2 h + k]: block i, row (h ? rowB : rowA), k = 0 real part, 1 minus the imaginary part
  float zv[4 * ZB];
#pragma unroll
  for (int j = 0; j < 4 * ZB; ++j) zv[j] = 0.f;
  if (worker) {
    const TIn* Bp = reinterpret_cast<const TIn*>(p.Bprev);
    const TIn* Up = reinterpret_cast<const TIn*>(p.Uprev);
    float cr = 0.f, ci = 0.f, up[2] = {0.f, 0.f};
    if (Bp) {  // pending prev-tap of the token before the sequence: u_prev (x) (kp_0 / m_0) b_prev
      const float mr = Mb[0], mi = Mb[1], kr = Kb[0], ki = Kb[1];
      const float den = mr * mr + mi * mi;
      cr = (kr * mr + ki * mi) / den; ci = (ki * mr - kr * mi) / den;
      up[0] = to_f32(Up[(size_t)bh * 64 + rowA]);
      up[1] = to_f32(Up[(size_t)bh * 64 + rowB]);
    }
#pragma unroll
    for (int i = 0; i < ZB; ++i) {
      const int d = d0 + 8 * i + 2 * cq;
      float br = 0.f, bi = 0.f;
      if (Bp) { br = to_f32(Bp[(size_t)bg * 128 + d]); bi = to_f32(Bp[(size_t)bg * 128 + d + 1]); }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float re = 0.f, im = 0.f;
        if (p.z0) {
          const float2 z = *reinterpret_cast<const float2*>(p.z0 + ((size_t)bh * 64 + (hh ? rowB : rowA)) * 128 + d);
          re = z.x; im = z.y;
        }
        re += up[hh] * (cr * br - ci * bi);
        im += up[hh] * (cr * bi + ci * br);
        zv[4 * i + 2 * hh] = re; zv[4 * i + 2 * hh + 1] = -im;
      }
    }
  }
  // 16-bit copy of the state for chunk c: rows p, K-major along d, in the Zv slots of stage c & 1
  // (directly below the K' rows, so that [K' ; Zv] is one 128-row operand)
  auto store_zv_tile = [&](int c) {
    uint8_t* stg = smem + (c & 1) * STAGE;
#pragma unroll
    for (int i = 0; i < ZB; ++i) {
      const int ci = d0 / 8 + i;   // 16-byte chunk index along d (0..15)
      uint8_t* tile = stg + (2 + 2 * (ci >> 3)) * TILE + 4 * cq;
      *reinterpret_cast<uint32_t*>(tile + sw128(rowA, ci & 7)) = PK::pack(zv[4 * i], zv[4 * i + 1]);
      *reinterpret_cast<uint32_t*>(tile + sw128(rowB, ci & 7)) = PK::pack(zv[4 * i + 2], zv[4 * i + 3]);
    }
  };
  if (worker) store_zv_tile(0);
  if (warp == 4 * NW) chunk_scalars(sc_tab, Mb, Kb, 0, T, lane);
  __syncthreads();

  constexpr uint32_t ID_S = make_idesc(64, 128, PK::fmt, 0, 0);    // K-major x K-major   [S | Yoff]
  constexpr uint32_t ID_Y = make_idesc(64, 64, PK::fmt, 0, 1);     // K-major x MN-major  Ydiag
  constexpr uint32_t ID_Z = make_idesc(64, 128, PK::fmt, 1, 1);    // MN-major x MN-major Inc
  const uint32_t aKPP = smem_u32(smem + OFF_KPP), aS = smem_u32(smem + OFF_S);
  bool ok = true;
  int issued_hi = 0;   // issue lane: the last chunk whose loads were requested (chunk 0 by thread 0 above)

  // ---- output epilogue of chunk cp: y = Y_diag + exp(l_t) Y_off.  It runs one iteration late, in the gap
  // while the [S | Yoff] MMAs of the next chunk execute (their accumulators alternate by chunk parity).
  float et_keep[2] = {0.f, 0.f};   // exp(l_t) of this thread's two rows in the chunk whose output is pending
  auto output_epilogue = [&](int cp, bool live) {
    float yadd[4 * SB];   // the summand of this thread's outputs, requested ahead of the wait
#pragma unroll
    for (int j = 0; j < 4 * SB; ++j) yadd[j] = 0.f;
    if (!STATES_ONLY && p.Yadd != nullptr && live) {
#pragma unroll
      for (int i = 0; i < SB; ++i)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int t = cp * L + (hh ? rowB : rowA);
          if (t < T) {
            const float2 a = __ldg(reinterpret_cast<const float2*>(
                p.Yadd + ((size_t)bh * T + t) * 64 + cg * SC + 8 * i + 2 * cq));
            yadd[4 * i + 2 * hh] = a.x; yadd[4 * i + 2 * hh + 1] = a.y;
          }
        }
    }
    if (live && !mbar_wait(&bar_mma[2], cp & 1, wl)) { report_timeout(4); s_abort = 1; live = false; }
    tc_fence_after_sync();
    if (live) {
      const int t0p = cp * L;
      uint32_t yd[4 * SB], yo[4 * SB];
      tmem_ld_16x256<SB>(tmem + lane_base + 256 + 64 * (cp & 1) + cg * SC, yd);
      tmem_ld_16x256<SB>(tmem + lane_base + 128 * (cp & 1) + 64 + cg * SC, yo);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < SB; ++i) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int R = hh ? rowB : rowA;
          const float et = hh ? et_keep[1] : et_keep[0];
          const float y0 = __uint_as_float(yd[4 * i + 2 * hh]) + et * __uint_as_float(yo[4 * i + 2 * hh]) +
                           yadd[4 * i + 2 * hh];
          const float y1 = __uint_as_float(yd[4 * i + 2 * hh + 1]) + et * __uint_as_float(yo[4 * i + 2 * hh + 1]) +
                           yadd[4 * i + 2 * hh + 1];
          if constexpr (sizeof(TY) == 2) {   // into the staging tile; rows beyond T are clipped by the store
            *reinterpret_cast<uint32_t*>(smem + OFF_Y + sw128(R, cg * SB + i) + 4 * cq) = Pack2<TY>::pack(y0, y1);
          } else if (t0p + R < T) {
            float* dst = reinterpret_cast<float*>(p.Y) + ((size_t)bh * T + t0p + R) * 64 + cg * SC + 8 * i + 2 * cq;
            *reinterpret_cast<float2*>(dst) = make_float2(y0, y1);
          }
        }
      }
    }
    if (Y_TMA) {   // the Y tile is complete once every worker warp has arrived
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_st);
    }
  };

  for (int c = 0; c < p.nchunks && ok; ++c) {
    const int t0 = c * L;
    uint8_t* st = smem + (c & 1) * STAGE;
    float* sc = sc_tab + (c & 1) * (NSCAL * 64);
    float* s_diag = sc + 11 * 64;
    if (warp == 4 * NW) {
      // scalars of the NEXT chunk, started once the workers are through the rotation pass (global
      // loads issued during the workers' shared-memory burst at the top of the iteration stalled
      // the whole SM for about a DRAM round trip)
      bar_sync(2, NT + 64);   // the workers only arrive here (bar_arrive): they never wait for this warp
      if (c + 1 < p.nchunks) chunk_scalars(sc_tab + ((c + 1) & 1) * (NSCAL * 64), Mb, Kb, t0 + L, T, lane);
    } else if (!worker) {
      // Issue warp (one lane): the MMAs of this chunk, the TMA loads of the NEXT one and the TMA
      // stores.  The workers never wait for this warp, only for the commit barriers of the products
      // they read: they arrive on named barriers 2 ("rotation done") and 4 ("S tile written") without
      // waiting and move on.
      const uint64_t bU = make_desc(smem_u32(st), 8192, 1024);
      const uint32_t tSY = tmem + 128 * (c & 1), tYD = tmem + 256 + 64 * (c & 1), tINC = tmem + 384;
      // scores and off-term: [S | Yoff] = Q [K' ; Zv]^T, accumulated over the state dimension
      const uint64_t bB = make_desc(smem_u32(st + TILE), 16, 1024);       // [K'_h ; Zv_h], h = k >> 2
      const uint64_t bC = make_desc(smem_u32(st + 5 * TILE), 16, 1024);   // Q
      if (lane == 0 && s_abort == 0 && c + 1 < p.nchunks) {
        // Next chunk's tiles, a whole iteration ahead (half an iteration was not always enough for the data
        // to arrive).  The stage being refilled held chunk c-1, whose last reader is its Y_diag MMA.
        if (!STATES_ONLY && c > 0 && !mbar_wait(&bar_mma[2], (c - 1) & 1, wl)) { report_timeout(8); s_abort = 1; }
        else { issue_loads(c + 1); issued_hi = c + 1; }
      }
      __syncwarp();
      bar_sync(5, NT + 32);   // first column halves of Q and K' rotated (the Zv tile is the previous chunk's)
      if (!STATES_ONLY && lane == 0 && s_abort == 0) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma(tSY, desc_adv(bC, k * 32), desc_adv(bB, k * 32), ID_S, k > 0);
      }
      __syncwarp();
      bar_sync(2, NT + 64);   // rotation done: Q, K', K'' written; U landed; Zv tile stored by the previous chunk
      const bool go = lane == 0 && s_abort == 0;
      if (go) {
        tc_fence_after_sync();
        if (!STATES_ONLY) {
#pragma unroll
          for (int k = 4; k < 8; ++k)
            umma(tSY, desc_adv(bC, TILE + (k & 3) * 32), desc_adv(bB, 2 * TILE + (k & 3) * 32), ID_S, 1);
          umma_commit(&bar_mma[0]);
        }
        // Inc = U^T K''
        const uint64_t bK = make_desc(aKPP, 8192, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma(tINC, desc_adv(bU, 2048 * k), desc_adv(bK, 2048 * k), ID_Z, k > 0);
        umma_commit(&bar_mma[1]);
        if (p.states16) {   // the 16-bit state tile of this chunk is exactly what the backward wants
          tma_store_3d(&p.tmS, st + 2 * TILE, 0, c * 64, bh);
          tma_store_3d(&p.tmS, st + 4 * TILE, 64, c * 64, bh);
          tma_store_commit();
        }
        if (Y_TMA && c > 0) {   // the workers stage the Y tile of the PREVIOUS chunk while the MMAs above run
          if (mbar_wait(&bar_st, (c - 1) & 1, wl)) {
            tma_store_3d(&p.tmY, smem + OFF_Y, 0, t0 - L, bh);
            tma_store_commit();
          } else { report_timeout(5); s_abort = 1; }
        }
      }
      __syncwarp();
      if (!STATES_ONLY) bar_sync(4, NT + 32);   // S tile written
      if (go && s_abort == 0) {
        if (!STATES_ONLY) {
          tc_fence_after_sync();
          const uint64_t bS = make_desc(aS, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // Y_diag = S U
            umma(tYD, desc_adv(bS, 32 * k), desc_adv(bU, 2048 * k), ID_Y, k > 0);
          umma_commit(&bar_mma[2]);
        }
        // the state tiles and the Y tile stored in this iteration are overwritten by the workers in
        // the next one: their stores must have read them by then (they were issued long ago)
        tma_store_wait_read();
      }
      __syncwarp();
    } else {
    bool live = true;   // cleared when a bounded wait expired: the rest of the chunk is skipped
    if (!mbar_wait(&bar_tma[c & 1], (c >> 1) & 1, wl)) { report_timeout(1); s_abort = 1; live = false; }

    // ---- rotation: C -> Q, B -> K' (both in place), K'' ; diagonal scores --------------------
    // Two phases, one per 64-column half of the state dimension: the score products accumulate over
    // that dimension, so the issue warp starts their first four k-steps (named barrier 5) while the
    // workers still rotate the second half.  A thread keeps its rows in both phases (8 threads per
    // row, one 16-byte piece each), so the diagonal sums stay in registers until the end.
    {
      constexpr int IPT = 512 / NT;   // (row, piece) items per thread and phase
      float dgk[IPT];
#pragma unroll
      for (int j = 0; j < IPT; ++j) dgk[j] = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (live) {
          uint8_t* tB = st + (1 + 2 * half) * TILE;
          uint8_t* tC = st + (5 + half) * TILE;
          uint8_t* tK = smem + OFF_KPP + half * TILE;
          uint4 cvk[IPT], bvk[IPT];
#pragma unroll
          for (int j = 0; j < IPT; ++j) {   // all loads first: the stores below are in place
            const int item = tid + NT * j;
            const uint32_t off = sw128(item >> 3, item & 7);
            cvk[j] = make_uint4(0u, 0u, 0u, 0u);
            if (!STATES_ONLY) cvk[j] = *reinterpret_cast<const uint4*>(tC + off);
            bvk[j] = *reinterpret_cast<const uint4*>(tB + off);
          }
#pragma unroll
          for (int j = 0; j < IPT; ++j) {
            const int item = tid + NT * j, r = item >> 3;
            const uint32_t off = sw128(r, item & 7);
            const float phr = sc[2 * 64 + r], phi = sc[3 * 64 + r];
            const float wr = sc[4 * 64 + r], wi = sc[5 * 64 + r];
            const float vr = sc[6 * 64 + r], vi = sc[7 * 64 + r];
            const float kr = sc[8 * 64 + r], ki = sc[9 * 64 + r];
            const uint4 cv = cvk[j], bv = bvk[j];
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
            dgk[j] += dg;
            *reinterpret_cast<uint4*>(tK + off) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
            if (!STATES_ONLY) {
              *reinterpret_cast<uint4*>(tC + off) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
              *reinterpret_cast<uint4*>(tB + off) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
            }
          }
        }
        if (half == 0) {   // first halves of Q and K' are complete: the score products may start
          fence_async_smem();
          tc_fence_before_sync();
          bar_arrive(5, NT + 32);
        }
      }
      if (live && !STATES_ONLY) {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
#pragma unroll
          for (int j = 0; j < IPT; ++j) dgk[j] += __shfl_xor_sync(0xffffffffu, dgk[j], o);
        }
        if ((tid & 7) == 0) {
#pragma unroll
          for (int j = 0; j < IPT; ++j) s_diag[(tid + NT * j) >> 3] = dgk[j];
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    // no barrier among the workers here: what a warp does next (the previous chunk's output, its decay
    // factors) touches nothing the rotation of another warp reads or writes; the diagonal values of
    // other warps are read after the score products' barrier, which all rotations precede
    bar_arrive(2, NT + 64);      // the scalar and issue warps are told without being waited for
    live = s_abort == 0;

    if (!STATES_ONLY) {
      // ---- [S | Yoff] and Inc MMAs are issued by the issue warp; meanwhile the output of the previous
      // chunk is finished ---------------------------------------------------------------------------------
      if (c > 0) output_epilogue(c - 1, live);
      live = live && s_abort == 0;
      // The wait and the TMEM load below are compiler barriers: what the scores epilogue reads from
      // shared memory (and the exponentials of it) is computed BEFORE the wait it would otherwise
      // queue behind.
      float dfac[4 * SB], dg2[2];   // decay factors of this thread's cells [hh][i][q]; diagonal values
      {
        float ls[2 * SB];
#pragma unroll
        for (int i = 0; i < SB; ++i) {
          const float2 l2 = *reinterpret_cast<const float2*>(sc + cg * SC + 8 * i + 2 * cq);
          ls[2 * i] = l2.x; ls[2 * i + 1] = l2.y;
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int R = hh ? rowB : rowA;
          const float lt = sc[R];
#pragma unroll
          for (int k = 0; k < 2 * SB; ++k) dfac[hh * 2 * SB + k] = __expf(fminf(lt - ls[k], 0.f));
        }
      }
      const float et_next[2] = {sc[1 * 64 + rowA], sc[1 * 64 + rowB]};
      if (live && !mbar_wait(&bar_mma[0], c & 1, wl)) { report_timeout(2); s_abort = 1; live = false; }
      tc_fence_after_sync();

      // ---- scores epilogue: decay, causal mask, diagonal -> 16-bit S tile ------------------------
      if (live) {
        uint32_t r[4 * SB];
        tmem_ld_16x256<SB>(tmem + lane_base + 128 * (c & 1) + cg * SC, r);
        tmem_ld_wait();
        et_keep[0] = et_next[0]; et_keep[1] = et_next[1];
        dg2[0] = s_diag[rowA]; dg2[1] = s_diag[rowB];
        uint8_t* tS = smem + OFF_S + 4 * cq;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int R = hh ? rowB : rowA;
          const float dgv = dg2[hh];
#pragma unroll
          for (int i = 0; i < SB; ++i) {
            float v2[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int s = cg * SC + 8 * i + 2 * cq + q;
              float v = __uint_as_float(r[4 * i + 2 * hh + q]) * dfac[hh * 2 * SB + 2 * i + q];
              v = s < R ? v : (s == R ? dgv : 0.f);
              v2[q] = v;
            }
            *reinterpret_cast<uint32_t*>(tS + sw128(R, cg * SB + i)) = PK::pack(v2[0], v2[1]);
          }
        }
      }
      fence_async_smem();
      tc_fence_before_sync();
      bar_arrive(4, NT + 32);   // the issue warp now issues Y_diag = S U (no barrier among the workers)
      live = s_abort == 0;
    }

    // ---- state update (hides the Y_diag MMAs; the output epilogue follows in the next iteration) ---------
    if (live && !mbar_wait(&bar_mma[1], c & 1, wl)) { report_timeout(3); s_abort = 1; live = false; }
    tc_fence_after_sync();
    // ---- state update: zv = conj(Pi_end) zv + Inc ---------------------------------------------------
    if (live) {
      const float pr = sc[10 * 64 + 0], pi = sc[10 * 64 + 1];
#pragma unroll
      for (int part = 0; part < ZB / 4; ++part) {
        uint32_t inc[16];
        tmem_ld_16x256<4>(tmem + lane_base + 384 + d0 + 32 * part, inc);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {   // 8 complex values: 4 blocks x 2 rows
          const float a = zv[16 * part + 2 * j], bq = zv[16 * part + 2 * j + 1];
          zv[16 * part + 2 * j] = pr * a + pi * bq + __uint_as_float(inc[2 * j]);
          zv[16 * part + 2 * j + 1] = pr * bq - pi * a + __uint_as_float(inc[2 * j + 1]);
        }
      }
      store_zv_tile(c + 1);
    }
    fence_async_smem();
    tc_fence_before_sync();
    }  // worker
    __syncthreads();
    if (s_abort) { ok = false; break; }
  }

  if (!STATES_ONLY && ok) {
    if (worker) {
      output_epilogue(p.nchunks - 1, true);
    } else if (Y_TMA && warp == 4 * NW + 1 && lane == 0) {
      if (mbar_wait(&bar_st, (p.nchunks - 1) & 1, wl)) {
        tma_store_3d(&p.tmY, smem + OFF_Y, 0, (p.nchunks - 1) * L, bh);
        tma_store_commit();
      } else { report_timeout(5); s_abort = 1; }
    }
  }
  if (ok && p.zfinal && worker) {
#pragma unroll
    for (int i = 0; i < ZB; ++i) {
      const int d = d0 + 8 * i + 2 * cq;
      *reinterpret_cast<float2*>(p.zfinal + ((size_t)bh * 64 + rowA) * 128 + d) = make_float2(zv[4 * i], -zv[4 * i + 1]);
      *reinterpret_cast<float2*>(p.zfinal + ((size_t)bh * 64 + rowB) * 128 + d) = make_float2(zv[4 * i + 2], -zv[4 * i + 3]);
    }
  }
  // Unwind: nothing of this CTA may still be in flight when shared memory and TMEM are released.  Every
  // asynchronous operation was started by the issue lane (but for the loads of chunk 0), so it drains them:
  // after an expired wait the loads of the last two requested chunks (their barriers, default long limit),
  // every tcgen05.mma issued so far (one more commit) and, always, its TMA stores.
  if (warp == 4 * NW + 1 && lane == 0) {
    if (s_abort)
      for (int cc = issued_hi > 0 ? issued_hi - 1 : 0; cc <= issued_hi; ++cc) mbar_wait(&bar_tma[cc & 1], (cc >> 1) & 1);
    umma_commit(&bar_drain);
    mbar_wait(&bar_drain, 0);
    tma_store_wait_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}
