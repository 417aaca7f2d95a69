// The per-request part of decode_kernel: warp groups, TMA producer, q prologue, the main loop over the chunks, the
// combination of the warps and the epilogue. Not a header: decode_kernel includes this text where it handles one request,
// with GS_C in scope: the group size as a compile-time constant, or 0 when it is only known at run time (rs.gs). Every
// name used here (a, rs, req, p0, p1, u, uend, ts geometry, the ring and its barriers ...) is decode_kernel's.
    // ---- warp groups for this request; the ring and its barriers are re-partitioned when the group size changes
    //      (everything issued so far has been consumed at this point) ----
    const int GS = GS_C ? GS_C : rs.gs, lgs = GS >> 1 /* log2 of 1, 2, 4 */, NG = NWARPS >> lgs, gidx = warp >> lgs,
              msl = warp & (GS - 1);
    // Ring geometry of a group. m-tile groups: 3 * GS stages of one chunk of one head; head groups: 3 stages of one
    // chunk of GS heads. Either way the group owns 3 * GS * STAGE bytes and keeps PD chunks in flight.
    const int HS = hgm ? GS : 1;                                 // heads per TMA box
    const int RD = hgm ? NSTAGE : NSTAGE * GS;                   // stages in the ring
    const int PD = hgm ? NSTAGE - 1 : (NSTAGE - 1) * GS;         // prefetch distance, in chunks of the group
    const uint32_t SB = HS * Gm::STAGE;                           // bytes per stage
    if (GS != cur_gs) {
      if (tid == 0) {
        for (int i = 0; i < NSTG; ++i) {
          mbar_inval(smem_u32(&s_full[i])), mbar_inval(smem_u32(&s_empty[i]));
          mbar_init(smem_u32(&s_full[i]), 1);
          mbar_init(smem_u32(&s_empty[i]), GS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      }
      fence_proxy_async();
      __syncthreads();
      cur_gs = GS;
      cst = 0, cpass = 0;
    }
    const uint32_t gring = ring + gidx * NSTAGE * GS * Gm::STAGE;
    const uint32_t gfull = smem_u32(&s_full[gidx * NSTAGE * GS]), gempty = smem_u32(&s_empty[gidx * NSTAGE * GS]);

    // ---- items (kv head, m-tile group) of this request that intersect [u, uend) ----
    while (u < uend && u < p1) {
      const int item = (u - p0) / nchunks, c0 = (u - p0) - item * nchunks;
      const int kv_base = hgm ? item * GS : item / rs.mgroups;       // first (or only) kv head of the item
      const int mg = hgm ? 0 : item - kv_base * rs.mgroups;           // m-tile group of the item
      const int kvh = kv_base + (hgm ? msl : 0);                      // this warp's kv head
      const int c1 = min(nchunks, c0 + (uend - u));
      const bool whole = (c0 == 0 && c1 == nchunks);
      // the group consumes chunks c0 + gidx + NG * i, i < nig; inside the group warp msl produces i = msl + GS * ip
      const int nig = (c1 - c0 - gidx + NG - 1) / NG;
      const int npw = (nig - msl + GS - 1) >> lgs;
      const int mtw = hgm ? 0 : mg * GS + msl;      // this warp's m tile
      const bool active = mtw < rs.mtiles;

      // -- TMA producer: page ids 16 chunks at a time, one lane per 16-key half chunk --
      int pg_cur = 0, pg_next = 0;
      auto chunk_of = [&](int ip) { return c0 + gidx + NG * (msl + GS * ip); };
      auto load_pages = [&](int batch) {
        const int ip = 16 * batch + (lane >> 1);
        int pg = 0;
        if (ip < npw) {
          const int c = chunk_of(ip);
          const int n0 = c * CHUNK + (lane & 1) * 16;
          pg = bt[(n0 < L ? n0 : c * CHUNK) >> a.lbs];
        }
        return pg;
      };
      // dist: how far ahead of the consumer position (in the group's chunk sequence) the chunk lies, < RD
      auto issue = [&](int ip, int dist) {
        if ((ip & 15) == 0) {
          pg_cur = (ip == 0) ? load_pages(0) : pg_next;
          pg_next = load_pages((ip >> 4) + 1);
        }
        const int pa = __shfl_sync(0xffffffffu, pg_cur, 2 * (ip & 15));
        const int pb = __shfl_sync(0xffffffffu, pg_cur, 2 * (ip & 15) + 1);
        int st = cst + dist, prev_pass = cpass - 1;   // pass in which the stage was last used
        if (st >= RD) st -= RD, prev_pass = cpass;
        if (GS > 1 && prev_pass >= 0)   // the other warps of the group must have left the stage's previous contents
          ok = ok && __all_sync(0xffffffffu, mbar_wait(gempty + st * 8, prev_pass & 1));
        if (lane == 0 && ok) {
          const uint32_t bar = gfull + st * 8, dst = gring + st * SB;
          const int c = chunk_of(ip);
          mbar_expect_tx(bar, SB);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int n0 = c * CHUNK + half * 16;
            const int off = (n0 < L ? n0 : c * CHUNK) & a.bs_mask;
            const int page = half ? pb : pa;
            // coordinate slot s holds whichever of (offset in block, head, block) the tensor map put there
            auto coord = [&](const int (&pos)[3], int s) { return pos[0] == s ? off : (pos[1] == s ? kv_base : page); };
            tma_load_4d(dst + half * 16 * HS * D, &tm_k, 0, coord(a.kpos, 1), coord(a.kpos, 2), coord(a.kpos, 3), bar);
            tma_load_4d(dst + SB / 2 + half * 16 * HS * D, &tm_v, 0, coord(a.vpos, 1), coord(a.vpos, 2),
                        coord(a.vpos, 3), bar);
          }
        }
      };
      // Single-token decode: this warp's q rows are requested before the K/V prefetch below. Behind a full ring of
      // bulk loads (~200 KB per SM) a plain load waits for microseconds; ahead of it, it costs one round trip.
      uint2 q_early[NROWS / NWARPS];
      float sk_early[4];
      const bool early_q = !ROWS16 && GS == 1;
      if (early_q) {
        q_load_scale<D>(a, kvh, lane, sk_early);
#pragma unroll
        for (int k = 0; k < NROWS / NWARPS; ++k)
          q_early[k] = q_load_row<D, NROWS>(a, tok, qlen, kvh, mg, warp + NWARPS * k, lane);
      }
      // A single-warp group refills a stage right after consuming it, so it can fill its whole ring now and keep
      // HBM busy through the q prologue; a shared ring keeps one stage back for the other warps of the group.
      if (ok)
        for (int ip = 0; ip < npw && msl + GS * ip < (GS == 1 ? NSTAGE : PD); ++ip) issue(ip, msl + GS * ip);

      // -- q prologue for every m tile of the group --
      if (early_q) {
#pragma unroll
        for (int k = 0; k < NROWS / NWARPS; ++k)
          q_quantize_row<D, QG>(a, q_early[k], sk_early, s_q, s_chi, s_clo, kvh, warp + NWARPS * k, lane);
      } else {
        for (int sl = 0; sl < GS; ++sl) {   // slot = m tile of the group, or kv head of the head group
          const int mts = hgm ? 0 : mg * GS + sl;
          if (mts < rs.mtiles)
            q_prologue<D, NROWS, QG>(a, s_q + sl * 16 * QROW, s_chi + sl * 16 * (QG ? KSTEPS : 1), s_clo + sl * 16, tok, qlen,
                                     kv_base + (hgm ? sl : 0), mts, warp, lane);
        }
      }
      __syncthreads();
      TileState<D, ROWS16, QG> ts;
      {
        const int8_t* q_t = s_q + msl * 16 * QROW;
#pragma unroll
        for (int s = 0; s < KSTEPS; ++s) {
          ts.qa[s][0] = *reinterpret_cast<const uint32_t*>(&q_t[g * QROW + 32 * s + 4 * t]);
          ts.qa[s][2] = *reinterpret_cast<const uint32_t*>(&q_t[g * QROW + 32 * s + 16 + 4 * t]);
          ts.qa[s][1] = ROWS16 ? *reinterpret_cast<const uint32_t*>(&q_t[(g + 8) * QROW + 32 * s + 4 * t]) : 0u;
          ts.qa[s][3] = ROWS16 ? *reinterpret_cast<const uint32_t*>(&q_t[(g + 8) * QROW + 32 * s + 16 + 4 * t]) : 0u;
        }
        if constexpr (QG) {
          // [slot][16 rows][slices] floats from s_chi on: with four slots this reaches into s_clo, s_m and s_l, which
          // nobody else uses between the prologue and the barrier below
          ts.ch0 = ts.cl0 = ts.ch1 = ts.cl1 = 0.f;
#pragma unroll
          for (int c = 0; c < KSTEPS; ++c) {
            ts.cg0[c] = s_chi[(msl * 16 + g) * KSTEPS + c];
            ts.cg1[c] = s_chi[(msl * 16 + g + 8) * KSTEPS + c];
          }
          __syncthreads();   // every warp holds its scales before a warp without chunks writes s_m / s_l at the item's end
        } else {
          ts.ch0 = s_chi[msl * 16 + g], ts.cl0 = s_clo[msl * 16 + g];
          ts.ch1 = s_chi[msl * 16 + g + 8], ts.cl1 = s_clo[msl * 16 + g + 8];
        }
        // causal key limit per row: key n is visible iff n < L - qlen + 1 + (query token of the row)
        auto row_lim = [&](int r) {
          const int rt = (mtw * 16 + r) / a.G;
          return rt < qlen ? L - qlen + 1 + rt : L;
        };
        ts.lim0 = row_lim(g), ts.lim1 = row_lim(g + 8);
        ts.m0 = ts.m1 = -1e30f, ts.l0 = ts.l1 = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int e = 0; e < (ROWS16 ? 4 : 2); ++e) ts.acc[j][e] = 0.f;
      }
      const int lim_all = L - qlen + 1;  // every row sees keys below this

      // -- main loop over the group's chunks --
      for (int i = 0; i < nig && ok; ++i) {
        // keep PD chunks of the group in flight: chunk i + PD is issued by the warp whose turn it is
        // (a single-warp group pre-issued NSTAGE chunks, so its first in-loop issue is chunk NSTAGE at i == 1)
        const int jn = i + PD;
        if ((jn & (GS - 1)) == msl && jn < nig && (GS > 1 || i > 0)) issue(jn >> lgs, PD);
        const int st = cst;
        ok = ok && __all_sync(0xffffffffu, mbar_wait(gfull + st * 8, cpass & 1));
        if (!ok) break;
        if (active) {
          const uint32_t sk = gring + st * SB;
          chunk_step<D, ROWS16, QG>(ts, sk, sk + SB / 2, (c0 + gidx + NG * i) * CHUNK, lim_all, krow, kmat, vrow, t, HS,
                                    hgm ? msl : 0);
        }
        __syncwarp();  // every lane is done with this stage before it is refilled
        if (GS > 1 && lane == 0) mbar_arrive(gempty + st * 8);
        if (++cst == RD) cst = 0, ++cpass;
      }
      if (!ok) a.cta_status[blockIdx.x] = 1;

      // -- combine the warps that worked on the same m tile (slot msl of every group): weights exp(m_w - M) --
      if (t == 0) {
        s_m[warp * 16 + g] = ts.m0, s_l[warp * 16 + g] = ts.l0;
        s_m[warp * 16 + g + 8] = ts.m1, s_l[warp * 16 + g + 8] = ts.l1;
      }
      __syncthreads();  // also: every warp has left the ring, which s_acc aliases
      {
        float M0 = -1e30f, M1 = -1e30f;
        for (int w = msl; w < NWARPS; w += GS) M0 = fmaxf(M0, s_m[w * 16 + g]), M1 = fmaxf(M1, s_m[w * 16 + g + 8]);
        const float w0 = ex2((ts.m0 - M0) * LOG2E), w1 = ex2((ts.m1 - M1) * LOG2E);
        float* dst0 = s_acc + (warp * NROWS + g) * ACC_RS + 2 * t;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          *reinterpret_cast<float2*>(dst0 + 8 * j) = make_float2(ts.acc[j][0] * w0, ts.acc[j][1] * w0);
          if (ROWS16)
            *reinterpret_cast<float2*>(dst0 + 8 * ACC_RS + 8 * j) =
                make_float2(ts.acc[j][ROWS16 ? 2 : 0] * w1, ts.acc[j][ROWS16 ? 3 : 1] * w1);
        }
        if (tid < GS * 16) {
          const int sl = tid >> 4, r = tid & 15;
          float Mr = -1e30f, Lr = 0.f;
          for (int w = sl; w < NWARPS; w += GS) Mr = fmaxf(Mr, s_m[w * 16 + r]);
          for (int w = sl; w < NWARPS; w += GS) Lr += s_l[w * 16 + r] * ex2((s_m[w * 16 + r] - Mr) * LOG2E);
          s_M[tid] = Mr;
          s_inv[tid] = whole ? 1.f / fmaxf(Lr, 1e-30f) : Lr;
        }
      }
      __syncthreads();

      // -- epilogue: 4 channels per thread and step; s_v applied here --
      const int seg_slot = first_seg ? 0 : 1;
      const int slot_base = (blockIdx.x * 2 + seg_slot) * a.part_rows;
      for (int i = tid; i < GS * NROWS * (D / 4); i += NTHREADS) {
        const int sl = i / (NROWS * (D / 4)), rem = i - sl * (NROWS * (D / 4));
        const int row = rem / (D / 4), c4 = (rem - row * (D / 4)) * 4;
        const int mts = hgm ? 0 : mg * GS + sl, kvs = kv_base + (hgm ? sl : 0);   // m tile and kv head of the slot
        const int R = mts * 16 + row, rt = R / a.G, rh = R - rt * a.G;
        if (mts >= rs.mtiles || rt >= qlen) continue;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int w = sl; w < NWARPS; w += GS) {   // fixed order: deterministic
          const float4 x = *reinterpret_cast<const float4*>(s_acc + (w * NROWS + row) * ACC_RS + c4);
          v.x += x.x, v.y += x.y, v.z += x.z, v.w += x.w;
        }
        float4 sv4;
        if (a.pc_v) {
          sv4 = __ldg(reinterpret_cast<const float4*>(a.vs + kvs * D + c4));
        } else {
          const float one = __ldg(a.vs + kvs);
          sv4 = make_float4(one, one, one, one);
        }
        if (whole) {
          const float inv = s_inv[sl * 16 + row];
          const uint2 o = make_uint2(pack_bf16x2(v.x * inv * sv4.x, v.y * inv * sv4.y),
                                     pack_bf16x2(v.z * inv * sv4.z, v.w * inv * sv4.w));
          *reinterpret_cast<uint2*>(a.out + (tok + rt) * a.o_st + (kvs * a.G + rh) * a.o_sh + c4) = o;
        } else {
          const int prow = slot_base + sl * 16 + row;
          *reinterpret_cast<float4*>(a.part_acc + static_cast<int64_t>(prow) * D + c4) =
              make_float4(v.x * sv4.x, v.y * sv4.y, v.z * sv4.z, v.w * sv4.w);
          if (c4 == 0) {
            a.part_ml[prow * 2] = s_M[sl * 16 + row];
            a.part_ml[prow * 2 + 1] = s_inv[sl * 16 + row];
          }
        }
      }
      // generic-proxy writes to the ring (s_acc) come before the next item's TMA writes
      fence_proxy_async();
      __syncthreads();
      u += c1 - c0;
      first_seg = false;
      if (u == uend && tid == 0) {
        // Boundary record for the merge kernel: the item this CTA's range ends inside of, if this is the first CTA
        // boundary inside that item (an item cut several times is merged once, by its first boundary).
        const int A = p0 + item * nchunks;
        int4* rec = reinterpret_cast<int4*>(a.bnd + blockIdx.x * 8);
        if (c1 < nchunks && A >= ubeg) {
          rec[0] = make_int4(req, kv_base, mg, A);
          // the last CTA the item reaches: the one whose cost range holds the item's last unit
          const int f_last = f0 + item * (nchunks + P) + P + nchunks - 1;
          rec[1] = make_int4(f_last / Wf, tok, qlen, (seg_slot << 16) | (GS << 8) | rs.mtiles);
        } else {
          rec[0] = make_int4(-1, 0, 0, 0);
        }
      }
    }
