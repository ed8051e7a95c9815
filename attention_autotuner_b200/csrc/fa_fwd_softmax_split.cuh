// Softmax role of fa_fwd_sm100_kernel for Cfg::SPLIT == 2: two warpgroups per query tile, two threads per
// score row (64 columns each). Textually included inside the kernel body (it uses the kernel's locals).
//
// Warp w < 8*NQ:  query tile s = w / 8,  column half h = (w / 4) % 2,  TMEM lane quadrant w % 4.
// Per KV block the two threads of a row exchange their partial row maximum through shared memory (one named
// barrier of the tile's 256 threads; the buffer alternates with the block parity so that a thread that is one
// block ahead never overwrites a value its partner has not read yet). Row sums stay partial until the epilogue.
{
  constexpr int BNH = BN / 2;   // score columns per thread
  constexpr int DVH = DV / 2;   // output columns per thread (rescale, epilogue)
  const int s = warp >> 3;
  const int h = (warp >> 2) & 1;
  const int row_in_tile = threadIdx.x & 127;  // TMEM lane
  const int row = m_base + s * BM + row_in_tile;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
  const uint32_t tS = tmem_addr(tmem_base, lane_base, s * 128 + h * BNH);        // my 64 score columns
  // my 32 packed P columns overlay the FIRST half of my own 64 score columns (P of the tile is therefore at
  // columns [0,32) and [64,96) of its S region; the MMA warp addresses it accordingly)
  const uint32_t tP = tS;
  const uint32_t tO = tmem_addr(tmem_base, lane_base, NQ * 128 + s * DV + h * DVH);
  const int n_my = nblk[s];
  const int causal_shift = p.Lkv - p.Lq;
  float* xmax = xchg + s * (3 * 2 * 128);  // [2 parities][2 halves][128 rows]
  float* xsum = xmax + 2 * 2 * 128;        // [2 halves][128 rows]
  const int bar_id = 1 + s;

  float m_ref = -INFINITY;
  float l_sum = 0.f;  // partial: my 64 columns only
  bool ok = true;

  for (int j = 0; j < n_my; ++j) {
    ok = mbar_wait_warp(&s_full[s], j & 1, ab, kTagSFull);
    if (!ok) break;
    tc_fence_after();
    // Two passes over my 64 score columns, 32 at a time, so that a thread never holds more than one chunk:
    // with four softmax warpgroups the register budget is 96 per thread. Pass 1 finds the row maximum,
    // pass 2 (after the exchange) re-reads the scores from tensor memory and exponentiates them.
    const int n0 = j * BN + h * BNH;  // first key of my columns
    const bool tail_blk = (j * BN + BN > p.Lkv);
    const bool diag_blk = p.causal && (j * BN + BN - 1 > m_base + s * BM + causal_shift);
    int limit = BNH;  // my columns [limit, BNH) are masked
    if (tail_blk || diag_blk) {
      limit = p.Lkv - n0;
      if (p.causal) {
        const int cl = row + causal_shift - n0 + 1;
        limit = cl < limit ? cl : limit;
      }
    }
    float m_loc = -INFINITY;
#pragma unroll
    for (int c0 = 0; c0 < BNH; c0 += 32) {
      float sv[32];
      tmem_ld32(tS + c0, reinterpret_cast<uint32_t*>(sv));
      tc_wait_ld();
      if (tail_blk || diag_blk) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c0 + c >= limit) sv[c] = -INFINITY;
      }
      float mA = sv[0], mB = sv[1], mC = sv[2], mD = sv[3];
#pragma unroll
      for (int c = 4; c < 28; c += 8) {
        mA = fmax3(mA, sv[c], sv[c + 1]);
        mB = fmax3(mB, sv[c + 2], sv[c + 3]);
        mC = fmax3(mC, sv[c + 4], sv[c + 5]);
        mD = fmax3(mD, sv[c + 6], sv[c + 7]);
      }
      mA = fmax3(mA, sv[28], sv[29]);
      mB = fmax3(mB, sv[30], sv[31]);
      m_loc = fmaxf(m_loc, fmaxf(fmaxf(mA, mB), fmaxf(mC, mD)));
    }
    // exchange with the thread that owns the other half of this row
    float* xm = xmax + (j & 1) * (2 * 128);
    xm[h * 128 + row_in_tile] = m_loc;
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    const float m_blk = fmaxf(m_loc, xm[(h ^ 1) * 128 + row_in_tile]);

    // Lazy rescale (both halves take the same decision: it depends on the combined maximum only)
    bool need = (j == 0) || ((m_blk - m_ref) * p.scale_log2 > 8.0f);
    if (m_blk == -INFINITY) need = false;
    if (__any_sync(0xffffffffu, need)) {
      float alpha = 1.0f;
      if (need) {
        alpha = (m_ref == -INFINITY) ? 0.0f : ex2_approx((m_ref - m_blk) * p.scale_log2);
        m_ref = m_blk;
        l_sum *= alpha;
      }
      if (j > 0) {
        // O was last written by PV(j-1); wait for it, then scale my half of the columns in place
        ok = mbar_wait_warp(&o_done[s], (j - 1) & 1, ab, kTagODone);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < DVH; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tO + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tO + c0, r);
        }
      }
    }
    const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref * p.scale_log2;
    const uint64_t sl2 = f2_pack(p.scale_log2, p.scale_log2);
    const uint64_t nm2 = f2_pack(neg_m, neg_m);
    uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int c0 = 0; c0 < BNH; c0 += 32) {
      float sv[32];
      tmem_ld32(tS + c0, reinterpret_cast<uint32_t*>(sv));
      tc_wait_ld();
      if (tail_blk || diag_blk) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c0 + c >= limit) sv[c] = -INFINITY;
      }
      uint32_t pk[16];
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const uint64_t x2 = ffma2(f2_pack(sv[c], sv[c + 1]), sl2, nm2);
        float e0, e1;
        if (((c >> 1) & 7) < Cfg::EXP_EMU) {
          exp2_poly2(x2, e0, e1);
        } else {
          float x0, x1;
          f2_unpack(x2, x0, x1);
          e0 = ex2_approx(x0);
          e1 = ex2_approx(x1);
        }
        acc[(c >> 1) & 3] = fadd2(acc[(c >> 1) & 3], f2_pack(e0, e1));
        pk[c >> 1] = pack2<BF16>(e0, e1);
      }
      // overlays score columns this thread has already re-read (chunk c0 is written into columns [c0/2, c0/2+16))
      tmem_st16(tP + c0 / 2, pk);
    }
    {
      float a0, a1;
      f2_unpack(fadd2(fadd2(acc[0], acc[1]), fadd2(acc[2], acc[3])), a0, a1);
      l_sum += a0 + a1;
    }
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(&p_full[s]);
  }

  // epilogue: combine the two partial row sums, O / l -> global (my half of the columns), lse
  if (ok && n_my > 0) {
    xsum[h * 128 + row_in_tile] = l_sum;
    asm volatile("bar.sync %0, 256;" ::"r"(bar_id) : "memory");
    const float l_tot = l_sum + xsum[(h ^ 1) * 128 + row_in_tile];
    ok = mbar_wait_warp(&o_done[s], (n_my - 1) & 1, ab, kTagODone);
    if (ok) {
      tc_fence_after();
      const float inv_l = l_tot > 0.f ? 1.0f / l_tot : 0.f;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (static_cast<size_t>(bh) * p.Lq + row) * p.dv_total + dv_off + h * DVH;
#pragma unroll
      for (int c0 = 0; c0 < DVH; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tO + c0, r);
        tc_wait_ld();
        if (row < p.Lq) {
#pragma unroll
          for (int i = 0; i < 32; i += 16) {
            uint32_t v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = pack2<BF16>(__uint_as_float(r[i + 2 * e]) * inv_l, __uint_as_float(r[i + 2 * e + 1]) * inv_l);
            st_global_v8(orow + c0 + i, v);
          }
        }
      }
      if (p.lse != nullptr && dv_off == 0 && h == 0 && row < p.Lq) {
        p.lse[static_cast<size_t>(bh) * p.Lq + row] = (l_tot > 0.f) ? (m_ref * p.scale + __logf(l_tot)) : -INFINITY;
      }
    }
  } else if (ok && n_my == 0 && row < p.Lq) {
    uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (static_cast<size_t>(bh) * p.Lq + row) * p.dv_total + dv_off + h * DVH;
    for (int c = 0; c < DVH; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
    if (p.lse != nullptr && dv_off == 0 && h == 0) p.lse[static_cast<size_t>(bh) * p.Lq + row] = -INFINITY;
  }
}
