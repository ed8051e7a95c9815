// MMA role of fa_fwd_sm100_kernel for Cfg::NMMA == 2 (needs NQ == 2): one issuing warp per query tile, taking
// strict turns. Textually included inside the kernel body (it uses the kernel's locals).
//
// Why: a tcgen05.mma costs its issuing thread about as long as it keeps the tensor pipe busy (~50 of 64 cycles
// for 128x128x16) and the pipe's queue is short, so every barrier wait (~100 cycles even when already complete)
// and commit between two batches of a single issuing thread is idle time of the pipe. Here each warp does its
// waits (K/V landed, P written) while the other warp is issuing, and issues as soon as it is handed the turn.
// The turns keep the two tiles in ping-pong order: tile 0 issues [PV(j), S(j+1)], then tile 1, then tile 0 ...
//
// Turn u of tile s:  u = 0: S(0);  u = j + 1: PV(j) and S(j + 1).  Both warps walk every ring item in order and
// release it once (kv_empty counts two arrivals): with a tcgen05.commit after the MMAs that read it, or with a
// plain arrival if the tile does not use that block (causal mask).
{
  const int s = warp - kMmaWarp;
  const int n_my = nblk[s];
  constexpr uint32_t idesc_qk = umma_idesc(BM, BN, BF16, false, false);
  constexpr uint32_t idesc_pv = umma_idesc(BM, DV, BF16, false, true);
  bool ok = true;
  uint32_t full_waited = 0;
  auto wait_item = [&](int t) -> bool {
    while (ok && static_cast<int>(full_waited) <= t) {
      ok = mbar_wait_warp(&kv_full[full_waited % NSTAGE], (full_waited / NSTAGE) & 1, ab, kTagKvFull);
      ++full_waited;
    }
    return ok;
  };
  const uint32_t qa = smem_u32(sQ) + s * Cfg::Q_TILE_BYTES;
  const uint32_t kv_addr = smem_u32(sKV);
  const uint32_t tS = tmem_base + s * 128;
  const uint32_t tO = tmem_base + NQ * 128 + s * DV;
  if (n_my > 0) ok = mbar_wait_warp(&q_full[s], 0, ab, kTagQ);

  for (int u = 0; u <= nmax && ok; ++u) {
    const int j = u - 1;
    const bool do_pv = (j >= 0 && j < n_my);
    const bool do_s = (u < n_my);
    // operands and P first: these waits run while the other tile's warp is issuing
    if (j >= 0 && !wait_item(2 * j + 1)) break;
    if (u < nmax && !wait_item(2 * u)) break;
    if (do_pv) {
      ok = mbar_wait_warp(&p_full[s], j & 1, ab, kTagPFull);
      if (!ok) break;
    }
    // then the turn: tile 0 goes first in every round
    if (s == 0) {
      if (u > 0) ok = mbar_wait_warp(&turn[0], (u - 1) & 1, ab, kTagTurn);
    } else {
      ok = mbar_wait_warp(&turn[1], u & 1, ab, kTagTurn);
    }
    if (!ok) break;
    tc_fence_after();
    if (elect_one()) {
      if (j >= 0) {
        const int slot = (2 * j + 1) % NSTAGE;
        if (do_pv) {
          const uint32_t va = kv_addr + slot * Cfg::KV_SLOT_BYTES;
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            const uint32_t pcol = (SPLIT == 2 && ks >= 4) ? 64 + (ks - 4) * 8 : ks * 8;
            umma_ts(tO, tS + pcol, umma_smem_desc(va + ks * 2048, BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(&o_done[s]);
          tc_commit(&kv_empty[slot]);
        } else {
          mbar_arrive(&kv_empty[slot]);
        }
      }
      if (u < nmax) {
        const int slot = (2 * u) % NSTAGE;
        if (do_s) {
          const uint32_t ka = kv_addr + slot * Cfg::KV_SLOT_BYTES;
#pragma unroll
          for (int ks = 0; ks < DQK / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (BM * 128) + (ks & 3) * 32;
            umma_ss(tS, umma_smem_desc(qa + off, 16, 1024), umma_smem_desc(ka + off, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc_commit(&s_full[s]);
          tc_commit(&kv_empty[slot]);
        } else {
          mbar_arrive(&kv_empty[slot]);
        }
      }
      mbar_arrive(&turn[s ^ 1]);  // the other tile's warp may issue now
    }
    __syncwarp();
  }
}
