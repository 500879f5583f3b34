// dQ on pairs of SMs (tcgen05 cta_group::2), for 64-row q and kv blocks and
// head dim 128.  Included by sparse_bwd.cu after sparse_bwd_dkv2.cuh (shares
// BwdParams and the cluster helpers).
//
// A cluster of two CTAs owns 256 query rows (four q-blocks); each CTA keeps its
// own 128 rows of Q and dO in TMEM, its own S / dP buffers and its own dQ
// accumulator, exactly as in the one-CTA kernel, and both walk the union of
// the four q-blocks' candidate lists.  Per kv block each CTA loads only
//   kv rows 32 r .. 32 r + 31 of K and of V (all of d) - its half of the B
//        operand of S = Q K^T and dP = dO V^T (N = 64 kv rows split in two),
//   d columns 64 r .. 64 r + 63 of K (all 64 rows) - its half of the B operand
//        of dQ += dS K (N = 128 split in two),
// 24 KB per tile for twice the query rows (the one-CTA kernel loads 32 KB),
// and the M = 256 UMMAs cost 43 cycles at N = 64 and 64 at N = 128 for both
// CTAs together, against 42 and 74 per CTA.  CTA 0 issues every UMMA;
// tcgen05.commit multicasts its arrivals; CTA 1's warp 1 forwards "my tiles
// have landed"; its compute warps arrive on CTA 0's barriers through the
// cluster shared-memory window.  No TMA load is multicast.
#pragma once

namespace ftk {

constexpr int DQ2_STAGES = 5;

// TMEM columns per CTA: Q 0..63, dO 64..127, S[2] 128/192, dP[2] 256/320 (dS
// over their first half), dQ 384..   Shared memory per CTA: Q 32 KB, dO 32 KB,
// 5 stages of [K rows-half 8 KB][V rows-half 8 KB][K d-half 8 KB].
template <int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BW_THREADS, 1)
sparse_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_k32,
                      const __grid_constant__ CUtensorMap tm_v32, const BwdParams p) {
  constexpr int D = 128;
  constexpr int NCH = 2;
  constexpr int ROW_TILE_BYTES = NCH * 128 * 128;
  constexpr int G = 64;
  constexpr int STAGE = 24576;
  constexpr int OFF_VROW = 8192, OFF_KCOL = 16384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + ROW_TILE_BYTES;
  uint8_t* sKV = smem + 2 * ROW_TILE_BYTES;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[2 + 3 * DQ2_STAGES + 5];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int m0 = (blockIdx.x >> 1) * 4;       // first of the pair's four q-blocks
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(4, p.QM - m0);
  const int tile_row0 = (m0 + 2 * static_cast<int>(rank)) * G - p.q_pad_head;   // my 128 rows

  const uint32_t bar_q = smem_u32(&bars[0]);         // my Q / dO tiles in shared memory
  const uint32_t bar_qt = smem_u32(&bars[1]);        // CTA 0: Q / dO of both CTAs sit in TMEM
  auto bar_kvfull = [&](int s) { return smem_u32(&bars[2 + s]); };
  auto bar_kvempty = [&](int s) { return smem_u32(&bars[2 + DQ2_STAGES + s]); };
  auto bar_peer_kv = [&](int s) { return smem_u32(&bars[2 + 2 * DQ2_STAGES + s]); };  // CTA 0 only
  constexpr int BAR_A0 = 2 + 3 * DQ2_STAGES;
  auto bar_afull = [&](int s) { return smem_u32(&bars[BAR_A0 + s]); };
  auto bar_dsfull = [&](int s) { return smem_u32(&bars[BAR_A0 + 2 + s]); };           // CTA 0 only
  const uint32_t bar_final = smem_u32(&bars[BAR_A0 + 4]);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_qt, 16);   // the 8 copying warps of each CTA
    for (int s = 0; s < DQ2_STAGES; s++) {
      mbar_init(bar_kvfull(s), 1);
      mbar_init(bar_kvempty(s), 1);
      mbar_init(bar_peer_kv(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_afull(s), 1);
      mbar_init(bar_dsfull(s), 16);   // 8 warps of the owning group in each CTA
    }
    mbar_init(bar_final, 1);
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_k32);
    tma_prefetch_desc(&tm_v32);
  }
  if (warp == 0) {
    tmem_alloc2(smem_u32(&tmem_base_s), 512);
    tmem_relinquish2();
  }
  // both CTAs build the same union over the pair's four candidate lists
  const int n = build_union(un, p.lists + (static_cast<int64_t>(bh) * p.QM + m0) * p.W, p.W,
                            groups, p.W, nullptr, p.Mkv, p.status);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_q, 2 * ROW_TILE_BYTES);
      for (int c = 0; c < NCH; c++) {
        tma_load_4d(smem_u32(sQ) + c * 128 * 128, &tm_q, bar_q, c * 64, h_idx, tile_row0, b_idx);
        tma_load_4d(smem_u32(sDO) + c * 128 * 128, &tm_do, bar_q, c * 64, h_idx, tile_row0, b_idx);
      }
      const int dcol = 64 * static_cast<int>(rank), rsub = 32 * static_cast<int>(rank);
      const int hk = h_idx / p.kv_hdiv;
      for (int i = 0; i < n; i++) {
        const int s = i % DQ2_STAGES;
        if (!mbar_wait(bar_kvempty(s), ((i / DQ2_STAGES) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const int tok0 = static_cast<int>(un.ids[i]) * G - p.kv_pad_head;
        const uint32_t base = smem_u32(sKV) + s * STAGE;
        mbar_expect_tx(bar_kvfull(s), STAGE);
        for (int c = 0; c < NCH; c++) {
          tma_load_4d(base + c * 4096, &tm_k32, bar_kvfull(s), c * 64, hk, tok0 + rsub, b_idx);
          tma_load_4d(base + OFF_VROW + c * 4096, &tm_v32, bar_kvfull(s), c * 64, hk, tok0 + rsub,
                      b_idx);
        }
        tma_load_4d(base + OFF_KCOL, &tm_k, bar_kvfull(s), dcol, hk, tok0, b_idx);
      }
    }
  } else if (warp == 1 && rank == 1) {
    // ----------------------- CTA 1: tell CTA 0 when my tiles have landed
    for (int i = 0; i < n; i++) {
      const int s = i % DQ2_STAGES;
      if (!mbar_wait(bar_kvfull(s), (i / DQ2_STAGES) & 1, w, FTK_DEV_TIMEOUT_MMA)) break;
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_peer_kv(s), 0);
    }
  } else if (warp == 1) {
    // ----------------------------- CTA 0: UMMA issuer for the CTA pair
    if (n > 0) {
      const uint32_t idesc_a = umma_idesc(256, G, FMT, 0, 0);
      const uint32_t idesc_b = umma_idesc(256, D, FMT, 0, 1);
      const uint64_t rowdesc0 = smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t coldesc0 = smem_desc_sw128(smem_u32(sKV) + OFF_KCOL, 8192, 1024);
      bool ok = mbar_wait(bar_qt, 0, w, FTK_DEV_TIMEOUT_MMA);
      auto kv_bars = [&](int i, uint32_t& b0, uint32_t& b1, uint32_t& ph) {
        const int s = i % DQ2_STAGES;
        b0 = bar_kvfull(s);
        b1 = bar_peer_kv(s);
        ph = (i / DQ2_STAGES) & 1;
      };
      auto mma_a = [&](int i) {   // elected lane only
        const int s = i % DQ2_STAGES;
        const uint64_t kdesc = desc_advance(rowdesc0, s * STAGE);
        const uint64_t vdesc = desc_advance(kdesc, OFF_VROW);
        const uint32_t sb = i & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++)
          umma2_ts(tmem + 128 + sb * 64, tmem + ks * 8,
                   desc_advance(kdesc, (ks / 4) * 4096 + (ks % 4) * 32), idesc_a, ks > 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++)
          umma2_ts(tmem + 256 + sb * 64, tmem + 64 + ks * 8,
                   desc_advance(vdesc, (ks / 4) * 4096 + (ks % 4) * 32), idesc_a, ks > 0);
        umma2_commit(bar_afull(sb), 3);
      };
      auto mma_b = [&](int i) {   // elected lane only
        const int s = i % DQ2_STAGES, sb = i & 1;
        const uint64_t kcol = desc_advance(coldesc0, s * STAGE);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
          umma2_ts(tmem + 384, tmem + 256 + sb * 64 + (ks >> 1) * 32 + (ks & 1) * 8,
                   desc_advance(kcol, ks * 2048), idesc_b, (i > 0) || (ks > 0));
        umma2_commit(bar_kvempty(s), 3);
      };
      {
        uint32_t b0, b1, ph;
        kv_bars(0, b0, b1, ph);
        const uint32_t wb[2] = {b0, b1};
        const uint32_t wp[2] = {ph, ph};
        if (ok) ok = mbar_wait_all<2>(wb, wp, w, FTK_DEV_TIMEOUT_MMA);
        if (ok && n > 1) {
          kv_bars(1, b0, b1, ph);
          const uint32_t wb1[2] = {b0, b1};
          const uint32_t wp1[2] = {ph, ph};
          ok = mbar_wait_all<2>(wb1, wp1, w, FTK_DEV_TIMEOUT_MMA);
        }
      }
      tc_fence_after();
      if (ok && elect_one()) {
        mma_a(0);
        if (n > 1) mma_a(1);
      }
      __syncwarp();
      // per round every barrier is waited for first (together), then dQ of
      // tile i and S, dP of tile i + 2 go out as one batch
      for (int i = 0; ok && i < n; i++) {
        const bool more = i + 2 < n;
        uint32_t b0 = bar_dsfull(i & 1), b1 = b0, ph = (i >> 1) & 1;
        if (more) kv_bars(i + 2, b0, b1, ph);
        const uint32_t wb[3] = {bar_dsfull(i & 1), b0, b1};
        const uint32_t wp[3] = {static_cast<uint32_t>((i >> 1) & 1), ph, ph};
        if (!mbar_wait_all<3>(wb, wp, w, FTK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        if (elect_one()) {
          mma_b(i);
          if (more) mma_a(i + 2);
        }
        __syncwarp();
      }
      if (elect_one()) umma2_commit(bar_final, 3);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // Two groups of 8 warps per CTA; group w drains the buffers of tiles
    // i = w (mod 2); two warps share each 32-row lane quarter and take one half
    // of the kv columns each.
    const int cw = warp - 2;
    const int wg = cw >> 3;
    const int colhalf = (cw >> 2) & 1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int grp = 2 * static_cast<int>(rank) + r / G;   // q-block of the pair
    const int qrow = tile_row0 + r;
    const bool row_valid = (grp < groups) && qrow >= 0 && qrow < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + 128 + wg * 64;
    const uint32_t dp_addr = lane_addr + 256 + wg * 64;
    const int cbeg = colhalf * 32;
    const float c = p.scale_log2;
    float lse2 = 0.f, dl = 0.f;
    if (row_valid) {
      lse2 = p.lse[static_cast<int64_t>(bh) * p.N + qrow] * 1.4426950408889634f;
      dl = p.delta[static_cast<int64_t>(bh) * p.N + qrow];
    }
    bool ok = true;
    if (n > 0 && colhalf == 0) {
      // group 0 moves the Q tile, group 1 the dO tile, from (swizzled) shared
      // memory into TMEM: row r -> lane r, two 16-bit values per column
      ok = mbar_wait(bar_q, 0, w, FTK_DEV_TIMEOUT_CONSUMER);
      if (ok) {
        const uint8_t* src = wg == 0 ? sQ : sDO;
#pragma unroll
        for (int ch = 0; ch < NCH; ch++) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint4 t4 = *reinterpret_cast<const uint4*>(src + ch * 128 * 128 +
                                                             sw128_offset(r, j));
            v[j * 4 + 0] = t4.x;
            v[j * 4 + 1] = t4.y;
            v[j * 4 + 2] = t4.z;
            v[j * 4 + 3] = t4.w;
          }
          tmem_st32(lane_addr + wg * 64 + ch * 32, v);
        }
        tmem_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_qt, 0);
    }
    for (int i = wg; ok && i < n; i += 2) {
      // A(i) complete also means B(i-2) has retired (same issue order), so the
      // dS columns of this buffer are free again.
      if (!mbar_wait(bar_afull(wg), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int tok0 = static_cast<int>(un.ids[i]) * G - p.kv_pad_head;
      const int lo = max(0, -tok0), hi = min(G, p.N - tok0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == G;
      uint32_t sv[32], dv[32], pk[16];
      tmem_ld32(s_addr + cbeg, sv);
      tmem_ld32(dp_addr + cbeg, dv);
      tmem_wait_ld();
      if (fast) {
        ds_pairs<FMT>(sv, dv, pk, c, -lse2, -dl);
      } else {
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          float d0 = 0.f, d1 = 0.f;
          if (act && cbeg + x >= lo && cbeg + x < hi)
            d0 = fast_exp2(fmaf(__uint_as_float(sv[x]), c, -lse2)) * (__uint_as_float(dv[x]) - dl);
          if (act && cbeg + x + 1 >= lo && cbeg + x + 1 < hi)
            d1 = fast_exp2(fmaf(__uint_as_float(sv[x + 1]), c, -lse2)) *
                 (__uint_as_float(dv[x + 1]) - dl);
          pk[x >> 1] = pack2f<FMT>(d0, d1);
        }
      }
      // dS over the dP columns this thread has read
      tmem_st16(dp_addr + cbeg, pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_dsfull(wg), 0);
    }
    // epilogue: 32-column chunks of the head dim dealt to the four warps of a
    // lane quarter
    if (ok && n > 0) ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = static_cast<uint8_t*>(p.out0) +
               2 * (static_cast<int64_t>(b_idx) * p.s0_b + static_cast<int64_t>(qrow) * p.s0_n +
                    static_cast<int64_t>(h_idx) * p.s0_h);
      const int c0 = (wg * 2 + colhalf) * 32;
      uint32_t v[32];
      if (n > 0) {
        tmem_ld32(lane_addr + 384 + c0, v);
        tmem_wait_ld();
      }
      if (row_valid) {
        uint32_t pk[16];
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float a = n > 0 ? __uint_as_float(v[x]) * p.scale : 0.f;
          const float b = n > 0 ? __uint_as_float(v[x + 1]) * p.scale : 0.f;
          pk[x >> 1] = pack2f<FMT>(a, b);
        }
        uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
        for (int x = 0; x < 4; x++)
          dst[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag)
    for (int i = 0; i < 200; i++) __nanosleep(1000);
  // neither CTA may leave (or free TMEM) while the other can still touch it
  cluster_sync_all();
  if (warp == 0) tmem_dealloc2(tmem, 512);
}

}  // namespace ftk
