// dK/dV on pairs of SMs (tcgen05 cta_group::2), for 64-row q and kv blocks and
// head dim 128.  Included by sparse_bwd.cu (shares BwdParams).
//
// Measured on B200: a UMMA of M = 128 with both operands in shared memory costs
// 75 cycles at N = 64, and the dK/dV kernel spends two thirds of its tensor
// time in such UMMAs (S^T = K Q^T, dP^T = V dO^T: K and V cannot live in TMEM
// next to four accumulators).  The same instruction issued for a CTA pair
// (M = 256: 128 rows in each CTA, the N columns of B split between the two)
// costs 43 cycles for twice the rows, and 64 at N = 128.  So a cluster of two
// CTAs owns 256 kv rows; each CTA keeps its own K / V tile, accumulators and
// compute warps exactly as in the one-CTA kernel, both walk the union of the
// four kv-blocks' reverse lists, and per q-block tile each CTA loads only
//   rows  32 r .. 32 r + 31 of Q and dO (all of d)  - its half of the B operand
//         of S^T / dP^T (N = 64 q rows split in two), and
//   d columns 64 r .. 64 r + 63 of Q and dO (all 64 rows) - its half of the B
//         operand of dK / dV (N = 128 split in two),
// 32 KB per tile as before, but for twice the kv rows.  CTA 0 issues every
// UMMA; tcgen05.commit multicasts its arrivals to both CTAs' barriers; the
// other CTA's warp 1 forwards "my tiles have landed" to CTA 0 and its compute
// warps arrive on CTA 0's barriers through the cluster shared-memory window.
// No TMA load is multicast.  With the UMMAs this cheap the compute warps set
// the pace: they use two-column instructions (fma / add / mul .f32x2), fetch
// lse / delta a round ahead, and all 16 of them work on every tile.
#pragma once

namespace ftk {

constexpr int DK2_STAGES = 4;

// TMEM columns per CTA as in the one-CTA kernel: S^T[2] 0/64 (P^T over their
// first half), dP^T[2] 128/192 (dS^T likewise), dV 256.., dK 384..
// Shared memory per CTA: K 32 KB, V 32 KB, 4 stages of
//   [Q rows-half 8 KB][dO rows-half 8 KB][Q d-half 8 KB][dO d-half 8 KB].
template <int FMT>
__device__ __forceinline__ uint32_t pack2f(float a, float b) {
  if (FMT == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BW_THREADS, 1)
sparse_bwd_dkv2_kernel(const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_q32,
                       const __grid_constant__ CUtensorMap tm_do32,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const BwdParams p) {
  constexpr int D = 128;
  constexpr int NCH = 2;
  constexpr int ROW_TILE_BYTES = NCH * 128 * 128;
  constexpr int G = 64;                       // q block = kv block = 64 rows
  constexpr int STAGE = 32768;
  constexpr int OFF_DOROW = 8192, OFF_QCOL = 16384, OFF_DOCOL = 24576;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + ROW_TILE_BYTES;
  uint8_t* sQD = smem + 2 * ROW_TILE_BYTES;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[2 + 3 * DK2_STAGES + 5];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ __align__(16) float s_lse2[2][2][128], s_delta[2][2][128];  // [group][parity][q row]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int j0 = (blockIdx.x >> 1) * 4;      // first of the pair's four kv blocks
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(4, p.Mkv - j0);     // kv blocks of the pair that exist
  const int tile_tok0 = (j0 + 2 * static_cast<int>(rank)) * G - p.kv_pad_head;   // my 128 rows

  const uint32_t bar_kv = smem_u32(&bars[0]);        // my K / V tiles
  const uint32_t bar_peer_kv = smem_u32(&bars[1]);   // CTA 0: CTA 1's K / V tiles
  auto bar_qfull = [&](int s) { return smem_u32(&bars[2 + s]); };
  auto bar_qempty = [&](int s) { return smem_u32(&bars[2 + DK2_STAGES + s]); };
  auto bar_peer_q = [&](int s) { return smem_u32(&bars[2 + 2 * DK2_STAGES + s]); };  // CTA 0 only
  constexpr int BAR_A0 = 2 + 3 * DK2_STAGES;
  auto bar_afull = [&](int s) { return smem_u32(&bars[BAR_A0 + s]); };
  auto bar_pfull = [&](int s) { return smem_u32(&bars[BAR_A0 + 2 + s]); };           // CTA 0 only
  const uint32_t bar_final = smem_u32(&bars[BAR_A0 + 4]);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_peer_kv, 1);
    for (int s = 0; s < DK2_STAGES; s++) {
      mbar_init(bar_qfull(s), 1);
      mbar_init(bar_qempty(s), 1);
      mbar_init(bar_peer_q(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_afull(s), 1);
      mbar_init(bar_pfull(s), 32);   // the 16 compute warps of each CTA
    }
    mbar_init(bar_final, 1);
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_q32);
    tma_prefetch_desc(&tm_do32);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc2(smem_u32(&tmem_base_s), 512);
    tmem_relinquish2();
  }
  // both CTAs build the same union over the pair's four reverse lists
  const int64_t kv_row = static_cast<int64_t>(bh) * p.Mkv + j0;
  const int n = build_union(un, p.lists + kv_row * p.QM, p.QM, groups, p.QM, p.counts + kv_row,
                            p.QM, p.status);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_kv, 2 * ROW_TILE_BYTES);
      for (int c = 0; c < NCH; c++) {
        tma_load_4d(smem_u32(sK) + c * 128 * 128, &tm_k, bar_kv, c * 64, h_idx / p.kv_hdiv,
                    tile_tok0, b_idx);
        tma_load_4d(smem_u32(sV) + c * 128 * 128, &tm_v, bar_kv, c * 64, h_idx / p.kv_hdiv,
                    tile_tok0, b_idx);
      }
      const int dcol = 64 * static_cast<int>(rank), rsub = 32 * static_cast<int>(rank);
      for (int i = 0; i < n; i++) {
        const int s = i % DK2_STAGES;
        if (!mbar_wait(bar_qempty(s), ((i / DK2_STAGES) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const int row0 = static_cast<int>(un.ids[i]) * G - p.q_pad_head;
        const uint32_t base = smem_u32(sQD) + s * STAGE;
        mbar_expect_tx(bar_qfull(s), STAGE);
        for (int c = 0; c < NCH; c++) {
          tma_load_4d(base + c * 4096, &tm_q32, bar_qfull(s), c * 64, h_idx, row0 + rsub, b_idx);
          tma_load_4d(base + OFF_DOROW + c * 4096, &tm_do32, bar_qfull(s), c * 64, h_idx,
                      row0 + rsub, b_idx);
        }
        tma_load_4d(base + OFF_QCOL, &tm_q, bar_qfull(s), dcol, h_idx, row0, b_idx);
        tma_load_4d(base + OFF_DOCOL, &tm_do, bar_qfull(s), dcol, h_idx, row0, b_idx);
      }
    }
  } else if (warp == 1 && rank == 1) {
    // ----------------------- CTA 1: tell CTA 0 when my tiles have landed
    if (n > 0) {
      bool ok = mbar_wait(bar_kv, 0, w, FTK_DEV_TIMEOUT_MMA);
      __syncwarp();
      if (ok && lane == 0) mbar_arrive_cta(bar_peer_kv, 0);
      for (int i = 0; ok && i < n; i++) {
        const int s = i % DK2_STAGES;
        if (!mbar_wait(bar_qfull(s), (i / DK2_STAGES) & 1, w, FTK_DEV_TIMEOUT_MMA)) break;
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(bar_peer_q(s), 0);
      }
    }
  } else if (warp == 1) {
    // ----------------------------- CTA 0: UMMA issuer for the CTA pair
    if (n > 0) {
      const uint32_t idesc_a = umma_idesc(256, G, FMT, 0, 0);
      const uint32_t idesc_b = umma_idesc(256, D, FMT, 0, 1);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t vdesc0 = smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t rowdesc0 = smem_desc_sw128(smem_u32(sQD), 16, 1024);
      const uint64_t coldesc0 = smem_desc_sw128(smem_u32(sQD) + OFF_QCOL, 8192, 1024);
      const uint32_t kvb[2] = {bar_kv, bar_peer_kv};
      const uint32_t kvp[2] = {0u, 0u};
      bool ok = mbar_wait_all<2>(kvb, kvp, w, FTK_DEV_TIMEOUT_MMA);
      auto wait_q = [&](int i) -> bool {
        const int s = i % DK2_STAGES;
        const uint32_t ph = (i / DK2_STAGES) & 1;
        const uint32_t wb[2] = {bar_qfull(s), bar_peer_q(s)};
        const uint32_t wp[2] = {ph, ph};
        return mbar_wait_all<2>(wb, wp, w, FTK_DEV_TIMEOUT_MMA);
      };
      auto mma_a = [&](int i) {   // elected lane only
        const int s = i % DK2_STAGES;
        const uint64_t qdesc = desc_advance(rowdesc0, s * STAGE);
        const uint64_t dodesc = desc_advance(qdesc, OFF_DOROW);
        const uint32_t sb = i & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          const uint32_t aoff = (ks / 4) * 128 * 128 + (ks % 4) * 32;
          const uint32_t boff = (ks / 4) * 4096 + (ks % 4) * 32;
          umma2_ss(tmem + sb * 64, desc_advance(kdesc0, aoff), desc_advance(qdesc, boff), idesc_a,
                   ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          const uint32_t aoff = (ks / 4) * 128 * 128 + (ks % 4) * 32;
          const uint32_t boff = (ks / 4) * 4096 + (ks % 4) * 32;
          umma2_ss(tmem + 128 + sb * 64, desc_advance(vdesc0, aoff), desc_advance(dodesc, boff),
                   idesc_a, ks > 0);
        }
        umma2_commit(bar_afull(sb), 3);
      };
      auto mma_b = [&](int i) {   // elected lane only
        const int s = i % DK2_STAGES, sb = i & 1;
        const uint64_t qcol = desc_advance(coldesc0, s * STAGE);
        const uint64_t docol = desc_advance(qcol, OFF_DOCOL - OFF_QCOL);
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
          const bool acc = (i > 0) || (ks > 0);
          const uint32_t col = sb * 64 + ks * 16;   // written by the warps of column quarter ks
          umma2_ts(tmem + 256, tmem + col, desc_advance(docol, ks * 2048), idesc_b, acc);
          umma2_ts(tmem + 384, tmem + 128 + col, desc_advance(qcol, ks * 2048), idesc_b, acc);
        }
        umma2_commit(bar_qempty(s), 3);
      };
      if (ok) ok = wait_q(0);
      if (ok && n > 1) ok = wait_q(1);
      tc_fence_after();
      if (ok && elect_one()) {
        mma_a(0);
        if (n > 1) mma_a(1);
      }
      __syncwarp();
      for (int i = 0; ok && i < n; i++) {
        if (!mbar_wait(bar_pfull(i & 1), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        if (elect_one()) mma_b(i);
        __syncwarp();
        if (i + 2 < n) {
          if (!wait_q(i + 2)) break;
          tc_fence_after();
          if (elect_one()) mma_a(i + 2);
          __syncwarp();
        }
      }
      if (elect_one()) umma2_commit(bar_final, 3);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // All 16 compute warps of a CTA work on every tile: four warps share each
    // 32-row lane quarter and take 16 of the 64 q columns each.  A tile's
    // exponentials then take half as long as with one 8-warp group per
    // buffer, and that time is part of the per-buffer chain
    //   S^T, dP^T ready -> P^T, dS^T -> dV, dK -> next S^T, dP^T
    // that bounds the kernel; the two buffers still overlap each other.
    const int cw = warp - 2;
    const int colq = cw >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int ct = tid - 64;                 // index among the compute threads
    const int grp = 2 * static_cast<int>(rank) + r / G;   // kv block of the pair
    const int tok = tile_tok0 + r;
    const bool row_valid = (grp < groups) && tok >= 0 && tok < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const int cbeg = colq * 16;
    const float c = p.scale_log2;
    bool ok = true;
    // lse / delta of a q-block are fetched from global memory one round ahead
    // (into registers, while the previous tile is being worked on) and only
    // then staged in shared memory: their latency stays out of the chain.
    auto fetch = [&](int i, float& l2, float& dl) {
      l2 = 0.f;
      dl = 0.f;
      if (ct < G && i < n) {
        const int t = static_cast<int>(un.ids[i]) * G - p.q_pad_head + ct;
        if (t >= 0 && t < p.N) {   // stored negated: the packed fma / add take them as they are
          l2 = -p.lse[static_cast<int64_t>(bh) * p.N + t] * 1.4426950408889634f;
          dl = -p.delta[static_cast<int64_t>(bh) * p.N + t];
        }
      }
    };
    float l2_next, dl_next;
    fetch(0, l2_next, dl_next);
    for (int i = 0; i < n; i++) {
      const int sb = i & 1;                  // S^T / dP^T buffer, and lse / delta buffer
      const int row0 = static_cast<int>(un.ids[i]) * G - p.q_pad_head;
      if (ct < G) {
        s_lse2[0][sb][ct] = l2_next;
        s_delta[0][sb][ct] = dl_next;
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      fetch(i + 1, l2_next, dl_next);
      if (!ok) continue;
      if (!mbar_wait(bar_afull(sb), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        continue;
      }
      tc_fence_after();
      const uint32_t st_addr = lane_addr + sb * 64;         // S^T, then P^T
      const uint32_t dp_addr = lane_addr + 128 + sb * 64;   // dP^T, then dS^T
      const int lo = max(0, -row0), hi = min(G, p.N - row0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == G;
      const float4* l4 = reinterpret_cast<const float4*>(s_lse2[0][sb]);
      const float4* d4 = reinterpret_cast<const float4*>(s_delta[0][sb]);
      // P^T / dS^T of the thread's 16 columns go over the first 8 of them in
      // the S^T / dP^T regions: columns this thread has already read.
      // full tiles: two columns per instruction (fma.f32x2, add.f32x2,
      // mul.f32x2, one cvt per pair); lse / delta come negated from shared
      // memory as one 16-byte broadcast load per four columns
      auto work = [&](const uint32_t (&sv)[16], const uint32_t (&dv)[16], int c0) {
        uint32_t pp[8], pd[8];
        const float2 c2 = make_float2(c, c);
        if (fast) {
#pragma unroll
          for (int x = 0; x < 16; x += 4) {
            const float4 lq = l4[(c0 + x) >> 2];
            const float4 dq = d4[(c0 + x) >> 2];
#pragma unroll
            for (int y = 0; y < 4; y += 2) {
              const float2 nl = y == 0 ? make_float2(lq.x, lq.y) : make_float2(lq.z, lq.w);
              const float2 nd = y == 0 ? make_float2(dq.x, dq.y) : make_float2(dq.z, dq.w);
              const float2 t = __ffma2_rn(
                  make_float2(__uint_as_float(sv[x + y]), __uint_as_float(sv[x + y + 1])), c2, nl);
              const float2 pr = make_float2(fast_exp2(t.x), fast_exp2(t.y));
              const float2 dd = __fadd2_rn(
                  make_float2(__uint_as_float(dv[x + y]), __uint_as_float(dv[x + y + 1])), nd);
              const float2 dsv = __fmul2_rn(pr, dd);
              pp[(x + y) >> 1] = pack2f<FMT>(pr.x, pr.y);
              pd[(x + y) >> 1] = pack2f<FMT>(dsv.x, dsv.y);
            }
          }
        } else {
#pragma unroll
          for (int x = 0; x < 16; x += 4) {
            const float4 lq = l4[(c0 + x) >> 2];
            const float4 dq = d4[(c0 + x) >> 2];
            const float ls[4] = {lq.x, lq.y, lq.z, lq.w};
            const float ds[4] = {dq.x, dq.y, dq.z, dq.w};
            float pv[4], dsv[4];
#pragma unroll
            for (int y = 0; y < 4; y++) {
              const bool on = act && c0 + x + y >= lo && c0 + x + y < hi;
              const float pr = on ? fast_exp2(fmaf(__uint_as_float(sv[x + y]), c, ls[y])) : 0.f;
              pv[y] = pr;
              dsv[y] = pr * (__uint_as_float(dv[x + y]) + ds[y]);
            }
            pp[x >> 1] = pack2f<FMT>(pv[0], pv[1]);
            pp[(x >> 1) + 1] = pack2f<FMT>(pv[2], pv[3]);
            pd[x >> 1] = pack2f<FMT>(dsv[0], dsv[1]);
            pd[(x >> 1) + 1] = pack2f<FMT>(dsv[2], dsv[3]);
          }
        }
        tmem_st8(st_addr + c0, pp);
        tmem_st8(dp_addr + c0, pd);
      };
      {
        uint32_t sa[16], da[16];
        tmem_ld16(st_addr + cbeg, sa);
        tmem_ld16(dp_addr + cbeg, da);
        tmem_wait_ld();
        work(sa, da, cbeg);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_pfull(sb), 0);
    }
    if (ok && n > 0) ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      // column quarters 0, 1 store dV (TMEM 256..), 2, 3 store dK (TMEM 384.., scaled)
      const int which = colq >> 1, colhalf = colq & 1;
      uint8_t* base = static_cast<uint8_t*>(which == 0 ? p.out1 : p.out0);
      const int64_t sb_ = which == 0 ? p.s1_b : p.s0_b, sn_ = which == 0 ? p.s1_n : p.s0_n,
                    sh_ = which == 0 ? p.s1_h : p.s0_h;
      const float mul = which == 0 ? 1.f : p.scale;
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = base + 2 * (static_cast<int64_t>(b_idx) * sb_ + static_cast<int64_t>(tok) * sn_ +
                           static_cast<int64_t>(h_idx) * sh_);
      for (int c0 = colhalf * 32; c0 < D; c0 += 64) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld32(lane_addr + 256 + which * 128 + c0, v);
          tmem_wait_ld();
        }
        if (row_valid) {
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float a = n > 0 ? __uint_as_float(v[x]) * mul : 0.f;
            const float b = n > 0 ? __uint_as_float(v[x + 1]) * mul : 0.f;
            pk[x >> 1] = pack2f<FMT>(a, b);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
          for (int x = 0; x < 4; x++)
            dst[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
        }
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
