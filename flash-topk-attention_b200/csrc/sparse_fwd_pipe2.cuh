// The pipelined forward kernel (sparse_fwd_pipe.cuh) on pairs of SMs (tcgen05
// cta_group::2), head dim 128.  Included by sparse_fwd.cu after it.
//
// A cluster of two CTAs owns 256 query rows (four q-blocks).  Each CTA keeps its
// own 128 rows of Q in TMEM, its own four S / P buffers, O accumulator and
// softmax warps, exactly as in the one-CTA kernel; both walk the union of the
// four q-blocks' candidate lists (and the up to four prologue blocks that give
// the rows their reference exponents).  Per kv block each CTA loads only
//   kv rows 32 r .. 32 r + 31 of K (all of d)    - its half of the B operand of
//        S = Q K^T (N = 64 kv rows split in two), and
//   d columns 64 r .. 64 r + 63 of V (all 64 rows) - its half of the B operand
//        of O += P V (N = 128 split in two),
// 16 KB per tile for twice the query rows (the one-CTA kernel loads 32 KB and
// is co-limited by the L2 -> SM path), and the M = 256 UMMAs cost 43 cycles at
// N = 64 and 64 at N = 128 for both CTAs together.  CTA 0 issues every UMMA;
// tcgen05.commit multicasts its arrivals; CTA 1's warp 1 forwards "my tiles
// have landed"; softmax warps of CTA 1 arrive on CTA 0's barriers through the
// cluster shared-memory window.  No TMA load is multicast.
#pragma once

namespace ftk {

constexpr int FP2_KST = 6;   // K half tiles (8 KB) in the ring
constexpr int FP2_VST = 8;   // V half tiles (8 KB) in the ring

template <int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FP_THREADS, 1)
sparse_fwd_pipe2_kernel(const __grid_constant__ CUtensorMap tm_q,
                        const __grid_constant__ CUtensorMap tm_k32,
                        const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  constexpr int D = 128;
  constexpr int NCH = D / 64;
  constexpr int Q_BYTES = NCH * 128 * 128;
  constexpr int KVB = 64;
  constexpr int TILE = 8192;                   // half a K tile (32 rows x 128 d) or half a V tile
                                               // (64 rows x 64 d)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Q_BYTES;
  uint8_t* sV = sK + FP2_KST * TILE;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[4 + 3 * FP2_KST + 3 * FP2_VST + 2 * FP_GROUPS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ int s_ovf;
  __shared__ int s_first[4];
  __shared__ float s_l[FP_GROUPS][128];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const int m0 = (blockIdx.x >> 1) * 4;       // first of the pair's four q-blocks
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(4, p.QM - m0);
  const int tile_row0 = (m0 + 2 * static_cast<int>(rank)) * 64 - p.q_pad_head;   // my 128 rows

  const uint32_t bar_q = smem_u32(&bars[0]);
  const uint32_t bar_final = smem_u32(&bars[1]);
  const uint32_t bar_qt = smem_u32(&bars[2]);    // CTA 0: Q of both CTAs copied into TMEM
  const uint32_t bar_pro = smem_u32(&bars[3]);   // CTA 0: every softmax warp has its reference
  auto bar_kfull = [&](int s) { return smem_u32(&bars[4 + s]); };
  auto bar_kempty = [&](int s) { return smem_u32(&bars[4 + FP2_KST + s]); };
  auto bar_peer_k = [&](int s) { return smem_u32(&bars[4 + 2 * FP2_KST + s]); };   // CTA 0 only
  constexpr int BAR_V0 = 4 + 3 * FP2_KST;
  auto bar_vfull = [&](int s) { return smem_u32(&bars[BAR_V0 + s]); };
  auto bar_vempty = [&](int s) { return smem_u32(&bars[BAR_V0 + FP2_VST + s]); };
  auto bar_peer_v = [&](int s) { return smem_u32(&bars[BAR_V0 + 2 * FP2_VST + s]); };   // CTA 0 only
  constexpr int BAR_S0 = 4 + 3 * FP2_KST + 3 * FP2_VST;
  auto bar_sfull = [&](int b) { return smem_u32(&bars[BAR_S0 + b]); };
  auto bar_pfull = [&](int b) { return smem_u32(&bars[BAR_S0 + FP_GROUPS + b]); };

  if (tid == 0) {
    abort_flag = 0;
    s_ovf = 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_final, 1);
    mbar_init(bar_qt, 8);                  // the 4 copying warps of each CTA
    mbar_init(bar_pro, 8 * FP_GROUPS);     // the 16 softmax warps of each CTA
    for (int s = 0; s < FP2_KST; s++) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
      mbar_init(bar_peer_k(s), 1);
    }
    for (int s = 0; s < FP2_VST; s++) {
      mbar_init(bar_vfull(s), 1);
      mbar_init(bar_vempty(s), 1);
      mbar_init(bar_peer_v(s), 1);
    }
    for (int b = 0; b < FP_GROUPS; b++) {
      mbar_init(bar_sfull(b), 1);
      mbar_init(bar_pfull(b), 8);          // the group's 4 warps in each CTA
    }
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k32);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc2(smem_u32(&tmem_base_s), 512);
    tmem_relinquish2();
  }
  const int n = build_union(un, p.merged + (static_cast<int64_t>(bh) * p.QM + m0) * p.W, p.W,
                            groups, p.W, nullptr, p.Mkv, p.status);
  // lowest listed block of each q-block: its scores give the rows' reference
  if (warp < 4) {
    int best = 0x7fffffff;
    if (warp < groups) {
#pragma unroll
      for (int q = 0; q < AT_WORDS / 32; q++) {
        const unsigned wv = un.bm[warp][q * 32 + lane];
        if (wv && best == 0x7fffffff) best = (q * 32 + lane) * 32 + __ffs(wv) - 1;
      }
    }
    best = __reduce_min_sync(0xffffffffu, best);
    if (lane == 0) s_first[warp] = (best == 0x7fffffff) ? -1 : best;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};

  // prologue entries: one per q-block of the pair with a non-empty list (the
  // same in both CTAs); entry e goes through S buffer e
  int npro = 0;
  int pro_id[4] = {0, 0, 0, 0};
  int pro_buf[4] = {-1, -1, -1, -1};
#pragma unroll
  for (int g = 0; g < 4; g++) {
    if (g < groups && s_first[g] >= 0) {
#pragma unroll
      for (int e = 0; e < 4; e++)
        if (e == npro) pro_id[e] = s_first[g];
      pro_buf[g] = npro;
      npro++;
    }
  }
  auto pro_block = [&](int e) {
    return e == 0 ? pro_id[0] : e == 1 ? pro_id[1] : e == 2 ? pro_id[2] : pro_id[3];
  };

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_q, Q_BYTES);
      for (int c = 0; c < NCH; c++)
        tma_load_4d(smem_u32(sQ) + c * 128 * 128, &tm_q, bar_q, c * 64, h_idx, tile_row0, b_idx);
      // K entry j: the prologue blocks first, then the union; V entry i: the
      // union only.  Every wait depends on tiles loaded earlier only.
      const int total = npro + n;
      const int dcol = 64 * static_cast<int>(rank), rsub = 32 * static_cast<int>(rank);
      for (int j = 0; j < total; j++) {
        const int sk = j % FP2_KST;
        if (!mbar_wait(bar_kempty(sk), ((j / FP2_KST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const bool pro = j < npro;
        const int id = pro ? pro_block(j) : static_cast<int>(un.ids[j - npro]);
        const int tok0 = id * KVB - p.kv_pad_head;
        const uint32_t kb = smem_u32(sK) + sk * TILE;
        mbar_expect_tx(bar_kfull(sk), TILE);
        for (int c = 0; c < NCH; c++)
          tma_load_4d(kb + c * 4096, &tm_k32, bar_kfull(sk), c * 64, h_idx / p.kv_hdiv,
                      tok0 + rsub, b_idx);
        if (!pro) {
          const int i = j - npro, sv = i % FP2_VST;
          if (!mbar_wait(bar_vempty(sv), ((i / FP2_VST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
          mbar_expect_tx(bar_vfull(sv), TILE);
          tma_load_4d(smem_u32(sV) + sv * TILE, &tm_v, bar_vfull(sv), dcol, h_idx / p.kv_hdiv,
                      tok0, b_idx);
        }
      }
    }
  } else if (warp == 1 && rank == 1) {
    // ----------------------- CTA 1: tell CTA 0 when my tiles have landed
    const int total = npro + n;
    for (int j = 0; n > 0 && j < total; j++) {
      const int sk = j % FP2_KST;
      if (!mbar_wait(bar_kfull(sk), (j / FP2_KST) & 1, w, FTK_DEV_TIMEOUT_MMA)) break;
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_peer_k(sk), 0);
      if (j >= npro) {
        const int i = j - npro, sv = i % FP2_VST;
        if (!mbar_wait(bar_vfull(sv), (i / FP2_VST) & 1, w, FTK_DEV_TIMEOUT_MMA)) break;
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(bar_peer_v(sv), 0);
      }
    }
  } else if (warp == 1) {
    // ----------------------------- CTA 0: UMMA issuer for the CTA pair
    if (n > 0) {
      const uint32_t idesc_s = umma_idesc(256, KVB, FMT, 0, 0);
      const uint32_t idesc_pv = umma_idesc(256, D, FMT, 0, 1);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t vdesc0 = smem_desc_sw128(smem_u32(sV), 8192, 1024);
      bool ok = mbar_wait(bar_qt, 0, w, FTK_DEV_TIMEOUT_MMA);
      tc_fence_after();
      auto wait_k = [&](int j) -> bool {
        const int s = j % FP2_KST;
        const uint32_t ph = (j / FP2_KST) & 1;
        const uint32_t wb[2] = {bar_kfull(s), bar_peer_k(s)};
        const uint32_t wp[2] = {ph, ph};
        return mbar_wait_all<2>(wb, wp, w, FTK_DEV_TIMEOUT_MMA);
      };
      // S = Q K^T for K entry j into S buffer `buf`; Q read from TMEM (elected lane only)
      auto mma_s = [&](int j, int buf) {
        const int s = j % FP2_KST;
        const uint64_t kdesc = desc_advance(kdesc0, s * TILE);
        const uint32_t d_tmem = tmem + FP_COL_S + buf * 64;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++)
          umma2_ts(d_tmem, tmem + ks * 8, desc_advance(kdesc, (ks / 4) * 4096 + (ks % 4) * 32),
                   idesc_s, ks > 0);
        umma2_commit(bar_sfull(buf), 3);
        umma2_commit(bar_kempty(s), 3);
      };
      for (int e = 0; ok && e < npro; e++) ok = wait_k(e);
      tc_fence_after();
      if (ok && elect_one())
        for (int e = 0; e < npro; e++) mma_s(e, e);
      __syncwarp();
      if (ok) ok = mbar_wait(bar_pro, 0, w, FTK_DEV_TIMEOUT_MMA);
      for (int i = 0; ok && i < FP_GROUPS && i < n; i++) ok = wait_k(npro + i);
      tc_fence_after();
      if (ok && elect_one())
        for (int i = 0; i < FP_GROUPS && i < n; i++) mma_s(npro + i, i);
      __syncwarp();
      // per round every barrier is waited for first (together), then P V of
      // tile i and S of tile i + 4 go out as one batch
      for (int i = 0; ok && i < n; i++) {
        const int j = npro + i;
        const int s = i % FP2_VST, sb = i & (FP_GROUPS - 1);
        const bool more = i + FP_GROUPS < n;
        const int j4 = j + FP_GROUPS;
        const uint32_t pf = bar_pfull(sb), pfp = (i / FP_GROUPS) & 1;
        const uint32_t vph = (i / FP2_VST) & 1, kph = (j4 / FP2_KST) & 1;
        const uint32_t wb[5] = {bar_vfull(s), bar_peer_v(s), pf,
                                more ? bar_kfull(j4 % FP2_KST) : pf,
                                more ? bar_peer_k(j4 % FP2_KST) : pf};
        const uint32_t wp[5] = {vph, vph, pfp, more ? kph : pfp, more ? kph : pfp};
        if (!mbar_wait_all<5>(wb, wp, w, FTK_DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t vdesc = desc_advance(vdesc0, s * TILE);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < KVB / 16; ks++)
            umma2_ts(tmem + FP_COL_O, tmem + FP_COL_S + sb * 64 + ks * 8,
                     desc_advance(vdesc, ks * 2048), idesc_pv, (i > 0) || (ks > 0));
          umma2_commit(bar_vempty(s), 3);
          // S(i+4) lands on the columns PV(i) reads P from; UMMAs run in issue order
          if (more) mma_s(j4, sb);
        }
        __syncwarp();
      }
      if (elect_one()) umma2_commit(bar_final, 3);
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------- softmax threads
    const int gw = (warp - 2) >> 2;          // softmax group = S buffer it drains
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int grp = 2 * static_cast<int>(rank) + r / 64;   // q-block of the pair (warp-uniform)
    const int qrow = tile_row0 + r;
    const bool row_valid = (grp < groups) && qrow >= 0 && qrow < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + FP_COL_S + gw * 64;
    const float c = p.scale_log2;
    float mref = 0.f, l = 0.f;
    bool ok = true, ovf = false;

    if (n > 0 && gw == 0) {
      // group 0 moves the Q tile from (swizzled) shared memory into TMEM
      ok = mbar_wait(bar_q, 0, w, FTK_DEV_TIMEOUT_CONSUMER);
      if (ok) {
#pragma unroll
        for (int ch = 0; ch < NCH; ch++) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const uint4 t4 =
                *reinterpret_cast<const uint4*>(sQ + ch * 128 * 128 + sw128_offset(r, j));
            v[j * 4 + 0] = t4.x;
            v[j * 4 + 1] = t4.y;
            v[j * 4 + 2] = t4.z;
            v[j * 4 + 3] = t4.w;
          }
          tmem_st32(lane_addr + ch * 32, v);
        }
        tmem_wait_st();
        tc_fence_before();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_qt, 0);
    }

    if (n > 0) {
      // ---- reference exponent: scaled row maximum over the q-block's first block
      // Every warp waits for every prologue buffer, also the ones it does not
      // read: its later parity waits on those buffers must not start while
      // their first phase is still open.
      const int pb = grp == 0 ? pro_buf[0] : grp == 1 ? pro_buf[1] : grp == 2 ? pro_buf[2]
                                                                               : pro_buf[3];
      for (int e = 0; ok && e < npro; e++)
        ok = mbar_wait(bar_sfull(e), 0, w, FTK_DEV_TIMEOUT_CONSUMER);
      if (ok && pb >= 0) {
        {
          tc_fence_after();
          const int tok0 = pro_block(pb) * KVB - p.kv_pad_head;
          const int lo = max(0, -tok0), hi = min(KVB, p.N - tok0);
          uint32_t v0[32], v1[32];
          tmem_ld32(lane_addr + FP_COL_S + pb * 64, v0);
          tmem_ld32(lane_addr + FP_COL_S + pb * 64 + 32, v1);
          tmem_wait_ld();
          float mx = -INFINITY;
#pragma unroll
          for (int x = 0; x < 32; x++) {
            if (x >= lo && x < hi) mx = fmaxf(mx, __uint_as_float(v0[x]));
            if (x + 32 >= lo && x + 32 < hi) mx = fmaxf(mx, __uint_as_float(v1[x]));
          }
          mref = (mx > -INFINITY) ? mx * c : 0.f;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_pro, 0);
    }

    const float2 c2 = make_float2(c, c);
    const float2 nm = make_float2(-mref, -mref);
    for (int i = gw; ok && i < n; i += FP_GROUPS) {
      // S(i) complete also means PV(i-4) has retired: the P columns are free
      const int u = (gw < npro ? 1 : 0) + (i / FP_GROUPS);
      if (!mbar_wait(bar_sfull(gw), u & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int tok0 = static_cast<int>(un.ids[i]) * KVB - p.kv_pad_head;
      const int lo = max(0, -tok0), hi = min(KVB, p.N - tok0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool any_act = __any_sync(0xffffffffu, act);
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == KVB;

      if (any_act) {
        uint32_t v0[32], v1[32];
        tmem_ld32(s_addr, v0);
        tmem_ld32(s_addr + 32, v1);
        tmem_wait_ld();
        uint32_t pk[16];
        float2 acc = make_float2(0.f, 0.f);
        if (fast) {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float2 t = __ffma2_rn(
                make_float2(__uint_as_float(v0[x]), __uint_as_float(v0[x + 1])), c2, nm);
            const float2 e = make_float2(fast_exp2(t.x), fast_exp2(t.y));
            acc = __fadd2_rn(acc, e);
            pk[x >> 1] = pack16<FMT>(e.x, e.y);
          }
          tmem_st16(s_addr, pk);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float2 t = __ffma2_rn(
                make_float2(__uint_as_float(v1[x]), __uint_as_float(v1[x + 1])), c2, nm);
            const float2 e = make_float2(fast_exp2(t.x), fast_exp2(t.y));
            acc = __fadd2_rn(acc, e);
            pk[x >> 1] = pack16<FMT>(e.x, e.y);
          }
          tmem_st16(s_addr + 16, pk);
        } else {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float a0 = 0.f, a1 = 0.f;
            if (act && x >= lo && x < hi) a0 = fast_exp2(fmaf(__uint_as_float(v0[x]), c, -mref));
            if (act && x + 1 >= lo && x + 1 < hi)
              a1 = fast_exp2(fmaf(__uint_as_float(v0[x + 1]), c, -mref));
            acc.x += a0;
            acc.y += a1;
            pk[x >> 1] = pack16<FMT>(a0, a1);
          }
          tmem_st16(s_addr, pk);
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float b0 = 0.f, b1 = 0.f;
            if (act && x + 32 >= lo && x + 32 < hi)
              b0 = fast_exp2(fmaf(__uint_as_float(v1[x]), c, -mref));
            if (act && x + 33 >= lo && x + 33 < hi)
              b1 = fast_exp2(fmaf(__uint_as_float(v1[x + 1]), c, -mref));
            acc.x += b0;
            acc.y += b1;
            pk[x >> 1] = pack16<FMT>(b0, b1);
          }
          tmem_st16(s_addr + 16, pk);
        }
        const float lt = acc.x + acc.y;
        if (!(lt <= fp_overflow_bound<FMT>())) ovf = true;   // also catches NaN
        l += lt;
      } else {
        uint32_t z[16];
#pragma unroll
        for (int x = 0; x < 16; x++) z[x] = 0u;
        tmem_st16(s_addr, z);
        tmem_st16(s_addr + 16, z);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(bar_pfull(gw), 0);
    }

    // ------------------------------------------------------------ epilogue
    // row sums of the four groups add up (same reference); each group converts
    // and stores a quarter of the head dimension
    s_l[gw][r] = l;
    if (ovf) atomicOr(&s_ovf, 1);
    asm volatile("bar.sync 1, 512;" ::: "memory");
    if (ok && n > 0) ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      const float lt = ((s_l[0][r] + s_l[1][r]) + s_l[2][r]) + s_l[3][r];
      const bool have = (n > 0) && lt > 0.f;
      const float inv = have ? 1.f / lt : 0.f;
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = static_cast<uint8_t*>(p.o) +
               2 * (static_cast<int64_t>(b_idx) * p.so_b + static_cast<int64_t>(qrow) * p.so_n +
                    static_cast<int64_t>(h_idx) * p.so_h);
      constexpr int QUART = D / 4;   // 32 columns per group
      const int c0 = gw * QUART;
      uint32_t ov[QUART];
      if (n > 0) {
        tmem_ld32(lane_addr + FP_COL_O + c0, ov);
        tmem_wait_ld();
      }
      if (row_valid) {
        uint32_t pk[QUART / 2];
#pragma unroll
        for (int x = 0; x < QUART; x += 2) {
          const float a = have ? __uint_as_float(ov[x]) * inv : 0.f;
          const float b = have ? __uint_as_float(ov[x + 1]) * inv : 0.f;
          pk[x >> 1] = pack16<FMT>(a, b);
        }
        uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
        for (int x = 0; x < QUART / 8; x++)
          dst[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
      }
      if (row_valid && gw == 0)
        p.lse[static_cast<int64_t>(bh) * p.N + qrow] =
            have ? (mref + log2f(lt)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  // the exact kernel redoes 128-row tiles: this CTA's rows are its tile 2 * pair + rank
  const int units_x = (p.QM + 1) / 2;
  const int unit_x = static_cast<int>(blockIdx.x >> 1) * 2 + static_cast<int>(rank);
  if (tid == 0 && p.redo_out && unit_x < units_x)
    p.redo_out[blockIdx.y * units_x + unit_x] = s_ovf;
  if (abort_flag)
    for (int i = 0; i < 200; i++) __nanosleep(1000);
  // neither CTA may leave (or free TMEM) while the other can still touch it
  cluster_sync_all();
  if (warp == 0) tmem_dealloc2(tmem, 512);
}

}  // namespace ftk
