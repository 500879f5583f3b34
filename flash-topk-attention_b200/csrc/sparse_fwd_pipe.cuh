// Deeply pipelined forward kernel for 64-row kv blocks and q-blocks of 64 or 32
// rows.  Included by sparse_fwd.cu (shares FwdParams).
//
// The exact kernel keeps a running maximum per softmax group, which ties every
// P tile to its group's accumulator: two groups, two O accumulators, two S
// buffers are all that fit in TMEM, and with two tiles in flight the tensor
// core idles while a group does its exponentials.  Here every row uses ONE
// fixed reference exponent for the whole list: the scaled maximum of the first
// kv block its q-block lists (a short prologue computes it).  P = 2^(c S - ref)
// then needs no rescaling, all tiles add into a single O accumulator, and four
// softmax groups work on four S buffers at once:
//   TMEM columns  Q 0..63 | S/P buffers 64,128,192,256 | O 320..447
// bf16 and fp32 share the exponent range, so a later block may exceed the
// reference by up to 2^80 before anything overflows (fp16: 2^15, P must stay
// below 65504); a row whose tile sum
// passes that bound marks its CTA's word in `redo_out`, and the exact kernel,
// launched behind this one, recomputes exactly those CTAs (all others return
// on their first instruction).
#pragma once

namespace ftk {

constexpr int FP_THREADS = 576;  // TMA warp, UMMA warp, 4 softmax groups x 4 warps
constexpr int FP_GROUPS = 4;
constexpr int FP_KST = 4;         // K tiles in the ring (free again once S is computed)
constexpr int FP_VST = 6;         // V tiles in the ring (held until P V has run)
constexpr int FP_COL_S = 64;
constexpr int FP_COL_O = 320;
// A tile's row sum of P above this marks the CTA for the exact kernel: 2^80 for
// bf16 (fp32 exponent range), 2^15 for fp16 (P itself must stay below 65504).
template <int FMT>
__device__ __forceinline__ float fp_overflow_bound() {
  return FMT == 1 ? 1.2089258196146292e24f : 32768.f;
}

template <int FMT>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
  if (FMT == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int FMT>
__global__ void __launch_bounds__(FP_THREADS, 1)
sparse_fwd_pipe_kernel(const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int Q_BYTES = NCH * 128 * 128;
  constexpr int KVB = 64;
  constexpr int CHUNK = KVB * 128;             // one 64-wide chunk of a K or V tile
  constexpr int TILE = NCH * CHUNK;            // one K or V tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Q_BYTES;
  uint8_t* sV = sK + FP_KST * TILE;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[4 + 2 * FP_KST + 2 * FP_VST + 2 * FP_GROUPS];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ int s_ovf;
  __shared__ int s_first[4];
  __shared__ float s_l[FP_GROUPS][128];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * p.G;
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(p.G, p.QM - m0);
  const int tile_row0 = m0 * p.g - p.q_pad_head;

  const uint32_t bar_q = smem_u32(&bars[0]);
  const uint32_t bar_final = smem_u32(&bars[1]);
  const uint32_t bar_qt = smem_u32(&bars[2]);    // Q copied into TMEM
  const uint32_t bar_pro = smem_u32(&bars[3]);   // every softmax warp has its reference
  auto bar_kfull = [&](int s) { return smem_u32(&bars[4 + s]); };
  auto bar_kempty = [&](int s) { return smem_u32(&bars[4 + FP_KST + s]); };
  auto bar_vfull = [&](int s) { return smem_u32(&bars[4 + 2 * FP_KST + s]); };
  auto bar_vempty = [&](int s) { return smem_u32(&bars[4 + 2 * FP_KST + FP_VST + s]); };
  constexpr int BAR_S0 = 4 + 2 * FP_KST + 2 * FP_VST;
  auto bar_sfull = [&](int b) { return smem_u32(&bars[BAR_S0 + b]); };
  auto bar_pfull = [&](int b) { return smem_u32(&bars[BAR_S0 + FP_GROUPS + b]); };

  if (tid == 0) {
    abort_flag = 0;
    s_ovf = 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_final, 1);
    mbar_init(bar_qt, 4);
    mbar_init(bar_pro, 4 * FP_GROUPS);
    for (int s = 0; s < FP_KST; s++) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
    }
    for (int s = 0; s < FP_VST; s++) {
      mbar_init(bar_vfull(s), 1);
      mbar_init(bar_vempty(s), 1);
    }
    for (int b = 0; b < FP_GROUPS; b++) {
      mbar_init(bar_sfull(b), 1);
      mbar_init(bar_pfull(b), 4);
    }
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
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
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};

  // prologue entries: one per q-block of the tile (two of 64 rows or four of
  // 32) with a non-empty list; entry e goes through S buffer e
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
      for (int j = 0; j < total; j++) {
        const int sk = j % FP_KST;
        if (!mbar_wait(bar_kempty(sk), ((j / FP_KST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const bool pro = j < npro;
        const int id = pro ? pro_block(j) : static_cast<int>(un.ids[j - npro]);
        const int tok0 = id * KVB - p.kv_pad_head;
        const uint32_t kb = smem_u32(sK) + sk * TILE;
        mbar_expect_tx(bar_kfull(sk), TILE);
        for (int c = 0; c < NCH; c++)
          tma_load_4d(kb + c * CHUNK, &tm_k, bar_kfull(sk), c * 64, h_idx / p.kv_hdiv, tok0, b_idx);
        if (!pro) {
          const int i = j - npro, sv = i % FP_VST;
          if (!mbar_wait(bar_vempty(sv), ((i / FP_VST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
          const uint32_t vb = smem_u32(sV) + sv * TILE;
          mbar_expect_tx(bar_vfull(sv), TILE);
          for (int c = 0; c < NCH; c++)
            tma_load_4d(vb + c * CHUNK, &tm_v, bar_vfull(sv), c * 64, h_idx / p.kv_hdiv, tok0,
                        b_idx);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- UMMA issuer
    if (n > 0) {
      const uint32_t idesc_s = umma_idesc(128, KVB, FMT, 0, 0);
      const uint32_t idesc_pv = umma_idesc(128, D, FMT, 0, 1);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t vdesc0 = smem_desc_sw128(smem_u32(sV), CHUNK, 1024);
      bool ok = mbar_wait(bar_qt, 0, w, FTK_DEV_TIMEOUT_MMA);
      tc_fence_after();
      // The tensor core runs dry whenever the issuing thread waits, so every
      // barrier of a round is waited for first and the round's UMMAs (P V of
      // tile i, then S of tile i + 4) go out as one uninterrupted batch.
      auto wait_k = [&](int j) -> bool {
        return mbar_wait(bar_kfull(j % FP_KST), (j / FP_KST) & 1, w, FTK_DEV_TIMEOUT_MMA);
      };
      // S = Q K^T for K entry j into S buffer `buf`; Q read from TMEM (elected lane only)
      auto mma_s = [&](int j, int buf) {
        const int s = j % FP_KST;
        const uint64_t kdesc = desc_advance(kdesc0, s * TILE);
        const uint32_t d_tmem = tmem + FP_COL_S + buf * 64;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++)
          umma_ts(d_tmem, tmem + ks * 8, desc_advance(kdesc, (ks / 4) * CHUNK + (ks % 4) * 32),
                  idesc_s, ks > 0);
        umma_commit(bar_sfull(buf));
        umma_commit(bar_kempty(s));
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
      for (int i = 0; ok && i < n; i++) {
        const int j = npro + i;
        const int s = i % FP_VST, sb = i & (FP_GROUPS - 1);
        const bool more = i + FP_GROUPS < n;
        const int j4 = j + FP_GROUPS;
        const uint32_t wb[3] = {bar_vfull(s), bar_pfull(sb),
                                more ? bar_kfull(j4 % FP_KST) : bar_pfull(sb)};
        const uint32_t wp[3] = {static_cast<uint32_t>((i / FP_VST) & 1),
                                static_cast<uint32_t>((i / FP_GROUPS) & 1),
                                static_cast<uint32_t>(more ? (j4 / FP_KST) & 1
                                                           : (i / FP_GROUPS) & 1)};
        if (!mbar_wait_all<3>(wb, wp, w, FTK_DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t vdesc = desc_advance(vdesc0, s * TILE);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < KVB / 16; ks++)
            umma_ts(tmem + FP_COL_O, tmem + FP_COL_S + sb * 64 + ks * 8,
                    desc_advance(vdesc, ks * 2048), idesc_pv, (i > 0) || (ks > 0));
          umma_commit(bar_vempty(s));
          // S(i+4) lands on the columns PV(i) reads P from; UMMAs run in issue order
          if (i + FP_GROUPS < n) mma_s(j + FP_GROUPS, sb);
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(bar_final);
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------- softmax threads
    const int gw = (warp - 2) >> 2;          // softmax group = S buffer it drains
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int grp = r / p.g;                 // warp-uniform: q-blocks are 64 or 32 rows
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
      if (lane == 0) mbar_arrive(bar_qt);
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
      if (lane == 0) mbar_arrive(bar_pro);
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
      if (lane == 0) mbar_arrive(bar_pfull(gw));
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
      constexpr int QUART = D / 4;   // 32 or 16 columns per group
      const int c0 = gw * QUART;
      uint32_t ov[QUART];
      if (n > 0) {
        if constexpr (QUART == 32) tmem_ld32(lane_addr + FP_COL_O + c0, ov);
        else tmem_ld16(lane_addr + FP_COL_O + c0, ov);
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
  if (tid == 0 && p.redo_out) p.redo_out[blockIdx.y * gridDim.x + blockIdx.x] = s_ovf;
  if (abort_flag)
    for (int i = 0; i < 200; i++) __nanosleep(1000);
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace ftk
