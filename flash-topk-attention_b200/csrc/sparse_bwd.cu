// Sparse-attention backward for sm_100a: delta, dQ and dK/dV.
//
// Replaces preprocess_delta (flash_topk_attn_v2/sparse_attn_bwd.py:12-33),
// sparse_attn_bwd_dq_kernel (csrc/sparse_attn_bwd_dq_kernel.cu:6-419) and
// sparse_attn_bwd_dkv_sorted_kernel (csrc/sparse_attn_bwd_dkv_kernel.cu:6-435).
//
// Both kernels use the 128-row union tiles of attn_common.cuh and the same
// three roles as the forward: TMA producer warp, UMMA issuer warp, and 16
// compute warps in two groups (one per S / dP buffer); inside a group two
// warps share each TMEM lane quarter and take half of a tile's columns each.
// With P = 2^(c S - lse2):
//   dQ  kernel, per candidate KV block:  S = Q K^T, dP = dO V^T  (Q, dO in TMEM),
//        dS = P (dP - delta) rounded to the I/O dtype in TMEM, dQ += dS K
//        (A from TMEM, K read MN-major from the tile that fed S).
//   dKV kernel, per q-block of the reverse list: S^T = K Q^T, dP^T = V dO^T,
//        P^T and dS^T written over the S^T / dP^T columns they came from,
//        dV += P^T dO, dK += dS^T Q (dO, Q read MN-major).  One CTA owns its
//        128 kv rows, so dK/dV need no atomics.
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "attn_common.cuh"
#include "ftk_host.cuh"
#include "ftk_sm100.cuh"

namespace ftk {

// ------------------------------------------------------------------- delta
// delta[bh][n] = sum_d o * do.  D / 8 lanes per (b, n, h) row, each with one
// 16-byte load per tensor (rows start on 16-byte boundaries: base pointers are
// 16-byte aligned and strides multiples of 8 elements), so a warp covers
// 256 / D rows at once.
__global__ void delta_kernel(const uint8_t* __restrict__ o, const uint8_t* __restrict__ dout,
                             int fmt, int64_t B, int64_t N, int64_t H, int D, int64_t so_b,
                             int64_t so_n, int64_t so_h, int64_t sd_b, int64_t sd_n, int64_t sd_h,
                             float* __restrict__ delta) {
  const int lpr = D >> 3;                         // lanes per row: 8, 16 or 32
  const int rpw = 32 / lpr;                       // rows per warp
  const int lane = threadIdx.x & 31;
  const int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t row = wid * rpw + lane / lpr;
  const int c = lane % lpr;
  float acc = 0.f;
  if (row < B * N * H) {
    const int64_t h = row % H, n = (row / H) % N, b = row / (H * N);
    const uint4 vo = __ldg(reinterpret_cast<const uint4*>(o + 2 * (b * so_b + n * so_n + h * so_h)) + c);
    const uint4 vd =
        __ldg(reinterpret_cast<const uint4*>(dout + 2 * (b * sd_b + n * sd_n + h * sd_h)) + c);
    const uint32_t wo[4] = {vo.x, vo.y, vo.z, vo.w}, wd[4] = {vd.x, vd.y, vd.z, vd.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 a = unpack2(wo[i], fmt), g = unpack2(wd[i], fmt);
      acc = fmaf(a.x, g.x, acc);
      acc = fmaf(a.y, g.y, acc);
    }
  }
  for (int d = lpr >> 1; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (c == 0 && row < B * N * H) {
    const int64_t h = row % H, n = (row / H) % N, b = row / (H * N);
    delta[(b * H + h) * N + n] = acc;
  }
}

// dS = 2^(c s - lse2) (dp - delta) for 32 columns of one row, two columns per
// instruction (fma.f32x2, add.f32x2, mul.f32x2, one cvt per pair).
template <int FMT>
__device__ __forceinline__ void ds_pairs(const uint32_t (&sv)[32], const uint32_t (&dv)[32],
                                         uint32_t (&pk)[16], float c, float neg_lse2,
                                         float neg_delta) {
  const float2 c2 = make_float2(c, c), nl = make_float2(neg_lse2, neg_lse2),
               nd = make_float2(neg_delta, neg_delta);
#pragma unroll
  for (int x = 0; x < 32; x += 2) {
    const float2 t =
        __ffma2_rn(make_float2(__uint_as_float(sv[x]), __uint_as_float(sv[x + 1])), c2, nl);
    const float2 pr = make_float2(fast_exp2(t.x), fast_exp2(t.y));
    const float2 dd =
        __fadd2_rn(make_float2(__uint_as_float(dv[x]), __uint_as_float(dv[x + 1])), nd);
    const float2 ds = __fmul2_rn(pr, dd);
    if (FMT == 1) {
      __nv_bfloat162 v = __floats2bfloat162_rn(ds.x, ds.y);
      pk[x >> 1] = *reinterpret_cast<uint32_t*>(&v);
    } else {
      __half2 v = __floats2half2_rn(ds.x, ds.y);
      pk[x >> 1] = *reinterpret_cast<uint32_t*>(&v);
    }
  }
}

// P^T = 2^(c s - lse2) and dS^T = P^T (dp - delta) for 16 columns (= q rows) of
// one kv row, two columns per instruction; lse2 / delta of the columns come
// NEGATED from shared memory, one 16-byte broadcast load per four columns.
template <int FMT>
__device__ __forceinline__ void pt_pairs(const uint32_t (&sv)[16], const uint32_t (&dv)[16],
                                         const float4* nl4, const float4* nd4, float c,
                                         uint32_t (&pp)[8], uint32_t (&pd)[8]) {
  const float2 c2 = make_float2(c, c);
#pragma unroll
  for (int x = 0; x < 16; x += 4) {
    const float4 lq = nl4[x >> 2];
    const float4 dq = nd4[x >> 2];
#pragma unroll
    for (int y = 0; y < 4; y += 2) {
      const float2 nl = y == 0 ? make_float2(lq.x, lq.y) : make_float2(lq.z, lq.w);
      const float2 nd = y == 0 ? make_float2(dq.x, dq.y) : make_float2(dq.z, dq.w);
      const float2 t = __ffma2_rn(
          make_float2(__uint_as_float(sv[x + y]), __uint_as_float(sv[x + y + 1])), c2, nl);
      const float2 pr = make_float2(fast_exp2(t.x), fast_exp2(t.y));
      const float2 dd = __fadd2_rn(
          make_float2(__uint_as_float(dv[x + y]), __uint_as_float(dv[x + y + 1])), nd);
      const float2 ds = __fmul2_rn(pr, dd);
      if (FMT == 1) {
        __nv_bfloat162 a = __floats2bfloat162_rn(pr.x, pr.y), b = __floats2bfloat162_rn(ds.x, ds.y);
        pp[(x + y) >> 1] = *reinterpret_cast<uint32_t*>(&a);
        pd[(x + y) >> 1] = *reinterpret_cast<uint32_t*>(&b);
      } else {
        __half2 a = __floats2half2_rn(pr.x, pr.y), b = __floats2half2_rn(ds.x, ds.y);
        pp[(x + y) >> 1] = *reinterpret_cast<uint32_t*>(&a);
        pd[(x + y) >> 1] = *reinterpret_cast<uint32_t*>(&b);
      }
    }
  }
}

constexpr int BW_THREADS = 576;  // 2 + 2 x 8 warps
constexpr int BW_MAX_STAGES = 4;
constexpr int DQ_KST = 7;        // dQ kernel: K tiles in the ring (held until dQ += dS K ran)
constexpr int DQ_VST = 5;        // dQ kernel: V tiles in the ring (free once dP is computed)

struct BwdParams {
  int N, H, QM, W, Mkv;
  int g, kvb, q_pad_head, kv_pad_head;
  int G, fmt, nstages;
  float scale, scale_log2;
  const int32_t* lists;      // dQ: merged [BH][QM][W]; dKV: reverse_idx [BH][Mkv][QM]
  const int32_t* counts;     // dKV: reverse_counts [BH][Mkv]
  const float* lse;
  const float* delta;
  void* out0;                // dQ kernel: dq ; dKV kernel: dk
  void* out1;                //                  dKV kernel: dv
  int64_t s0_b, s0_n, s0_h, s1_b, s1_n, s1_h;
  int* status;
  int kv_hdiv;               // query heads per kv head (grouped-query attention), 1 otherwise
  const int32_t* order;      // dKV: kv blocks by fan-in, heaviest first ([BH][Mkv]) or null
};

// ---------------------------------------------------------------------- dQ
// TMEM columns: Q 0..63 and dO 64..127 (16-bit pairs: the A operands of the
// S and dP UMMAs are read from TMEM, which leaves shared-memory bandwidth to
// the K/V tiles), S[2] 128/192, dP[2] 256/320 (dS written over their first
// half), dQ 384..
// Shared memory: the Q and dO tiles are dead once they sit in TMEM, so their
// 2 x 128 rows become four slots of the V ring (the fifth follows the K ring);
// K has its own ring.  K and V travel in
// separate rings because V is released after dP while K stays until dQ: the
// producer runs several tiles ahead, which is what lets the loads overlap the
// UMMAs instead of alternating with them.
template <int D>
__global__ void __launch_bounds__(BW_THREADS, 1)
sparse_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const BwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int ROW_TILE_BYTES = NCH * 128 * 128;
  // Head dim 256: Q and dO (128 TMEM columns each) no longer fit next to S, dP
  // and a 256-column dQ, so they stay in shared memory as SS operands; the
  // rings shrink to three K and two V tiles of at most 32 rows, all behind
  // the Q / dO tiles.  TMEM: S[2] 0/64, dP[2] 128/192, dQ 256..511.
  constexpr bool BIG = D > 128;
  constexpr int KST = BIG ? 3 : DQ_KST, VST = BIG ? 2 : DQ_VST;
  constexpr uint32_t COL_S = BIG ? 0 : 128, COL_DP = BIG ? 128 : 256, COL_DQ = BIG ? 256 : 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + ROW_TILE_BYTES;
  uint8_t* sV = smem;                          // over Q / dO once they are in TMEM
  uint8_t* sK = smem + 2 * ROW_TILE_BYTES;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[1 + 2 * DQ_KST + 2 * DQ_VST + 6];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * p.G;
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(p.G, p.QM - m0);
  const int tile_row0 = m0 * p.g - p.q_pad_head;
  const int kv_chunk_bytes = p.kvb * 128;
  const int tile_bytes = NCH * kv_chunk_bytes;   // one K or V tile
  auto v_slot = [&](int sv) {
    if (BIG) return smem_u32(sK) + (KST + sv) * tile_bytes;
    return sv < 4 ? smem_u32(sV) + sv * tile_bytes
                  : smem_u32(sK) + (DQ_KST + sv - 4) * tile_bytes;
  };

  const uint32_t bar_q = smem_u32(&bars[0]);
  auto bar_kfull = [&](int s) { return smem_u32(&bars[1 + s]); };
  auto bar_kempty = [&](int s) { return smem_u32(&bars[1 + DQ_KST + s]); };
  auto bar_vfull = [&](int s) { return smem_u32(&bars[1 + 2 * DQ_KST + s]); };
  auto bar_vempty = [&](int s) { return smem_u32(&bars[1 + 2 * DQ_KST + DQ_VST + s]); };
  constexpr int BAR_A0 = 1 + 2 * DQ_KST + 2 * DQ_VST;
  auto bar_afull = [&](int s) { return smem_u32(&bars[BAR_A0 + s]); };
  auto bar_dsfull = [&](int s) { return smem_u32(&bars[BAR_A0 + 2 + s]); };
  // arrives once, after the last UMMA of the CTA has retired
  const uint32_t bar_final = smem_u32(&bars[BAR_A0 + 4]);
  // Q and dO copied from shared memory into TMEM by the compute warps
  const uint32_t bar_qt = smem_u32(&bars[BAR_A0 + 5]);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < DQ_KST; s++) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
    }
    for (int s = 0; s < DQ_VST; s++) {
      mbar_init(bar_vfull(s), 1);
      mbar_init(bar_vempty(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_afull(s), 1);
      mbar_init(bar_dsfull(s), 8);  // one arrival per warp of the owning group
    }
    mbar_init(bar_final, 1);
    mbar_init(bar_qt, 8);   // the 8 warps that copy Q / dO
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  const int n = build_union(un, p.lists + (static_cast<int64_t>(bh) * p.QM + m0) * p.W, p.W,
                            groups, p.W, nullptr, p.Mkv, p.status);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};
  const bool split = (p.kvb % 32) == 0;   // kv columns of a tile shared by two warps per row

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_q, 2 * ROW_TILE_BYTES);
      for (int c = 0; c < NCH; c++) {
        tma_load_4d(smem_u32(sQ) + c * 128 * 128, &tm_q, bar_q, c * 64, h_idx, tile_row0, b_idx);
        tma_load_4d(smem_u32(sDO) + c * 128 * 128, &tm_do, bar_q, c * 64, h_idx, tile_row0, b_idx);
      }
      for (int i = 0; i < n; i++) {
        const int sk = i % KST, sv = i % VST;
        const int tok0 = static_cast<int>(un.ids[i]) * p.kvb - p.kv_pad_head;
        if (!mbar_wait(bar_kempty(sk), ((i / KST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const uint32_t kb = smem_u32(sK) + sk * tile_bytes;
        mbar_expect_tx(bar_kfull(sk), tile_bytes);
        for (int c = 0; c < NCH; c++)
          tma_load_4d(kb + c * kv_chunk_bytes, &tm_k, bar_kfull(sk), c * 64, h_idx / p.kv_hdiv,
                      tok0, b_idx);
        // the V ring lies over the Q / dO tiles: wait until they sit in TMEM
        if (!BIG && i == 0 && !mbar_wait(bar_qt, 0, w, FTK_DEV_TIMEOUT_TMA)) break;
        if (!mbar_wait(bar_vempty(sv), ((i / VST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const uint32_t vb = v_slot(sv);
        mbar_expect_tx(bar_vfull(sv), tile_bytes);
        for (int c = 0; c < NCH; c++)
          tma_load_4d(vb + c * kv_chunk_bytes, &tm_v, bar_vfull(sv), c * 64, h_idx / p.kv_hdiv,
                      tok0, b_idx);
      }
    }
  } else if (warp == 1) {
    if (n > 0) {
      // the whole warp runs this path; one elected lane issues the UMMAs
      const uint32_t idesc_a = umma_idesc(128, p.kvb, p.fmt, 0, 0);
      const uint32_t idesc_b = umma_idesc(128, D, p.fmt, 0, 1);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t kmn0 = smem_desc_sw128(smem_u32(sK), kv_chunk_bytes, 1024);
      // dS column of k-step ks: each half of the kv columns is written by its
      // own warps over the dP columns those warps read (see the compute part)
      // (kh is 1 or 2: shifts and masks only, the single issuing thread must
      // not spend longer between two UMMAs than the tensor core needs for one)
      const int kh = p.kvb / 32, kh_shift = kh >> 1, half_cols = p.kvb / 2;
      auto ds_col = [&](int ks) {
        return split ? (ks >> kh_shift) * half_cols + (ks & (kh - 1)) * 8 : ks * 8;
      };
      const uint64_t qdesc0 = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dodesc0 = smem_desc_sw128(smem_u32(sDO), 16, 1024);
      bool ok = mbar_wait(BIG ? bar_q : bar_qt, 0, w, FTK_DEV_TIMEOUT_MMA);
      tc_fence_after();
      // The tensor core runs dry whenever the issuing thread waits, so every
      // barrier of a round is waited for first and the round's UMMAs (dQ of
      // tile i, then S and dP of tile i + 2) go out as one uninterrupted batch.
      auto wait_kv = [&](int i) -> bool {
        return mbar_wait(bar_kfull(i % KST), (i / KST) & 1, w, FTK_DEV_TIMEOUT_MMA) &&
               mbar_wait(bar_vfull(i % VST), (i / VST) & 1, w, FTK_DEV_TIMEOUT_MMA);
      };
      auto mma_a = [&](int i) {   // elected lane only
        const int sk = i % KST, sv = i % VST;
        const uint64_t kdesc = desc_advance(kdesc0, sk * tile_bytes);
        const uint64_t vdesc = smem_desc_sw128(v_slot(sv), 16, 1024);
        const uint32_t sb = i & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          const uint32_t koff = (ks / 4) * kv_chunk_bytes + (ks % 4) * 32;
          if (BIG)
            umma_ss(tmem + COL_S + sb * 64,
                    desc_advance(qdesc0, (ks / 4) * 128 * 128 + (ks % 4) * 32),
                    desc_advance(kdesc, koff), idesc_a, ks > 0);
          else
            umma_ts(tmem + 128 + sb * 64, tmem + ks * 8, desc_advance(kdesc, koff), idesc_a,
                    ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          const uint32_t koff = (ks / 4) * kv_chunk_bytes + (ks % 4) * 32;
          if (BIG)
            umma_ss(tmem + COL_DP + sb * 64,
                    desc_advance(dodesc0, (ks / 4) * 128 * 128 + (ks % 4) * 32),
                    desc_advance(vdesc, koff), idesc_a, ks > 0);
          else
            umma_ts(tmem + 256 + sb * 64, tmem + 64 + ks * 8, desc_advance(vdesc, koff), idesc_a,
                    ks > 0);
        }
        umma_commit(bar_afull(sb));
        umma_commit(bar_vempty(sv));
      };
      auto mma_b = [&](int i) {   // elected lane only
        const int s = i % KST, sb = i & 1;
        const uint64_t kmn = desc_advance(kmn0, s * tile_bytes);
        if (p.kvb == 64) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++)
            umma_ts(tmem + COL_DQ, tmem + COL_DP + sb * 64 + (ks >> 1) * 32 + (ks & 1) * 8,
                    desc_advance(kmn, ks * 2048), idesc_b, (i > 0) || (ks > 0));
        } else {
          for (int ks = 0; ks < p.kvb / 16; ks++)
            umma_ts(tmem + COL_DQ, tmem + COL_DP + sb * 64 + ds_col(ks), desc_advance(kmn, ks * 2048),
                    idesc_b, (i > 0) || (ks > 0));
        }
        umma_commit(bar_kempty(s));
      };
      if (ok) ok = wait_kv(0);
      if (ok && n > 1) ok = wait_kv(1);
      tc_fence_after();
      if (ok && elect_one()) {
        mma_a(0);
        if (n > 1) mma_a(1);
      }
      __syncwarp();
      for (int i = 0; ok && i < n; i++) {
        const bool more = i + 2 < n;
        const int i2 = more ? i + 2 : i;   // last rounds: the dS barrier stands in
        const uint32_t wb[3] = {bar_dsfull(i & 1),
                                more ? bar_kfull(i2 % KST) : bar_dsfull(i & 1),
                                more ? bar_vfull(i2 % VST) : bar_dsfull(i & 1)};
        const uint32_t wp[3] = {static_cast<uint32_t>((i >> 1) & 1),
                                static_cast<uint32_t>(more ? (i2 / KST) & 1 : (i >> 1) & 1),
                                static_cast<uint32_t>(more ? (i2 / VST) & 1 : (i >> 1) & 1)};
        if (!mbar_wait_all<3>(wb, wp, w, FTK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
        if (elect_one()) {
          mma_b(i);
          if (i + 2 < n) mma_a(i + 2);
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(bar_final);
      __syncwarp();
    }
  } else {
    // Two groups of 8 warps; group w drains the buffers of tiles i = w (mod 2).
    // Inside a group two warps share each 32-row lane quarter and take one
    // half of the kv columns each, so a tile's latency-bound per-thread work
    // is 32 columns long and 4 compute warps per scheduler hide each other.
    const int cw = warp - 2;
    const int wg = cw >> 3;
    const int colhalf = (cw >> 2) & 1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int grp = r / p.g;
    const int qrow = tile_row0 + r;
    const bool row_valid = (grp < groups) && qrow >= 0 && qrow < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + COL_S + wg * 64;
    const uint32_t dp_addr = lane_addr + COL_DP + wg * 64;
    const int cbeg = split ? colhalf * (p.kvb / 2) : 0;
    const int cend = split ? cbeg + p.kvb / 2 : (colhalf == 0 ? p.kvb : 0);
    const float c = p.scale_log2;
    float lse2 = 0.f, dl = 0.f;
    if (row_valid) {
      lse2 = p.lse[static_cast<int64_t>(bh) * p.N + qrow] * 1.4426950408889634f;
      dl = p.delta[static_cast<int64_t>(bh) * p.N + qrow];
    }
    bool ok = true;
    if (!BIG && n > 0 && colhalf == 0) {
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
      if (lane == 0) mbar_arrive(bar_qt);
    }
    for (int i = wg; ok && i < n; i += 2) {
      // A(i) complete also means B(i-2) has retired (same issue order), so the
      // dS columns of this buffer are free again.
      if (!mbar_wait(bar_afull(wg), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int tok0 = static_cast<int>(un.ids[i]) * p.kvb - p.kv_pad_head;
      const int lo = max(0, -tok0), hi = min(p.kvb, p.N - tok0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == p.kvb;
      // dS of columns [c0, c0+w) is written over dP columns [cbeg + (c0-cbeg)/2, ..):
      // columns this thread has already read, never another warp's
      for (int c0 = cbeg; c0 < cend; c0 += 32) {
        const uint32_t ds_addr = dp_addr + cbeg + ((c0 - cbeg) >> 1);
        if (cend - c0 >= 32) {
          uint32_t sv[32], dv[32], pk[16];
          tmem_ld32(s_addr + c0, sv);
          tmem_ld32(dp_addr + c0, dv);
          tmem_wait_ld();
          if (fast) {
            if (p.fmt == 1) ds_pairs<1>(sv, dv, pk, c, -lse2, -dl);
            else ds_pairs<0>(sv, dv, pk, c, -lse2, -dl);
          } else {
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              float d0 = 0.f, d1 = 0.f;
              if (act && c0 + x >= lo && c0 + x < hi)
                d0 = fast_exp2(fmaf(__uint_as_float(sv[x]), c, -lse2)) *
                     (__uint_as_float(dv[x]) - dl);
              if (act && c0 + x + 1 >= lo && c0 + x + 1 < hi)
                d1 = fast_exp2(fmaf(__uint_as_float(sv[x + 1]), c, -lse2)) *
                     (__uint_as_float(dv[x + 1]) - dl);
              pk[x >> 1] = pack2(d0, d1, p.fmt);
            }
          }
          tmem_st16(ds_addr, pk);
        } else {
          uint32_t sv[16], dv[16], pk[8];
          tmem_ld16(s_addr + c0, sv);
          tmem_ld16(dp_addr + c0, dv);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 16; x += 2) {
            float d0 = 0.f, d1 = 0.f;
            if (act && c0 + x >= lo && c0 + x < hi)
              d0 = fast_exp2(fmaf(__uint_as_float(sv[x]), c, -lse2)) *
                   (__uint_as_float(dv[x]) - dl);
            if (act && c0 + x + 1 >= lo && c0 + x + 1 < hi)
              d1 = fast_exp2(fmaf(__uint_as_float(sv[x + 1]), c, -lse2)) *
                   (__uint_as_float(dv[x + 1]) - dl);
            pk[x >> 1] = pack2(d0, d1, p.fmt);
          }
          tmem_st8(ds_addr, pk);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dsfull(wg));
    }
    // epilogue: each group converts and stores one half of the head dimension
    if (ok && n > 0)
      ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = static_cast<uint8_t*>(p.out0) +
               2 * (static_cast<int64_t>(b_idx) * p.s0_b + static_cast<int64_t>(qrow) * p.s0_n +
                    static_cast<int64_t>(h_idx) * p.s0_h);
      // 32-column chunks of the head dim are dealt round-robin to the four
      // warps of a lane quarter
      for (int c0 = (wg * 2 + colhalf) * 32; c0 < D; c0 += 128) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld32(lane_addr + COL_DQ + c0, v);
          tmem_wait_ld();
        }
        if (row_valid) {
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float a = n > 0 ? __uint_as_float(v[x]) * p.scale : 0.f;
            const float b = n > 0 ? __uint_as_float(v[x + 1]) * p.scale : 0.f;
            pk[x >> 1] = pack2(a, b, p.fmt);
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
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// -------------------------------------------------------------------- dK/dV
// TMEM columns: S^T[2] 0/64 (P^T written over their first half), dP^T[2]
// 128/192 (dS^T likewise), dV 256.., dK 384..
// MODE 0 (head dims up to 128) produces dV and dK in one launch.  At head dim
// 256 two 256-column accumulators do not fit TMEM next to S^T and dP^T, so the
// work goes in two launches with one accumulator at columns 256..511 each:
// MODE 1 = dV only (needs neither V nor dP^T: K alone stays resident, which
// leaves room for four ring stages), MODE 2 = dK only.
template <int D, int MODE>
__global__ void __launch_bounds__(BW_THREADS, 1)
sparse_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_q,
                      const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const BwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int ROW_TILE_BYTES = NCH * 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + ROW_TILE_BYTES;
  uint8_t* sQD = smem + (MODE == 1 ? 1 : 2) * ROW_TILE_BYTES;
  constexpr uint32_t COL_DV = 256, COL_DK = MODE == 0 ? 384 : 256;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[1 + 2 * BW_MAX_STAGES + 6];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ __align__(16) float s_lse2[2][2][128], s_delta[2][2][128];  // [group][parity][q row]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  int j0 = blockIdx.x * p.G;                // first kv block of the tile
  if (p.order) {
    // Heaviest tiles first: the grid has one CTA per kv block, in the order of
    // `order` (fan-in descending, ties by lower id); the CTA whose block is the
    // first of its tile in that order does the tile, the others leave at once.
    const int32_t* cnt = p.counts + static_cast<int64_t>(bh) * p.Mkv;
    const int j = p.order[static_cast<int64_t>(bh) * p.Mkv + blockIdx.x];
    if (j < 0 || j >= p.Mkv) return;
    j0 = (j / p.G) * p.G;
    const int cj = cnt[j];
    for (int jj = j0; jj < min(j0 + p.G, p.Mkv); jj++) {
      const int cc = cnt[jj];
      if (jj != j && (cc > cj || (cc == cj && jj < j))) return;
    }
  }
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(p.G, p.Mkv - j0);
  const int tile_tok0 = j0 * p.kvb - p.kv_pad_head;
  const int q_chunk_bytes = p.g * 128;
  const int stage_bytes = 2 * NCH * q_chunk_bytes;
  const int NST = p.nstages;

  const uint32_t bar_kv = smem_u32(&bars[0]);
  auto bar_qfull = [&](int s) { return smem_u32(&bars[1 + s]); };
  auto bar_qempty = [&](int s) { return smem_u32(&bars[1 + BW_MAX_STAGES + s]); };
  auto bar_afull = [&](int s) { return smem_u32(&bars[1 + 2 * BW_MAX_STAGES + s]); };
  auto bar_pfull = [&](int s) { return smem_u32(&bars[1 + 2 * BW_MAX_STAGES + 2 + s]); };
  // arrives once, after the last UMMA of the CTA has retired
  const uint32_t bar_final = smem_u32(&bars[1 + 2 * BW_MAX_STAGES + 4]);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_kv, 1);
    for (int s = 0; s < BW_MAX_STAGES; s++) {
      mbar_init(bar_qfull(s), 1);
      mbar_init(bar_qempty(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_afull(s), 1);
      mbar_init(bar_pfull(s), 8);  // one arrival per warp of the owning group
    }
    mbar_init(bar_final, 1);
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  const int64_t kv_row = static_cast<int64_t>(bh) * p.Mkv + j0;
  const int n = build_union(un, p.lists + kv_row * p.QM, p.QM, groups, p.QM, p.counts + kv_row,
                            p.QM, p.status);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};
  const bool split = (p.g % 32) == 0;   // q columns of a tile shared by two warps per row

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_kv, (MODE == 1 ? 1 : 2) * ROW_TILE_BYTES);
      for (int c = 0; c < NCH; c++) {
        tma_load_4d(smem_u32(sK) + c * 128 * 128, &tm_k, bar_kv, c * 64, h_idx / p.kv_hdiv,
                    tile_tok0, b_idx);
        if (MODE != 1)
          tma_load_4d(smem_u32(sV) + c * 128 * 128, &tm_v, bar_kv, c * 64, h_idx / p.kv_hdiv,
                      tile_tok0, b_idx);
      }
      for (int i = 0; i < n; i++) {
        const int s = i % NST;
        if (!mbar_wait(bar_qempty(s), ((i / NST) & 1) ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const int row0 = static_cast<int>(un.ids[i]) * p.g - p.q_pad_head;
        const uint32_t base = smem_u32(sQD) + s * stage_bytes;
        mbar_expect_tx(bar_qfull(s), stage_bytes);
        for (int c = 0; c < NCH; c++) {
          tma_load_4d(base + c * q_chunk_bytes, &tm_q, bar_qfull(s), c * 64, h_idx, row0, b_idx);
          tma_load_4d(base + (NCH + c) * q_chunk_bytes, &tm_do, bar_qfull(s), c * 64, h_idx, row0,
                      b_idx);
        }
      }
    }
  } else if (warp == 1) {
    if (n > 0) {
      // the whole warp runs this path; one elected lane issues the UMMAs
      const uint32_t idesc_a = umma_idesc(128, p.g, p.fmt, 0, 0);
      const uint32_t idesc_b = umma_idesc(128, D, p.fmt, 0, 1);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t vdesc0 = smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t qdesc0 = smem_desc_sw128(smem_u32(sQD), 16, 1024);
      const uint64_t qmn0 = smem_desc_sw128(smem_u32(sQD), q_chunk_bytes, 1024);
      // P^T / dS^T column of k-step ks: each half of the q columns is written
      // by its own warps over the columns those warps read
      const int kh = p.g / 32, kh_shift = kh >> 1, half_cols = p.g / 2;
      auto pt_col = [&](int ks) {
        return split ? (ks >> kh_shift) * half_cols + (ks & (kh - 1)) * 8 : ks * 8;
      };
      bool ok = mbar_wait(bar_kv, 0, w, FTK_DEV_TIMEOUT_MMA);
      auto wait_q = [&](int i) -> bool {
        return mbar_wait(bar_qfull(i % NST), (i / NST) & 1, w, FTK_DEV_TIMEOUT_MMA);
      };
      auto mma_a = [&](int i) {   // elected lane only
        const int s = i % NST;
        const uint64_t qdesc = desc_advance(qdesc0, s * stage_bytes);
        const uint64_t dodesc = desc_advance(qdesc, NCH * q_chunk_bytes);
        const uint32_t sb = i & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
          const uint32_t aoff = (ks / 4) * 128 * 128 + (ks % 4) * 32;
          const uint32_t boff = (ks / 4) * q_chunk_bytes + (ks % 4) * 32;
          umma_ss(tmem + sb * 64, desc_advance(kdesc0, aoff), desc_advance(qdesc, boff), idesc_a,
                  ks > 0);
        }
        if (MODE != 1) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ks++) {
            const uint32_t aoff = (ks / 4) * 128 * 128 + (ks % 4) * 32;
            const uint32_t boff = (ks / 4) * q_chunk_bytes + (ks % 4) * 32;
            umma_ss(tmem + 128 + sb * 64, desc_advance(vdesc0, aoff), desc_advance(dodesc, boff),
                    idesc_a, ks > 0);
          }
        }
        umma_commit(bar_afull(sb));
      };
      auto mma_b = [&](int i) {   // elected lane only
        const int s = i % NST, sb = i & 1;
        const uint64_t qmn = desc_advance(qmn0, s * stage_bytes);
        const uint64_t domn = desc_advance(qmn, NCH * q_chunk_bytes);
        if (p.g == 64) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++) {
            const bool acc = (i > 0) || (ks > 0);
            const uint32_t col = sb * 64 + (ks >> 1) * 32 + (ks & 1) * 8;
            if (MODE != 2)
              umma_ts(tmem + COL_DV, tmem + col, desc_advance(domn, ks * 2048), idesc_b, acc);
            if (MODE != 1)
              umma_ts(tmem + COL_DK, tmem + 128 + col, desc_advance(qmn, ks * 2048), idesc_b, acc);
          }
        } else {
          for (int ks = 0; ks < p.g / 16; ks++) {
            const bool acc = (i > 0) || (ks > 0);
            if (MODE != 2)
              umma_ts(tmem + COL_DV, tmem + sb * 64 + pt_col(ks), desc_advance(domn, ks * 2048),
                      idesc_b, acc);
            if (MODE != 1)
              umma_ts(tmem + COL_DK, tmem + 128 + sb * 64 + pt_col(ks),
                      desc_advance(qmn, ks * 2048), idesc_b, acc);
          }
        }
        umma_commit(bar_qempty(s));
      };
      if (ok) ok = wait_q(0);
      if (ok && n > 1) ok = wait_q(1);
      tc_fence_after();
      if (ok && elect_one()) {
        mma_a(0);
        if (n > 1) mma_a(1);
      }
      __syncwarp();
      // The Q / dO ring is only as deep as the tiles in flight, so the next
      // tile's loads are often still on their way: dV / dK of tile i go out
      // first and the wait for tile i + 2 runs under them.
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
      if (ok && elect_one()) umma_commit(bar_final);
      __syncwarp();
    }
  } else {
    // Two groups of 8 warps; group w drains the buffers of tiles i = w (mod 2).
    // Inside a group two warps share each 32-row lane quarter and take one
    // half of the q columns each.
    const int cw = warp - 2;
    const int wg = cw >> 3;
    const int colhalf = (cw >> 2) & 1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int ct = (tid - 64) & 255;         // index inside the group
    const int grp = r / p.kvb;
    const int tok = tile_tok0 + r;
    const bool row_valid = (grp < groups) && tok >= 0 && tok < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t st_addr = lane_addr + wg * 64;         // S^T, then P^T
    const uint32_t dp_addr = lane_addr + 128 + wg * 64;   // dP^T, then dS^T
    const int cbeg = split ? colhalf * (p.g / 2) : 0;
    const int cend = split ? cbeg + p.g / 2 : (colhalf == 0 ? p.g : 0);
    const float c = p.scale_log2;
    bool ok = true;
    // every thread of a group runs all of the group's rounds (its named
    // barrier needs all 256); after a failed wait a thread only keeps the
    // barrier company and does no more work.
    for (int i = wg; i < n; i += 2) {
      const int pb = (i >> 1) & 1;           // per-group double buffer of lse / delta
      const int row0 = static_cast<int>(un.ids[i]) * p.g - p.q_pad_head;
      if (ct < p.g) {
        const int t = row0 + ct;
        float l2 = 0.f, dl = 0.f;
        if (t >= 0 && t < p.N) {   // staged negated: the packed fma / add take them as they are
          l2 = -p.lse[static_cast<int64_t>(bh) * p.N + t] * 1.4426950408889634f;
          dl = -p.delta[static_cast<int64_t>(bh) * p.N + t];
        }
        s_lse2[wg][pb][ct] = l2;
        s_delta[wg][pb][ct] = dl;
      }
      if (wg == 0)
        asm volatile("bar.sync 1, 256;" ::: "memory");
      else
        asm volatile("bar.sync 2, 256;" ::: "memory");
      if (!ok) continue;
      if (!mbar_wait(bar_afull(wg), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        continue;
      }
      tc_fence_after();
      const int lo = max(0, -row0), hi = min(p.g, p.N - row0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == p.g;
      const float4* l4 = reinterpret_cast<const float4*>(s_lse2[wg][pb]);
      const float4* d4 = reinterpret_cast<const float4*>(s_delta[wg][pb]);
      // P^T / dS^T of columns [c0, c0+16) go over columns cbeg + (c0-cbeg)/2 ..
      // of the S^T / dP^T regions: columns this thread has already read
      for (int c0 = cbeg; c0 < cend; c0 += 16) {
        uint32_t sv[16], dv[16], pp[8], pd[8];
        tmem_ld16(st_addr + c0, sv);
        if (MODE != 1) tmem_ld16(dp_addr + c0, dv);
        tmem_wait_ld();
        if (MODE == 1) {   // no dP^T in this launch: dS^T is computed and dropped
#pragma unroll
          for (int x = 0; x < 16; x++) dv[x] = 0u;
        }
        if (fast) {
          if (p.fmt == 1) pt_pairs<1>(sv, dv, l4 + (c0 >> 2), d4 + (c0 >> 2), c, pp, pd);
          else pt_pairs<0>(sv, dv, l4 + (c0 >> 2), d4 + (c0 >> 2), c, pp, pd);
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
            pp[x >> 1] = pack2(pv[0], pv[1], p.fmt);
            pp[(x >> 1) + 1] = pack2(pv[2], pv[3], p.fmt);
            pd[x >> 1] = pack2(dsv[0], dsv[1], p.fmt);
            pd[(x >> 1) + 1] = pack2(dsv[2], dsv[3], p.fmt);
          }
        }
        const int oc = cbeg + ((c0 - cbeg) >> 1);
        if (MODE != 2) tmem_st8(st_addr + oc, pp);
        if (MODE != 1) tmem_st8(dp_addr + oc, pd);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull(wg));
    }
    if (ok && n > 0)
      ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      // MODE 0: group 0 stores dV (TMEM 256..), group 1 stores dK (TMEM 384.., scaled);
      // otherwise both groups share the one accumulator's columns
      const int which = MODE == 0 ? wg : MODE - 1;
      uint8_t* base = static_cast<uint8_t*>(which == 0 ? p.out1 : p.out0);
      const int64_t sb_ = which == 0 ? p.s1_b : p.s0_b, sn_ = which == 0 ? p.s1_n : p.s0_n,
                    sh_ = which == 0 ? p.s1_h : p.s0_h;
      const float mul = which == 0 ? 1.f : p.scale;
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = base + 2 * (static_cast<int64_t>(b_idx) * sb_ + static_cast<int64_t>(tok) * sn_ +
                           static_cast<int64_t>(h_idx) * sh_);
      const int cfirst = MODE == 0 ? colhalf * 32 : (wg * 2 + colhalf) * 32;
      for (int c0 = cfirst; c0 < D; c0 += (MODE == 0 ? 64 : 128)) {
        uint32_t v[32];
        if (n > 0) {
          tmem_ld32(lane_addr + (which == 0 ? COL_DV : COL_DK) + c0, v);
          tmem_wait_ld();
        }
        if (row_valid) {
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float a = n > 0 ? __uint_as_float(v[x]) * mul : 0.f;
            const float b = n > 0 ? __uint_as_float(v[x + 1]) * mul : 0.f;
            pk[x >> 1] = pack2(a, b, p.fmt);
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
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace ftk

#include "sparse_bwd_dkv2.cuh"
#include "sparse_bwd_dq2.cuh"

namespace ftk {

static int bwd_common_checks(int dtype, int64_t B, int64_t H, int64_t N, int64_t D, int QM, int g,
                             int kvb, int q_pad_head, int kv_pad_head) {
  if (B <= 0 || H <= 0 || N <= 0 || QM <= 0) return FTK_ERR_BAD_ARG;
  if (dtype != FTK_DTYPE_F16 && dtype != FTK_DTYPE_BF16) return FTK_ERR_BAD_ARG;
  if (g <= 0 || kvb <= 0) return FTK_ERR_BAD_ARG;
  if (q_pad_head < 0 || q_pad_head >= g || kv_pad_head < 0 || kv_pad_head >= kvb)
    return FTK_ERR_BAD_ARG;
  if (static_cast<int64_t>(QM) * g < q_pad_head + N) return FTK_ERR_BAD_ARG;
  if (D != 64 && D != 128 && D != 256) return FTK_ERR_UNSUPPORTED;
  if (kvb % 16 != 0 || kvb > 64) return FTK_ERR_UNSUPPORTED;
  if (B * H > 65535) return FTK_ERR_BAD_ARG;
  return FTK_OK;
}

static bool aligned_out(const void* p, int64_t a, int64_t b, int64_t c) {
  return p && !(reinterpret_cast<uintptr_t>(p) & 15u) && !(a & 7) && !(b & 7) && !(c & 7);
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_sparse_bwd_dq(
    const void* q, const void* k, const void* v, const void* o, const void* dout, int dtype,
    int64_t B, int64_t H, int64_t Hkv, int64_t N, int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h,
    int64_t sk_b, int64_t sk_n, int64_t sk_h, int64_t sv_b, int64_t sv_n, int64_t sv_h,
    int64_t so_b, int64_t so_n, int64_t so_h, int64_t sdo_b, int64_t sdo_n, int64_t sdo_h,
    const int32_t* merged_idx, int QM, int W, int q_block_size, int kv_block_size, int q_pad_head,
    int kv_pad_head, float scale, const float* lse, float* delta, void* dq, int64_t sdq_b,
    int64_t sdq_n, int64_t sdq_h, int32_t* status, void* stream) {
  if (!q || !k || !v || !o || !dout || !merged_idx || !lse || !delta || W <= 0)
    return FTK_ERR_BAD_ARG;
  int e = bwd_common_checks(dtype, B, H, N, D, QM, q_block_size, kv_block_size, q_pad_head,
                            kv_pad_head);
  if (e) return e;
  if (Hkv <= 0) Hkv = H;
  if (H % Hkv != 0) return FTK_ERR_BAD_ARG;
  if (q_block_size > 128) return FTK_ERR_UNSUPPORTED;
  if (!aligned_out(dq, sdq_b, sdq_n, sdq_h)) return FTK_ERR_BAD_ARG;
  // delta reads O and dO with 16-byte loads
  if ((so_b | so_n | so_h | sdo_b | sdo_n | sdo_h) & 7) return FTK_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dout)) & 15u)
    return FTK_ERR_BAD_ARG;
  const int64_t Mkv = (kv_pad_head + N + kv_block_size - 1) / kv_block_size;
  if (Mkv > AT_MAX_BLOCKS) return FTK_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int64_t rows = B * N * H;
  const int64_t delta_warps = (rows + 256 / D - 1) / (256 / D);   // 256 / D rows per warp
  delta_kernel<<<static_cast<unsigned>((delta_warps * 32 + 255) / 256), 256, 0, st>>>(
      static_cast<const uint8_t*>(o), static_cast<const uint8_t*>(dout), dtype, B, N, H,
      static_cast<int>(D), so_b, so_n, so_h, sdo_b, sdo_n, sdo_h, delta);
  if (cudaGetLastError() != cudaSuccess) return FTK_ERR_CUDA;

  BwdParams p{};
  p.N = static_cast<int>(N);
  p.H = static_cast<int>(H);
  p.QM = QM;
  p.W = W;
  p.Mkv = static_cast<int>(Mkv);
  p.g = q_block_size;
  p.kvb = kv_block_size;
  p.q_pad_head = q_pad_head;
  p.kv_pad_head = kv_pad_head;
  p.G = std::max(1, std::min(AT_MAX_GROUPS, 128 / q_block_size));
  p.fmt = dtype;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lists = merged_idx;
  p.lse = lse;
  p.delta = delta;
  p.out0 = dq;
  p.s0_b = sdq_b;
  p.s0_n = sdq_n;
  p.s0_h = sdq_h;
  p.status = status;
  p.kv_hdiv = static_cast<int>(H / Hkv);

  CUtensorMap tq, tdo, tk, tv;
  if ((e = encode_tmap_bnhd(&tq, q, dtype, B, N, H, D, sq_b, sq_n, sq_h, 64, 128))) return e;
  if ((e = encode_tmap_bnhd(&tdo, dout, dtype, B, N, H, D, sdo_b, sdo_n, sdo_h, 64, 128))) return e;
  if ((e = encode_tmap_bnhd(&tk, k, dtype, B, N, Hkv, D, sk_b, sk_n, sk_h, 64, kv_block_size)))
    return e;
  if ((e = encode_tmap_bnhd(&tv, v, dtype, B, N, Hkv, D, sv_b, sv_n, sv_h, 64, kv_block_size)))
    return e;
  // head dim 128 with 64-row q and kv blocks: the kernel on pairs of SMs
  // (pairs walk the union of four lists: only when the lists can cover a good
  // part of the blocks, see ftk_sparse_fwd)
  const char* env2 = getenv("FTK_DQ_2CTA");
  if (D == 128 && q_block_size == 64 && kv_block_size == 64 &&
      4 * static_cast<int64_t>(W) >= Mkv && !(env2 && env2[0] == '0')) {
    CUtensorMap tk32, tv32;
    if ((e = encode_tmap_bnhd(&tk32, k, dtype, B, N, Hkv, D, sk_b, sk_n, sk_h, 64, 32))) return e;
    if ((e = encode_tmap_bnhd(&tv32, v, dtype, B, N, Hkv, D, sv_b, sv_n, sv_h, 64, 32))) return e;
    const size_t smem2 = 1024 + 2 * 2 * 128 * 128 + static_cast<size_t>(DQ2_STAGES) * 24576;
    dim3 grid2(2 * ((QM + 3) / 4), static_cast<unsigned>(B * H));
    if (dtype == FTK_DTYPE_BF16) {
      if (cudaFuncSetAttribute(sparse_bwd_dq2_kernel<1>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem2)) != cudaSuccess)
        return FTK_ERR_CUDA;
      sparse_bwd_dq2_kernel<1><<<grid2, BW_THREADS, smem2, st>>>(tq, tdo, tk, tk32, tv32, p);
    } else {
      if (cudaFuncSetAttribute(sparse_bwd_dq2_kernel<0>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem2)) != cudaSuccess)
        return FTK_ERR_CUDA;
      sparse_bwd_dq2_kernel<0><<<grid2, BW_THREADS, smem2, st>>>(tq, tdo, tk, tk32, tv32, p);
    }
    return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
  }
  const int nch = static_cast<int>(D / 64);
  dim3 grid((QM + p.G - 1) / p.G, static_cast<unsigned>(B * H));
  if (D == 256) {
    // Q and dO resident, three K and two V tiles behind them: kv blocks of at most 32 rows
    if (kv_block_size > 32) return FTK_ERR_UNSUPPORTED;
    const size_t smem_big =
        1024 + 2 * nch * 128 * 128 + static_cast<size_t>(3 + 2) * nch * kv_block_size * 128;
    if (cudaFuncSetAttribute(sparse_bwd_dq_kernel<256>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem_big)) != cudaSuccess)
      return FTK_ERR_CUDA;
    sparse_bwd_dq_kernel<256><<<grid, BW_THREADS, smem_big, st>>>(tq, tdo, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
  }
  // four V slots lie over the Q / dO tiles, the rest of the V ring behind the K ring
  const size_t smem = 1024 + 2 * nch * 128 * 128 +
                      static_cast<size_t>(DQ_KST + DQ_VST - 4) * nch * kv_block_size * 128;
  if (D == 64) {
    if (cudaFuncSetAttribute(sparse_bwd_dq_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    sparse_bwd_dq_kernel<64><<<grid, BW_THREADS, smem, st>>>(tq, tdo, tk, tv, p);
  } else {
    if (cudaFuncSetAttribute(sparse_bwd_dq_kernel<128>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    sparse_bwd_dq_kernel<128><<<grid, BW_THREADS, smem, st>>>(tq, tdo, tk, tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" int ftk_sparse_bwd_dkv(
    const void* q, const void* k, const void* v, const void* dout, int dtype, int64_t B, int64_t H,
    int64_t Hkv, int64_t N, int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h, int64_t sk_b, int64_t sk_n,
    int64_t sk_h, int64_t sv_b, int64_t sv_n, int64_t sv_h, int64_t sdo_b, int64_t sdo_n,
    int64_t sdo_h, const int32_t* reverse_idx, const int32_t* reverse_counts,
    const int32_t* sorted_kv, int QM, int M, int q_block_size, int kv_block_size, int q_pad_head,
    int kv_pad_head, float scale, const float* lse, const float* delta, void* dk, int64_t sdk_b,
    int64_t sdk_n, int64_t sdk_h, void* dv, int64_t sdv_b, int64_t sdv_n, int64_t sdv_h,
    int fwd_list_width, int32_t* status, void* stream) {
  if (!q || !k || !v || !dout || !reverse_idx || !reverse_counts || !lse || !delta)
    return FTK_ERR_BAD_ARG;
  int e = bwd_common_checks(dtype, B, H, N, D, QM, q_block_size, kv_block_size, q_pad_head,
                            kv_pad_head);
  if (e) return e;
  if (Hkv <= 0) Hkv = H;
  if (H % Hkv != 0) return FTK_ERR_BAD_ARG;
  if (q_block_size % 16 != 0 || q_block_size > 64) return FTK_ERR_UNSUPPORTED;
  if (QM > AT_MAX_BLOCKS) return FTK_ERR_UNSUPPORTED;
  if (M <= 0 || static_cast<int64_t>(M) * kv_block_size < kv_pad_head + N) return FTK_ERR_BAD_ARG;
  if (!aligned_out(dk, sdk_b, sdk_n, sdk_h) || !aligned_out(dv, sdv_b, sdv_n, sdv_h))
    return FTK_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  BwdParams p{};
  p.N = static_cast<int>(N);
  p.H = static_cast<int>(H);
  p.QM = QM;
  p.W = QM;
  p.Mkv = M;
  p.g = q_block_size;
  p.kvb = kv_block_size;
  p.q_pad_head = q_pad_head;
  p.kv_pad_head = kv_pad_head;
  p.G = std::max(1, std::min(AT_MAX_GROUPS, 128 / kv_block_size));
  p.fmt = dtype;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lists = reverse_idx;
  p.counts = reverse_counts;
  p.lse = lse;
  p.delta = delta;
  p.out0 = dk;
  p.s0_b = sdk_b;
  p.s0_n = sdk_n;
  p.s0_h = sdk_h;
  p.out1 = dv;
  p.s1_b = sdv_b;
  p.s1_n = sdv_n;
  p.s1_h = sdv_h;
  p.status = status;
  p.kv_hdiv = static_cast<int>(H / Hkv);

  CUtensorMap tq, tdo, tk, tv;
  if ((e = encode_tmap_bnhd(&tq, q, dtype, B, N, H, D, sq_b, sq_n, sq_h, 64, q_block_size)))
    return e;
  if ((e = encode_tmap_bnhd(&tdo, dout, dtype, B, N, H, D, sdo_b, sdo_n, sdo_h, 64, q_block_size)))
    return e;
  if ((e = encode_tmap_bnhd(&tk, k, dtype, B, N, Hkv, D, sk_b, sk_n, sk_h, 64, 128))) return e;
  if ((e = encode_tmap_bnhd(&tv, v, dtype, B, N, Hkv, D, sv_b, sv_n, sv_h, 64, 128))) return e;
  // head dim 128 with 64-row q and kv blocks: the kernel on pairs of SMs
  const char* env2 = getenv("FTK_DKV_2CTA");
  const bool long_lists = fwd_list_width <= 0 || 4 * static_cast<int64_t>(fwd_list_width) >= M;
  if (D == 128 && q_block_size == 64 && kv_block_size == 64 && long_lists &&
      !(env2 && env2[0] == '0')) {
    CUtensorMap tq32, tdo32;
    if ((e = encode_tmap_bnhd(&tq32, q, dtype, B, N, H, D, sq_b, sq_n, sq_h, 64, 32))) return e;
    if ((e = encode_tmap_bnhd(&tdo32, dout, dtype, B, N, H, D, sdo_b, sdo_n, sdo_h, 64, 32)))
      return e;
    const size_t smem2 = 1024 + 2 * 2 * 128 * 128 + static_cast<size_t>(DK2_STAGES) * 32768;
    dim3 grid2(2 * ((M + 3) / 4), static_cast<unsigned>(B * H));
    if (dtype == FTK_DTYPE_BF16) {
      if (cudaFuncSetAttribute(sparse_bwd_dkv2_kernel<1>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem2)) != cudaSuccess)
        return FTK_ERR_CUDA;
      sparse_bwd_dkv2_kernel<1><<<grid2, BW_THREADS, smem2, st>>>(tq, tdo, tq32, tdo32, tk, tv, p);
    } else {
      if (cudaFuncSetAttribute(sparse_bwd_dkv2_kernel<0>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem2)) != cudaSuccess)
        return FTK_ERR_CUDA;
      sparse_bwd_dkv2_kernel<0><<<grid2, BW_THREADS, smem2, st>>>(tq, tdo, tq32, tdo32, tk, tv, p);
    }
    return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
  }
  const int nch = static_cast<int>(D / 64);
  const int stage_bytes = 2 * nch * q_block_size * 128;
  const int tile_bytes = nch * 128 * 128;          // K or V of the CTA's 128 kv rows
  // 227 KB per CTA less the static part (union scratch, lse / delta staging: ~21 KB) and the
  // resident tiles; at head dim 256 that leaves two stages of q blocks of up to 32 rows next to
  // K and V, four next to K alone
  auto stages = [&](int resident) {
    const int ring_bytes = (227 - 23) * 1024 - resident * tile_bytes;
    return std::min(BW_MAX_STAGES, std::min(128 * 1024, ring_bytes) / stage_bytes);
  };
  auto smem_for = [&](int resident, int nst) {
    return static_cast<size_t>(1024) + static_cast<size_t>(resident) * tile_bytes +
           static_cast<size_t>(nst) * stage_bytes;
  };
  // one-CTA kernels: tiles in order of fan-in when the caller brings the order
  const char* oe = getenv("FTK_DKV_ORDER");
  p.order = (sorted_kv && !(oe && oe[0] == '0')) ? sorted_kv : nullptr;
  dim3 grid(p.order ? M : (M + p.G - 1) / p.G, static_cast<unsigned>(B * H));
  if (D == 256) {
    const int nst_dv = stages(1), nst_dk = stages(2);
    if (nst_dk < 2) return FTK_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(sparse_bwd_dkv_kernel<256, 1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem_for(1, nst_dv))) != cudaSuccess ||
        cudaFuncSetAttribute(sparse_bwd_dkv_kernel<256, 2>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem_for(2, nst_dk))) != cudaSuccess)
      return FTK_ERR_CUDA;
    p.nstages = nst_dv;
    sparse_bwd_dkv_kernel<256, 1><<<grid, BW_THREADS, smem_for(1, nst_dv), st>>>(tq, tdo, tk, tv, p);
    p.nstages = nst_dk;
    sparse_bwd_dkv_kernel<256, 2><<<grid, BW_THREADS, smem_for(2, nst_dk), st>>>(tq, tdo, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
  }
  p.nstages = stages(2);
  if (p.nstages < 2) return FTK_ERR_UNSUPPORTED;
  const size_t smem = smem_for(2, p.nstages);
  if (D == 64) {
    if (cudaFuncSetAttribute(sparse_bwd_dkv_kernel<64, 0>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    sparse_bwd_dkv_kernel<64, 0><<<grid, BW_THREADS, smem, st>>>(tq, tdo, tk, tv, p);
  } else {
    if (cudaFuncSetAttribute(sparse_bwd_dkv_kernel<128, 0>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    sparse_bwd_dkv_kernel<128, 0><<<grid, BW_THREADS, smem, st>>>(tq, tdo, tk, tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}
