// Gathered-KV flash attention forward for sm_100a.
//
// Replaces sparse_attn_fwd_kernel of the reference
// (flash_topk_attn_v2/csrc/sparse_attn_kernel.cu:6-365).
//
// Two kernels: the exact running-maximum kernel below (every supported shape
// and dtype) and the pipelined fixed-reference kernel of sparse_fwd_pipe.cuh
// (64-row q and kv blocks), which ftk_sparse_fwd launches first when the
// caller passes a workspace; the exact kernel then only redoes flagged CTAs.
//
// One CTA owns 128 consecutive virtual query rows = G q-blocks of one (batch,
// head) slice and walks the union of their candidate KV blocks in ascending
// order (see attn_common.cuh).  Roles: warp 0 = TMA producer (Q once, then a
// ring of K/V block tiles), warp 1 = UMMA issuer, warps 2..9 = two softmax
// groups of 128 threads, one query row per thread in each group.
//   S = Q K^T      tcgen05 SS, both operands K-major, accumulator in TMEM
//   P = 2^(c S - m) rounded to the I/O dtype, written over the S columns
//   O += P V       tcgen05 with A = P from TMEM, B = V read MN-major from the
//                  same row-major tile TMA delivered
// Even union entries go through S buffer 0 / softmax group 0 / accumulator
// O0, odd entries through buffer 1 / group 1 / O1, so the two groups work
// concurrently and the tensor core alternates between them; each group keeps
// its own running maximum and sum and the two partial results are merged in
// the epilogue (split-KV merge).  A group raises its running maximum only
// when a block exceeds it by more than 2^8 (P stays inside fp16 range); its
// O accumulator is then rescaled in TMEM by the row owners.
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "attn_common.cuh"
#include "ftk_host.cuh"
#include "ftk_sm100.cuh"

namespace ftk {

constexpr int FW_THREADS = 320;  // 2 + 2 x 4 warps
constexpr int FW_MAX_STAGES = 4;
// TMEM columns.  kv blocks of at most 64 rows: Q (16-bit pairs) 0..63, S[2]
// at 64 / 128, so the S UMMAs read their A operand from TMEM and shared-memory
// bandwidth is left to the K/V tiles (an SS UMMA of this shape spends more
// time fetching Q than multiplying).  Larger kv blocks: S[2] at 0 / 128 and Q
// stays in shared memory.  P is written over the S columns.  O[2] at 256 / 384.
constexpr int FW_COL_O = 256;

struct FwdParams {
  int N, H, QM, W, Mkv;
  int g, kvb, q_pad_head, kv_pad_head;
  int G, fmt, nstages;
  float scale_log2;
  const int32_t* merged;
  void* o;
  int64_t so_b, so_n, so_h;
  float* lse;
  int* status;
  int kv_hdiv;          // query heads per kv head (grouped-query attention), 1 otherwise
  int* redo_out;        // pipelined kernel: one word per CTA, 1 = redo with the exact kernel
  const int* redo_in;   // exact kernel: when set, CTAs whose word is 0 return at once
  int v_off;            // first head-dim column of V / O this launch produces (head dim 256)
};

// D = head dim of the Q.K^T contraction, DV = columns of V / O per launch
// (p.v_off = first column).  Head dim 256: two 256-column accumulators do not
// fit TMEM next to S, so there is ONE accumulator (columns 256..511) and one
// softmax group with one running maximum drains both S buffers in turn; Q
// stays in shared memory.  The tile's UMMAs (16 + 4 k-steps) outlast its
// softmax, so one group keeps up.  The second group only helps in the epilogue.
template <int D, int DV>
__global__ void __launch_bounds__(FW_THREADS, 1)
sparse_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  constexpr int NCH = D / 64;
  constexpr int NCV = DV / 64;
  constexpr bool SINGLE = DV > 128;     // one O accumulator, one softmax group
  constexpr int Q_BYTES = NCH * 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + Q_BYTES;
  __shared__ UnionScratch un;
  __shared__ __align__(8) uint64_t bars[3 + 2 * FW_MAX_STAGES + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ float s_m[2][128], s_l[2][128];

  if (p.redo_in && p.redo_in[blockIdx.y * gridDim.x + blockIdx.x] == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * p.G;
  const int bh = blockIdx.y;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;
  const int groups = min(p.G, p.QM - m0);
  const int tile_row0 = m0 * p.g - p.q_pad_head;
  const int kv_chunk_bytes = p.kvb * 128;
  const int stage_bytes = (NCH + NCV) * kv_chunk_bytes;
  const int NST = p.nstages;

  const uint32_t bar_q = smem_u32(&bars[0]);
  const uint32_t bar_final = smem_u32(&bars[1]);
  const uint32_t bar_qt = smem_u32(&bars[2]);   // Q copied into TMEM
  auto bar_kvfull = [&](int s) { return smem_u32(&bars[3 + s]); };
  auto bar_kvempty = [&](int s) { return smem_u32(&bars[3 + FW_MAX_STAGES + s]); };
  auto bar_sfull = [&](int s) { return smem_u32(&bars[3 + 2 * FW_MAX_STAGES + s]); };
  auto bar_pfull = [&](int s) { return smem_u32(&bars[3 + 2 * FW_MAX_STAGES + 2 + s]); };
  const bool q_tmem = D <= 128 && p.kvb <= 64;
  const uint32_t s_col0 = q_tmem ? 64u : 0u, s_stride = q_tmem ? 64u : 128u;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_final, 1);
    mbar_init(bar_qt, 4);
    for (int s = 0; s < FW_MAX_STAGES; s++) {
      mbar_init(bar_kvfull(s), 1);
      mbar_init(bar_kvempty(s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(bar_sfull(s), 1);
      mbar_init(bar_pfull(s), 4);  // one arrival per warp of the owning group
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0 && n > 0) {
      mbar_expect_tx(bar_q, Q_BYTES);
      for (int c = 0; c < NCH; c++)
        tma_load_4d(smem_u32(sQ) + c * 128 * 128, &tm_q, bar_q, c * 64, h_idx, tile_row0, b_idx);
      for (int i = 0; i < n; i++) {
        const int s = i % NST;
        const uint32_t ph = (i / NST) & 1;
        if (!mbar_wait(bar_kvempty(s), ph ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const int tok0 = static_cast<int>(un.ids[i]) * p.kvb - p.kv_pad_head;
        const uint32_t base = smem_u32(sKV) + s * stage_bytes;
        mbar_expect_tx(bar_kvfull(s), stage_bytes);
        for (int c = 0; c < NCH; c++)
          tma_load_4d(base + c * kv_chunk_bytes, &tm_k, bar_kvfull(s), c * 64, h_idx / p.kv_hdiv,
                      tok0, b_idx);
        for (int c = 0; c < NCV; c++)
          tma_load_4d(base + (NCH + c) * kv_chunk_bytes, &tm_v, bar_kvfull(s), p.v_off + c * 64,
                      h_idx / p.kv_hdiv, tok0, b_idx);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- UMMA issuer
    if (n > 0) {
      // the whole warp runs this path; one elected lane issues the UMMAs
      const uint32_t idesc_s = umma_idesc(128, p.kvb, p.fmt, 0, 0);
      const uint32_t idesc_pv = umma_idesc(128, DV, p.fmt, 0, 1);
      const uint64_t qdesc0 = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sKV), 16, 1024);
      const uint64_t vdesc0 =
          smem_desc_sw128(smem_u32(sKV) + NCH * kv_chunk_bytes, kv_chunk_bytes, 1024);
      bool ok = mbar_wait(q_tmem ? bar_qt : bar_q, 0, w, FTK_DEV_TIMEOUT_MMA);
      tc_fence_after();
      auto issue_s = [&](int i) -> bool {
        const int s = i % NST;
        if (!mbar_wait(bar_kvfull(s), (i / NST) & 1, w, FTK_DEV_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t kdesc = desc_advance(kdesc0, s * stage_bytes);
        const uint32_t d_tmem = tmem + s_col0 + (i & 1) * s_stride;
        if (elect_one()) {
          if (q_tmem) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ks++)
              umma_ts(d_tmem, tmem + ks * 8,
                      desc_advance(kdesc, (ks / 4) * kv_chunk_bytes + (ks % 4) * 32), idesc_s,
                      ks > 0);
          } else {
#pragma unroll
            for (int ks = 0; ks < D / 16; ks++)
              umma_ss(d_tmem, desc_advance(qdesc0, (ks / 4) * 128 * 128 + (ks % 4) * 32),
                      desc_advance(kdesc, (ks / 4) * kv_chunk_bytes + (ks % 4) * 32), idesc_s,
                      ks > 0);
          }
          umma_commit(bar_sfull(i & 1));
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok && n > 1) ok = issue_s(1);
      for (int i = 0; ok && i < n; i++) {
        const int s = i % NST, sb = i & 1;
        if (!mbar_wait(bar_pfull(sb), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint64_t vdesc = desc_advance(vdesc0, s * stage_bytes);
        const int ksteps = p.kvb / 16;
        if (elect_one()) {
          for (int ks = 0; ks < ksteps; ks++) {
            umma_ts(tmem + FW_COL_O + (SINGLE ? 0 : sb * 128),
                    tmem + s_col0 + sb * s_stride + ks * 8, desc_advance(vdesc, ks * 2048),
                    idesc_pv, (i >= (SINGLE ? 1 : 2)) || (ks > 0));
          }
          umma_commit(bar_kvempty(s));
        }
        __syncwarp();
        // S(i+2) overwrites the columns PV(i) reads P from; the tensor core
        // runs UMMAs in issue order, so issuing it after PV(i) is enough.
        if (i + 2 < n) ok = issue_s(i + 2);
      }
      if (ok && elect_one()) umma_commit(bar_final);
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------- softmax threads
    const int grp_w = (warp - 2) >> 2;       // softmax group = S buffer it drains
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int grp = r / p.g;
    const int qrow = tile_row0 + r;
    const bool row_valid = (grp < groups) && qrow >= 0 && qrow < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_addr = lane_addr + FW_COL_O + (SINGLE ? 0 : grp_w * 128);
    const float c = p.scale_log2;
    float m_run = -INFINITY, l = 0.f;
    bool ok = true;

    if (q_tmem && n > 0 && grp_w == 0) {
      // group 0 moves the Q tile from (swizzled) shared memory into TMEM:
      // row r -> lane r, two 16-bit values per column
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

    for (int i = SINGLE ? (grp_w == 0 ? 0 : n) : grp_w; ok && i < n; i += SINGLE ? 1 : 2) {
      // S(i) complete also means PV(i-2) has retired (same issue order), so
      // this buffer's P columns (and with two groups: this group's O
      // accumulator) are free to touch.
      const int sbuf = SINGLE ? (i & 1) : grp_w;
      const uint32_t s_addr = lane_addr + s_col0 + sbuf * s_stride;
      if (!mbar_wait(bar_sfull(sbuf), (i >> 1) & 1, w, FTK_DEV_TIMEOUT_CONSUMER)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // One shared accumulator: PV(i-1) may still be adding to it.  A thread
      // that has to rescale it first waits until that UMMA has retired (the
      // commit that hands tile i-1's K / V stage back to the producer).
      auto o_quiet = [&]() -> bool {
        if (!SINGLE || i == 0) return true;
        const int sp = (i - 1) % NST;
        if (!mbar_wait(bar_kvempty(sp), ((i - 1) / NST) & 1, w, FTK_DEV_TIMEOUT_CONSUMER))
          return false;
        tc_fence_after();
        return true;
      };
      const int tok0 = static_cast<int>(un.ids[i]) * p.kvb - p.kv_pad_head;
      const int lo = max(0, -tok0), hi = min(p.kvb, p.N - tok0);
      const bool act = row_valid && ((un.masks[i] >> grp) & 1) && hi > lo;
      const bool any_act = __any_sync(0xffffffffu, act);
      const bool fast = __all_sync(0xffffffffu, act) && lo == 0 && hi == p.kvb;

      if (any_act && p.kvb == 64) {
        // ---- whole row of S in registers, one TMEM round trip
        uint32_t v0[32], v1[32];
        tmem_ld32(s_addr, v0);
        tmem_ld32(s_addr + 32, v1);
        tmem_wait_ld();
        float mt = -INFINITY;
        if (fast) {
#pragma unroll
          for (int x = 0; x < 32; x++)
            mt = fmaxf(mt, fmaxf(__uint_as_float(v0[x]), __uint_as_float(v1[x])));
        } else if (act) {
#pragma unroll
          for (int x = 0; x < 32; x++) {
            if (x >= lo && x < hi) mt = fmaxf(mt, __uint_as_float(v0[x]));
            if (x + 32 >= lo && x + 32 < hi) mt = fmaxf(mt, __uint_as_float(v1[x]));
          }
        }
        const float mt2 = act ? mt * c : -INFINITY;
        const bool grow = act && (mt2 > m_run + 8.f || m_run == -INFINITY);
        const float m_new = grow ? mt2 : m_run;
        const bool resc = grow && l > 0.f;
        if (__any_sync(0xffffffffu, resc)) {
          if (!o_quiet()) {
            ok = false;
            break;
          }
          const float alpha = resc ? fast_exp2(m_run - m_new) : 1.f;
          for (int c0 = 0; c0 < DV; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(o_addr + c0, ov);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; x++) ov[x] = __float_as_uint(__uint_as_float(ov[x]) * alpha);
            tmem_st32(o_addr + c0, ov);
          }
          l *= alpha;
        }
        m_run = m_new;
        uint32_t pk[32];
        float l0 = 0.f, l1 = 0.f;
        if (fast) {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            const float a0 = fast_exp2(fmaf(__uint_as_float(v0[x]), c, -m_run));
            const float a1 = fast_exp2(fmaf(__uint_as_float(v0[x + 1]), c, -m_run));
            const float b0 = fast_exp2(fmaf(__uint_as_float(v1[x]), c, -m_run));
            const float b1 = fast_exp2(fmaf(__uint_as_float(v1[x + 1]), c, -m_run));
            l0 += a0 + a1;
            l1 += b0 + b1;
            pk[x >> 1] = pack2(a0, a1, p.fmt);
            pk[16 + (x >> 1)] = pack2(b0, b1, p.fmt);
          }
        } else {
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
            if (act && x >= lo && x < hi) a0 = fast_exp2(fmaf(__uint_as_float(v0[x]), c, -m_run));
            if (act && x + 1 >= lo && x + 1 < hi)
              a1 = fast_exp2(fmaf(__uint_as_float(v0[x + 1]), c, -m_run));
            if (act && x + 32 >= lo && x + 32 < hi)
              b0 = fast_exp2(fmaf(__uint_as_float(v1[x]), c, -m_run));
            if (act && x + 33 >= lo && x + 33 < hi)
              b1 = fast_exp2(fmaf(__uint_as_float(v1[x + 1]), c, -m_run));
            l0 += a0 + a1;
            l1 += b0 + b1;
            pk[x >> 1] = pack2(a0, a1, p.fmt);
            pk[16 + (x >> 1)] = pack2(b0, b1, p.fmt);
          }
        }
        l += l0 + l1;
        tmem_st32(s_addr, pk);
      } else if (any_act) {
        // ---- generic block size: two passes over S in 16-column chunks.  P
        // chunk k lands on columns S has already been read from.
        float mt = -INFINITY;
        for (int c0 = 0; c0 < p.kvb; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(s_addr + c0, v);
          tmem_wait_ld();
#pragma unroll
          for (int x = 0; x < 16; x++)
            if (c0 + x >= lo && c0 + x < hi) mt = fmaxf(mt, __uint_as_float(v[x]));
        }
        const float mt2 = act ? mt * c : -INFINITY;
        const bool grow = act && (mt2 > m_run + 8.f || m_run == -INFINITY);
        const float m_new = grow ? mt2 : m_run;
        const bool resc = grow && l > 0.f;
        if (__any_sync(0xffffffffu, resc)) {
          if (!o_quiet()) {
            ok = false;
            break;
          }
          const float alpha = resc ? fast_exp2(m_run - m_new) : 1.f;
          for (int c0 = 0; c0 < DV; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(o_addr + c0, ov);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; x++) ov[x] = __float_as_uint(__uint_as_float(ov[x]) * alpha);
            tmem_st32(o_addr + c0, ov);
          }
          l *= alpha;
        }
        m_run = m_new;
        for (int c0 = 0; c0 < p.kvb; c0 += 16) {
          uint32_t v[16];
          tmem_ld16(s_addr + c0, v);
          tmem_wait_ld();
          uint32_t pk[8];
#pragma unroll
          for (int x = 0; x < 16; x += 2) {
            float p0 = 0.f, p1 = 0.f;
            if (act && c0 + x >= lo && c0 + x < hi)
              p0 = fast_exp2(fmaf(__uint_as_float(v[x]), c, -m_run));
            if (act && c0 + x + 1 >= lo && c0 + x + 1 < hi)
              p1 = fast_exp2(fmaf(__uint_as_float(v[x + 1]), c, -m_run));
            l += p0 + p1;
            pk[x >> 1] = pack2(p0, p1, p.fmt);
          }
          tmem_st8(s_addr + (c0 >> 1), pk);
        }
      } else {
        uint32_t z[8];
#pragma unroll
        for (int x = 0; x < 8; x++) z[x] = 0u;
        for (int c0 = 0; c0 < p.kvb; c0 += 16) tmem_st8(s_addr + (c0 >> 1), z);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull(sbuf));
    }

    // ------------------------------------------------------------ epilogue
    // merge the two groups' partial softmax states, then each group converts
    // and stores one half of the head dimension
    s_m[grp_w][r] = m_run;
    s_l[grp_w][r] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (ok && n > 0) ok = mbar_wait(bar_final, 0, w, FTK_DEV_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      const float ma = s_m[0][r], mb = s_m[1][r];
      const float la = s_l[0][r], lb = s_l[1][r];
      const float mm = fmaxf(ma, mb);
      const float fa = la > 0.f ? fast_exp2(ma - mm) : 0.f;
      const float fb = lb > 0.f ? fast_exp2(mb - mm) : 0.f;
      const float lt = la * fa + lb * fb;
      const bool have = (n > 0) && lt > 0.f;
      const float inv = have ? 1.f / lt : 0.f;
      const float wa = fa * inv, wb = fb * inv;
      uint8_t* orow = nullptr;
      if (row_valid)
        orow = static_cast<uint8_t*>(p.o) +
               2 * (static_cast<int64_t>(b_idx) * p.so_b + static_cast<int64_t>(qrow) * p.so_n +
                    static_cast<int64_t>(h_idx) * p.so_h + p.v_off);
      constexpr int HALF = DV / 2;
      for (int c0 = grp_w * HALF; c0 < (grp_w + 1) * HALF; c0 += 32) {
        uint32_t va[32], vb[32];
        if (n > 0) tmem_ld32(lane_addr + FW_COL_O + c0, va);
        if (!SINGLE && n > 1) tmem_ld32(lane_addr + FW_COL_O + 128 + c0, vb);
        if (n > 0) tmem_wait_ld();
        if (row_valid) {
          uint32_t pk[16];
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float a = 0.f, b = 0.f;
            if (have) {
              a = __uint_as_float(va[x]) * wa;
              b = __uint_as_float(va[x + 1]) * wa;
              if (!SINGLE && n > 1) {
                a = fmaf(__uint_as_float(vb[x]), wb, a);
                b = fmaf(__uint_as_float(vb[x + 1]), wb, b);
              }
            }
            pk[x >> 1] = pack2(a, b, p.fmt);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
          for (int x = 0; x < 4; x++)
            dst[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
        }
      }
      if (row_valid && grp_w == 0)
        p.lse[static_cast<int64_t>(bh) * p.N + qrow] =
            have ? (mm + log2f(lt)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag)
    for (int i = 0; i < 200; i++) __nanosleep(1000);
  if (warp == 0) tmem_dealloc(tmem, 512);
}

}  // namespace ftk

#include "sparse_fwd_pipe.cuh"
#include "sparse_fwd_pipe2.cuh"

namespace ftk {

template <int D, int FMT>
static int launch_fwd_pipe(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const FwdParams& p, int64_t BH, cudaStream_t st) {
  constexpr int NCH = D / 64;
  const size_t smem = 1024 + NCH * 128 * 128 +
                      static_cast<size_t>(FP_KST + FP_VST) * NCH * 64 * 128;
  if (cudaFuncSetAttribute(sparse_fwd_pipe_kernel<D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return FTK_ERR_CUDA;
  dim3 grid((p.QM + p.G - 1) / p.G, static_cast<unsigned>(BH));
  sparse_fwd_pipe_kernel<D, FMT><<<grid, FP_THREADS, smem, st>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

template <int D, int DV = D>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      FwdParams p, int64_t BH, cudaStream_t st) {
  constexpr int NCH = D / 64, NCV = DV / 64;
  const int stage_bytes = (NCH + NCV) * p.kvb * 128;
  // 227 KB per CTA less the static part (union scratch, softmax state: ~19 KB) and the Q tile
  const int ring_bytes = (227 - 21) * 1024 - NCH * 128 * 128;
  int nst = std::min(FW_MAX_STAGES, std::min(168 * 1024, ring_bytes) / stage_bytes);
  if (nst < 2) return FTK_ERR_UNSUPPORTED;
  p.nstages = nst;
  const size_t smem = 1024 + NCH * 128 * 128 + static_cast<size_t>(nst) * stage_bytes;
  if (cudaFuncSetAttribute(sparse_fwd_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return FTK_ERR_CUDA;
  dim3 grid((p.QM + p.G - 1) / p.G, static_cast<unsigned>(BH));
  for (int v_off = 0; v_off < D; v_off += DV) {
    p.v_off = v_off;
    sparse_fwd_kernel<D, DV><<<grid, FW_THREADS, smem, st>>>(tq, tk, tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

}  // namespace ftk

using namespace ftk;

// One redo word per CTA of the pipelined kernel.
extern "C" size_t ftk_sparse_fwd_workspace(int64_t B, int64_t H, int QM, int q_block_size) {
  if (B <= 0 || H <= 0 || QM <= 0 || q_block_size <= 0) return 0;
  const int G = std::max(1, std::min(AT_MAX_GROUPS, 128 / q_block_size));
  return static_cast<size_t>(B * H) * ((QM + G - 1) / G) * sizeof(int32_t);
}

extern "C" int ftk_sparse_fwd(const void* q, const void* k, const void* v, int dtype, int64_t B,
                              int64_t H, int64_t Hkv, int64_t N, int64_t D, int64_t sq_b, int64_t sq_n,
                              int64_t sq_h, int64_t sk_b, int64_t sk_n, int64_t sk_h, int64_t sv_b,
                              int64_t sv_n, int64_t sv_h, const int32_t* merged_idx, int QM, int W,
                              int q_block_size, int kv_block_size, int q_pad_head, int kv_pad_head,
                              float scale, void* o, int64_t so_b, int64_t so_n, int64_t so_h,
                              float* lse, void* workspace, size_t workspace_bytes,
                              int32_t* status, void* stream) {
  if (!q || !k || !v || !merged_idx || !o || !lse) return FTK_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || N <= 0 || QM <= 0 || W <= 0) return FTK_ERR_BAD_ARG;
  if (dtype != FTK_DTYPE_F16 && dtype != FTK_DTYPE_BF16) return FTK_ERR_BAD_ARG;
  if (Hkv <= 0) Hkv = H;
  if (H % Hkv != 0) return FTK_ERR_BAD_ARG;
  if (q_block_size <= 0 || kv_block_size <= 0) return FTK_ERR_BAD_ARG;
  if (q_pad_head < 0 || q_pad_head >= q_block_size || kv_pad_head < 0 ||
      kv_pad_head >= kv_block_size)
    return FTK_ERR_BAD_ARG;
  if (static_cast<int64_t>(QM) * q_block_size < q_pad_head + N) return FTK_ERR_BAD_ARG;
  if (D != 64 && D != 128 && D != 256) return FTK_ERR_UNSUPPORTED;
  if (q_block_size > 128) return FTK_ERR_UNSUPPORTED;
  if (kv_block_size % 16 != 0 || kv_block_size > 128) return FTK_ERR_UNSUPPORTED;
  const int64_t Mkv = (kv_pad_head + N + kv_block_size - 1) / kv_block_size;
  if (Mkv > AT_MAX_BLOCKS) return FTK_ERR_UNSUPPORTED;
  if (B * H > 65535) return FTK_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(o) & 15u) || (so_b & 7) || (so_n & 7) || (so_h & 7))
    return FTK_ERR_BAD_ARG;

  FwdParams p{};
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
  p.scale_log2 = scale * 1.4426950408889634f;
  p.merged = merged_idx;
  p.o = o;
  p.so_b = so_b;
  p.so_n = so_n;
  p.so_h = so_h;
  p.lse = lse;
  p.status = status;
  p.kv_hdiv = static_cast<int>(H / Hkv);

  CUtensorMap tq, tk, tv;
  int e = encode_tmap_bnhd(&tq, q, dtype, B, N, H, D, sq_b, sq_n, sq_h, 64, 128);
  if (e) return e;
  e = encode_tmap_bnhd(&tk, k, dtype, B, N, Hkv, D, sk_b, sk_n, sk_h, 64, kv_block_size);
  if (e) return e;
  e = encode_tmap_bnhd(&tv, v, dtype, B, N, Hkv, D, sv_b, sv_n, sv_h, 64, kv_block_size);
  if (e) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 64-row kv blocks, q blocks of 64 or 32 rows and a workspace: the
  // pipelined kernel runs first and the exact kernel redoes the CTAs it flags.
  const char* env = getenv("FTK_FWD_PIPE");
  const bool pipe = D <= 128 && kv_block_size == 64 && (q_block_size == 64 || q_block_size == 32) && workspace &&
                    workspace_bytes >= ftk_sparse_fwd_workspace(B, H, QM, q_block_size) &&
                    !(env && env[0] == '0');
  if (pipe) {
    p.redo_out = static_cast<int*>(workspace);
    const char* env2 = getenv("FTK_FWD_2CTA");
    // Pairs walk the union of four lists: worth it when the lists can cover a
    // good part of the blocks (then the unions of two and of four are about
    // the same length); short lists keep the one-CTA kernel's unions of two.
    if (D == 128 && q_block_size == 64 && 4 * static_cast<int64_t>(W) >= Mkv &&
        !(env2 && env2[0] == '0')) {
      // head dim 128: the same kernel on pairs of SMs
      CUtensorMap tk32;
      e = encode_tmap_bnhd(&tk32, k, dtype, B, N, Hkv, D, sk_b, sk_n, sk_h, 64, 32);
      if (e) return e;
      const size_t smem2 = 1024 + 2 * 128 * 128 + static_cast<size_t>(FP2_KST + FP2_VST) * 8192;
      dim3 grid2(2 * ((QM + 3) / 4), static_cast<unsigned>(B * H));
      if (dtype == FTK_DTYPE_BF16) {
        if (cudaFuncSetAttribute(sparse_fwd_pipe2_kernel<1>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem2)) != cudaSuccess)
          return FTK_ERR_CUDA;
        sparse_fwd_pipe2_kernel<1><<<grid2, FP_THREADS, smem2, st>>>(tq, tk32, tv, p);
      } else {
        if (cudaFuncSetAttribute(sparse_fwd_pipe2_kernel<0>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem2)) != cudaSuccess)
          return FTK_ERR_CUDA;
        sparse_fwd_pipe2_kernel<0><<<grid2, FP_THREADS, smem2, st>>>(tq, tk32, tv, p);
      }
      e = cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
    } else if (dtype == FTK_DTYPE_BF16) {
      e = (D == 64) ? launch_fwd_pipe<64, 1>(tq, tk, tv, p, B * H, st)
                    : launch_fwd_pipe<128, 1>(tq, tk, tv, p, B * H, st);
    } else {
      e = (D == 64) ? launch_fwd_pipe<64, 0>(tq, tk, tv, p, B * H, st)
                    : launch_fwd_pipe<128, 0>(tq, tk, tv, p, B * H, st);
    }
    if (e) return e;
    p.redo_out = nullptr;
    p.redo_in = static_cast<const int*>(workspace);
  }
  if (D == 64) return launch_fwd<64>(tq, tk, tv, p, B * H, st);
  if (D == 256) return launch_fwd<256, 256>(tq, tk, tv, p, B * H, st);
  return launch_fwd<128>(tq, tk, tv, p, B * H, st);
}
