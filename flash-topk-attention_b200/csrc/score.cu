// Block scoring for sm_100a: dense Q.K^T on tcgen05 with TMEM accumulators,
// K tiles staged by TMA, softmax mass accumulated per score block.
//
// Replaces block_score_kernel / block_normalize_kernel of the reference
// (flash_topk_attn_v2/csrc/block_score_kernel.cu:19-314).
//
// One CTA owns 256 query rows of one (batch, head) slice and streams every
// key tile once.  Roles: warp 0 = TMA producer, warp 1 = UMMA issuer, warps
// 2..17 = two groups of 256 softmax threads, one query row each (TMEM lane ==
// row).  Two 128x128 fp32 accumulators per stage (rows 0-127 / 128-255 share
// the K tile), two stages: 4 x 128 = 512 TMEM columns.  Group s drains stage
// s, so the groups work concurrently on consecutive tiles while the tensor
// core refills whichever accumulator was handed back.
//
// Softmax is single pass against a fixed per-row reference exponent `mref`
// (an integer in log2 units): sum_j[t] = sum_{i in block j} 2^(c*s_ti - mref),
// L[t] = sum_j sum_j[t]; the block score is sum_j / L.  mref comes from the
// row maximum over the first key tile (mode 0).  Should any later logit
// exceed it by more than the fp32 exponent range the row total overflows;
// the kernel then raises `*fallback` and the launcher's two follow-up
// launches (mode 1: exact row maximum, mode 2: sums against it) redo the work.
// They return at once when the flag is clear.
#include <algorithm>
#include <cmath>
#include <cstdlib>

#include "ftk_host.cuh"
#include "ftk_sm100.cuh"

namespace ftk {

constexpr int SC_QROWS = 256;      // query rows per CTA
constexpr int SC_KT = 128;         // key rows per tile (UMMA N)
constexpr int SC_STAGES = 4;       // K tile ring depth
constexpr int SC_THREADS = 576;    // 2 + 2 x 8 warps
constexpr int SC_CHUNK_BYTES = 128 * 128;  // 128 rows x 64 16-bit elements
__host__ __device__ constexpr int score_ksplit(int d) { return d > 128 ? 2 : 1; }
__host__ __device__ constexpr int score_stages(int d) { return d > 128 ? 2 : SC_STAGES; }

struct ScoreParams {
  int N, M, D;
  int bsz, pad_head;          // score block size, virtual head padding
  int tile_rows;              // rows fetched per K tile (TMA box rows)
  int blocks_per_tile;        // bsz <= 128: whole blocks per tile, else 0
  int tiles_per_block;        // bsz > 128: tiles per block, else 0
  int num_tiles;
  int fmt;                    // 0 fp16, 1 bf16
  int mode;                   // 0 first-tile reference, 1 row max only, 2 given reference
  int H, bh_begin;
  float scale_log2;           // log2(e) * softmax scale
  float* sums;                // [bh_count][N][M]   unnormalised block sums
  float* row_total;           // [bh_count][N]      L
  float* row_max;             // [bh_count][N]      raw-logit row maximum (modes 1, 2)
  int* fallback;              // device flag
  int* status;
};

struct TileInfo {
  int row0;     // first key token of the tile (may be negative)
  int used;     // accumulator columns that belong to score blocks
  int block0;   // score block of column 0
  int col_in_block0;  // position of column 0 inside that block
};

__device__ __forceinline__ TileInfo tile_info(const ScoreParams& p, int t) {
  TileInfo ti;
  if (p.blocks_per_tile > 0) {
    ti.block0 = t * p.blocks_per_tile;
    int nb = min(p.blocks_per_tile, p.M - ti.block0);
    ti.row0 = ti.block0 * p.bsz - p.pad_head;
    ti.used = nb * p.bsz;
    ti.col_in_block0 = 0;
  } else {
    int j = t / p.tiles_per_block, part = t - j * p.tiles_per_block;
    ti.block0 = j;
    ti.row0 = j * p.bsz - p.pad_head + part * SC_KT;
    ti.used = min(SC_KT, p.bsz - part * SC_KT);
    ti.col_in_block0 = part * SC_KT;
  }
  return ti;
}

// Which softmax group drains tile t.  Tiles alternate between the two groups,
// each group bound to one accumulator stage, so a group meets every phase of
// its stage's barriers in order (a one-bit parity wait must never skip a
// phase).  When a score block spans several tiles (block size > 128) one
// thread has to see all of them, and group 0 takes every tile.
__device__ __forceinline__ int tile_owner(const ScoreParams& p, int t) {
  return p.tiles_per_block > 1 ? 0 : (t & 1);
}

template <int D>
__global__ void __launch_bounds__(SC_THREADS, 1)
score_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
             const ScoreParams p) {
  constexpr int NCH = D / 64;                       // 128-byte chunks per row
  constexpr int Q_BYTES = 2 * NCH * SC_CHUNK_BYTES; // 256 rows
  // Head dims above 128: a K tile travels as KSPLIT slices of the head dim,
  // one ring stage each (the 256-row Q tile leaves room for two 32 KB stages),
  // and the tile's UMMAs accumulate over the slices.
  constexpr int KSPLIT = score_ksplit(D);
  constexpr int NCHS = NCH / KSPLIT;                // chunks per stage
  constexpr int NSTG = score_stages(D);
  constexpr int K_STAGE_BYTES = NCHS * SC_CHUNK_BYTES;

  if (p.mode != 0 && *p.fallback == 0) return;  // uniform: follow-up launches idle

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Q_BYTES;
  __shared__ __align__(8) uint64_t bars[1 + 2 * SC_STAGES + 8 + 2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ float s_mref[SC_QROWS];   // group 0 -> group 1: reference exponent
  __shared__ float s_part[SC_QROWS];   // group 1 -> group 0: partial total / maximum

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = blockIdx.x * SC_QROWS;
  const int bh_local = blockIdx.y;
  const int bh = p.bh_begin + bh_local;
  const int b_idx = bh / p.H, h_idx = bh - b_idx * p.H;

  const uint32_t bar_q = smem_u32(&bars[0]);
  auto bar_kfull = [&](int s) { return smem_u32(&bars[1 + s]); };
  auto bar_kempty = [&](int s) { return smem_u32(&bars[1 + SC_STAGES + s]); };
  // one full / empty pair per accumulator (stage s, row half h): the four
  // warps that drain an accumulator start as soon as its 8 UMMAs retire and
  // hand it back on their own
  auto bar_afull = [&](int s, int h) { return smem_u32(&bars[1 + 2 * SC_STAGES + s * 2 + h]); };
  auto bar_aempty = [&](int s, int h) {
    return smem_u32(&bars[1 + 2 * SC_STAGES + 4 + s * 2 + h]);
  };
  const uint32_t bar_mref = smem_u32(&bars[1 + 2 * SC_STAGES + 8]);
  const uint32_t bar_part = smem_u32(&bars[1 + 2 * SC_STAGES + 9]);

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < SC_STAGES; s++) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
    }
    for (int s = 0; s < 2; s++)
      for (int h = 0; h < 2; h++) {
        mbar_init(bar_afull(s, h), 1);
        mbar_init(bar_aempty(s, h), 4);  // one arrival per warp draining the accumulator
      }
    mbar_init(bar_mref, 8);
    mbar_init(bar_part, 8);
    mbar_init_fence();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  WaitCtx w{&abort_flag, p.status};
  const int T = p.num_tiles;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar_q, Q_BYTES);
      for (int half = 0; half < 2; half++)
        for (int c = 0; c < NCH; c++)
          tma_load_4d(smem_u32(sQ) + (half * NCH + c) * SC_CHUNK_BYTES, &tm_q, bar_q, c * 64,
                      h_idx, q0 + half * 128, b_idx);
      const uint32_t tile_bytes = static_cast<uint32_t>(p.tile_rows) * 128u * NCHS;
      for (int u = 0; u < T * KSPLIT; u++) {
        const int s = u % NSTG;
        const uint32_t ph = (u / NSTG) & 1;
        if (!mbar_wait(bar_kempty(s), ph ^ 1, w, FTK_DEV_TIMEOUT_TMA)) break;
        const int t = u / KSPLIT, part = u % KSPLIT;
        const TileInfo ti = tile_info(p, t);
        mbar_expect_tx(bar_kfull(s), tile_bytes);
        for (int c = 0; c < NCHS; c++)
          tma_load_4d(smem_u32(sK) + s * K_STAGE_BYTES + c * SC_CHUNK_BYTES, &tm_k, bar_kfull(s),
                      (part * NCHS + c) * 64, h_idx, ti.row0, b_idx);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- UMMA issuer
    {
      // the whole warp runs this path; one elected lane issues the UMMAs
      const uint32_t idesc = umma_idesc(128, SC_KT, p.fmt, 0, 0);
      const uint64_t qdesc0 = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t kdesc0 = smem_desc_sw128(smem_u32(sK), 16, 1024);
      bool ok = mbar_wait(bar_q, 0, w, FTK_DEV_TIMEOUT_MMA);
      for (int t = 0; ok && t < T; t++) {
        const int u0 = t * KSPLIT;
        const int a = t & 1;
        const uint32_t pa = (t >> 1) & 1;
        // the three barriers of a tile are waited for together (a test of a
        // completed barrier still takes ~110 cycles) and the tile's UMMAs go
        // out as one batch, so the tensor core is not left idle in between
        const uint32_t wb[3] = {bar_kfull(u0 % NSTG), bar_aempty(a, 0), bar_aempty(a, 1)};
        const uint32_t wp[3] = {static_cast<uint32_t>((u0 / NSTG) & 1), pa ^ 1, pa ^ 1};
        if (!mbar_wait_all<3>(wb, wp, w, FTK_DEV_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int part = 0; part < KSPLIT; part++) {
          const int s = (u0 + part) % NSTG;
          if (part > 0) {
            if (!mbar_wait(bar_kfull(s), ((u0 + part) / NSTG) & 1, w, FTK_DEV_TIMEOUT_MMA)) {
              ok = false;
              break;
            }
            tc_fence_after();
          }
          const uint64_t kdesc = desc_advance(kdesc0, s * K_STAGE_BYTES);
          if (elect_one()) {
#pragma unroll
            for (int half = 0; half < 2; half++) {
              const uint32_t d_tmem = tmem + static_cast<uint32_t>((a * 2 + half) * SC_KT);
              const uint64_t qdesc =
                  desc_advance(qdesc0, (half * NCH + part * NCHS) * SC_CHUNK_BYTES);
#pragma unroll
              for (int ks = 0; ks < D / KSPLIT / 16; ks++) {
                const uint32_t off = (ks / 4) * SC_CHUNK_BYTES + (ks % 4) * 32;
                umma_ss(d_tmem, desc_advance(qdesc, off), desc_advance(kdesc, off), idesc,
                        part > 0 || ks > 0);
              }
              if (half == 1) umma_commit(bar_kempty(s));  // smem stage reusable once retired
              // this accumulator is readable
              if (part == KSPLIT - 1) umma_commit(bar_afull(a, half));
            }
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ---------------------------------------------------- softmax threads
    // Two groups of 8 warps.  Each tile is drained by exactly one group (see
    // tile_owner) so both groups run concurrently on consecutive tiles and
    // hide each other's TMEM-load and barrier latency.
    const int cw = warp - 2;               // 0..15
    const int group = cw >> 3;
    const int half = (cw >> 2) & 1;        // which 128-row accumulator
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int row_in_cta = half * 128 + quarter * 32 + lane;
    const int row = q0 + row_in_cta;
    const bool row_ok = row < p.N;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const size_t row_off = (static_cast<size_t>(bh_local) * p.N + (row_ok ? row : 0));
    float* out_row = p.sums + row_off * p.M;
    const float c = p.scale_log2;

    float mref = 0.f;
    float run_max = -INFINITY;
    float total = 0.f;
    bool ok = true;

    if (p.mode == 2) mref = ceilf(p.row_max[row_off] * c);

    if (p.mode == 0) {
      if (group == 0) {
        // reference exponent from the row maximum over the first key tile
        ok = mbar_wait(bar_afull(0, half), 0, w, FTK_DEV_TIMEOUT_CONSUMER);
        if (ok) {
          tc_fence_after();
          const TileInfo ti = tile_info(p, 0);
          const int lo = max(0, -ti.row0), hi = min(ti.used, p.N - ti.row0);
          float mx = -INFINITY;
          for (int c0 = 0; c0 < ti.used; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(lane_addr + static_cast<uint32_t>(half * SC_KT + c0), r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const int col = c0 + i;
              if (col >= lo && col < hi) mx = fmaxf(mx, __uint_as_float(r[i]));
            }
          }
          mref = ceilf(mx * c);
          if (!(fabsf(mref) < 1e30f)) mref = 0.f;
        }
        s_mref[row_in_cta] = mref;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_mref);
      } else {
        ok = mbar_wait(bar_mref, 0, w, FTK_DEV_TIMEOUT_CONSUMER);
        mref = s_mref[row_in_cta];
      }
    }

    float acc = 0.f;
    int j = 0, col_in_block = 0;
    for (int t = 0; ok && t < T; t++) {
      if (tile_owner(p, t) != group) continue;
      const int a = t & 1;
      const uint32_t pa = (t >> 1) & 1;
      if (!mbar_wait(bar_afull(a, half), pa, w, FTK_DEV_TIMEOUT_CONSUMER)) { ok = false; break; }
      tc_fence_after();
      const TileInfo ti = tile_info(p, t);
      const int lo = max(0, -ti.row0), hi = min(ti.used, p.N - ti.row0);
      const bool full = (lo == 0 && hi == ti.used);
      if (ti.col_in_block0 == 0) { j = ti.block0; col_in_block = 0; }
      const uint32_t acc_addr = lane_addr + static_cast<uint32_t>((a * 2 + half) * SC_KT);
      // one 32-column chunk: two 16-column halves, block sums flushed on the
      // 16-column grid (block sizes are multiples of 16)
      auto process = [&](const uint32_t (&r)[32], int c0) {
#pragma unroll
        for (int hc = 0; hc < 2; hc++) {
          const int cb = c0 + hc * 16;
          if (cb < ti.used) {
            if (p.mode == 1) {
#pragma unroll
              for (int i = 0; i < 16; i++) {
                const int col = cb + i;
                if (full || (col >= lo && col < hi))
                  run_max = fmaxf(run_max, __uint_as_float(r[hc * 16 + i]));
              }
            } else {
              float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
              if (full) {
                // two columns per instruction for the scaling (fma.f32x2) and for the
                // running sums (add.f32x2): 2 issue slots per logit instead of 3; the four
                // partial sums are the same additions in the same order as scalar code
                float2 s01 = make_float2(0.f, 0.f), s23 = make_float2(0.f, 0.f);
                const float2 c2 = make_float2(c, c), nm2 = make_float2(-mref, -mref);
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                  const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[hc * 16 + i + 0]),
                                                          __uint_as_float(r[hc * 16 + i + 1])),
                                              c2, nm2);
                  const float2 y = __ffma2_rn(make_float2(__uint_as_float(r[hc * 16 + i + 2]),
                                                          __uint_as_float(r[hc * 16 + i + 3])),
                                              c2, nm2);
                  s01 = __fadd2_rn(s01, make_float2(fast_exp2(x.x), fast_exp2(x.y)));
                  s23 = __fadd2_rn(s23, make_float2(fast_exp2(y.x), fast_exp2(y.y)));
                }
                a0 = s01.x;
                a1 = s01.y;
                a2 = s23.x;
                a3 = s23.y;
              } else {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                  const int col = cb + i;
                  if (col >= lo && col < hi)
                    a0 += fast_exp2(fmaf(__uint_as_float(r[hc * 16 + i]), c, -mref));
                }
              }
              acc += (a0 + a1) + (a2 + a3);
              col_in_block += 16;
              if (col_in_block == p.bsz) {
                if (row_ok) out_row[j] = acc;
                total += acc;
                acc = 0.f;
                col_in_block = 0;
                j++;
              }
            }
          }
        }
      };
      auto release = [&]() {
        // the tile's last chunk is in registers: hand the accumulator back
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_aempty(a, half));
      };
      if (ti.used == SC_KT) {
        // full tile: the load of chunk k+1 is in flight while chunk k is summed
        uint32_t ra[32], rb[32];
        tmem_ld32(acc_addr, ra);
        tmem_wait_ld();
        tmem_ld32(acc_addr + 32, rb);
        process(ra, 0);
        tmem_wait_ld();
        tmem_ld32(acc_addr + 64, ra);
        process(rb, 32);
        tmem_wait_ld();
        tmem_ld32(acc_addr + 96, rb);
        process(ra, 64);
        tmem_wait_ld();
        release();
        process(rb, 96);
      } else {
        for (int c0 = 0; c0 < ti.used; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(acc_addr + static_cast<uint32_t>(c0), r);
          tmem_wait_ld();
          if (c0 + 32 >= ti.used) release();
          process(r, c0);
        }
      }
    }
    // combine the two groups' partial results per row: group 1 publishes,
    // group 0 adds (total) or takes the larger (maximum) and writes
    const float mine = (p.mode == 1) ? run_max : total;
    if (group == 1) {
      s_part[row_in_cta] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_part);
    } else {
      if (ok) ok = mbar_wait(bar_part, 0, w, FTK_DEV_TIMEOUT_CONSUMER);
      if (ok && row_ok) {
        const float other = s_part[row_in_cta];
        if (p.mode == 1) {
          p.row_max[row_off] = fmaxf(mine, other);
        } else {
          const float tot = mine + other;
          p.row_total[row_off] = tot;
          if (!(tot > 0.f && tot < 3.0e38f)) atomicExch(p.fallback, 1);
        }
      }
    }
  }

  // ------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // give copies still in flight time to land before the smem is released
    for (int i = 0; i < 200; i++) __nanosleep(1000);
  }
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// block_scores[r][j] = sums[r][j] / total[r]
__global__ void score_normalize_kernel(const float* __restrict__ sums,
                                       const float* __restrict__ total, float* __restrict__ out,
                                       int64_t rows, int M) {
  const int64_t n = rows * M;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / M;
    out[i] = sums[i] * __frcp_rn(total[r]);  // same arithmetic as the fused select path
  }
}

template <int D>
static int launch_score_d(const CUtensorMap& tq, const CUtensorMap& tk, ScoreParams p,
                          int64_t bh_count, cudaStream_t st) {
  constexpr int NCH = D / 64;
  const size_t smem =
      1024 + (2 * NCH + score_stages(D) * (NCH / score_ksplit(D))) * SC_CHUNK_BYTES;
  if (cudaFuncSetAttribute(score_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return FTK_ERR_CUDA;
  dim3 grid((p.N + SC_QROWS - 1) / SC_QROWS, static_cast<unsigned>(bh_count));
  for (int mode = 0; mode < 3; mode++) {
    p.mode = mode;
    score_kernel<D><<<grid, SC_THREADS, smem, st>>>(tq, tk, p);
    if (cudaGetLastError() != cudaSuccess) return FTK_ERR_CUDA;
  }
  return FTK_OK;
}

struct ScoreWs {
  float* row_total;
  float* row_max;
  int* fallback;
  float* sums;
};

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

static size_t score_ws_layout(int64_t bh_count, int64_t N, int64_t M, bool with_sums, char* base,
                              ScoreWs* ws) {
  size_t off = 0;
  const size_t rows = static_cast<size_t>(bh_count) * N;
  if (ws) ws->fallback = reinterpret_cast<int*>(base + off);
  off += 256;
  if (ws) ws->row_total = reinterpret_cast<float*>(base + off);
  off += align256(rows * 4);
  if (ws) ws->row_max = reinterpret_cast<float*>(base + off);
  off += align256(rows * 4);
  if (ws) ws->sums = reinterpret_cast<float*>(base + off);
  if (with_sums) off += align256(rows * static_cast<size_t>(M) * 4);
  return off;
}

// Validates arguments, encodes the tensor maps and launches the three score
// passes; sums go to `sums` ([bh_count][N][M]).
static int run_score(const void* q, const void* k, int dtype, int64_t B, int64_t H, int64_t N,
                     int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h, int64_t sk_b,
                     int64_t sk_n, int64_t sk_h, int64_t bh_begin, int64_t bh_count, int bsz,
                     int pad_head, int pad_tail, float scale, float* sums, const ScoreWs& ws,
                     int32_t* status, cudaStream_t st) {
  if (!q || !k || B <= 0 || H <= 0 || N <= 0 || bsz <= 0 || !(scale > 0.f))
    return FTK_ERR_BAD_ARG;
  if (dtype != FTK_DTYPE_F16 && dtype != FTK_DTYPE_BF16) return FTK_ERR_BAD_ARG;
  if (pad_head < 0 || pad_tail < 0 || pad_head >= bsz || pad_tail >= bsz) return FTK_ERR_BAD_ARG;
  if ((pad_head + N + pad_tail) % bsz != 0) return FTK_ERR_BAD_ARG;
  if (bh_begin < 0 || bh_count <= 0 || bh_begin + bh_count > B * H) return FTK_ERR_BAD_ARG;
  if (D != 64 && D != 128 && D != 256) return FTK_ERR_UNSUPPORTED;
  if (bsz % 16 != 0) return FTK_ERR_UNSUPPORTED;
  if (bh_count > 65535) return FTK_ERR_BAD_ARG;

  ScoreParams p{};
  p.N = static_cast<int>(N);
  p.M = static_cast<int>((pad_head + N + pad_tail) / bsz);
  p.D = static_cast<int>(D);
  p.bsz = bsz;
  p.pad_head = pad_head;
  if (bsz <= SC_KT) {
    p.blocks_per_tile = SC_KT / bsz;
    p.tiles_per_block = 0;
    p.tile_rows = p.blocks_per_tile * bsz;
    p.num_tiles = (p.M + p.blocks_per_tile - 1) / p.blocks_per_tile;
  } else {
    p.blocks_per_tile = 0;
    p.tiles_per_block = (bsz + SC_KT - 1) / SC_KT;
    p.tile_rows = SC_KT;
    p.num_tiles = p.M * p.tiles_per_block;
  }
  p.fmt = dtype;
  p.H = static_cast<int>(H);
  p.bh_begin = static_cast<int>(bh_begin);
  p.scale_log2 = static_cast<float>(1.4426950408889634 * static_cast<double>(scale));
  p.sums = sums;
  p.row_total = ws.row_total;
  p.row_max = ws.row_max;
  p.fallback = ws.fallback;
  p.status = status;

  CUtensorMap tq, tk;
  int e = encode_tmap_bnhd(&tq, q, dtype, B, N, H, D, sq_b, sq_n, sq_h, 64, 128);
  if (e) return e;
  e = encode_tmap_bnhd(&tk, k, dtype, B, N, H, D, sk_b, sk_n, sk_h, 64, p.tile_rows);
  if (e) return e;
  if (cudaMemsetAsync(ws.fallback, 0, 4, st) != cudaSuccess) return FTK_ERR_CUDA;
  if (D == 64) return launch_score_d<64>(tq, tk, p, bh_count, st);
  if (D == 256) return launch_score_d<256>(tq, tk, p, bh_count, st);
  return launch_score_d<128>(tq, tk, p, bh_count, st);
}

int select_launch(const float* block_scores, const float* row_scale, int64_t rows, int M,
                  int max_topk, int bsz, int pad_head, int pad_tail, float threshold,
                  int32_t* topk_idx, float* topk_raw, float* topk_avg, cudaStream_t st);

}  // namespace ftk

using namespace ftk;

extern "C" size_t ftk_block_score_workspace(int64_t bh_count, int64_t N) {
  return score_ws_layout(bh_count, N, 0, false, nullptr, nullptr);
}

extern "C" int ftk_block_score(const void* q, const void* k, int dtype, int64_t B, int64_t H,
                               int64_t N, int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h,
                               int64_t sk_b, int64_t sk_n, int64_t sk_h, int64_t bh_begin,
                               int64_t bh_count, int score_block_size, int pad_head, int pad_tail,
                               float scale, float* block_scores, void* workspace,
                               size_t workspace_bytes,
                               int32_t* status, void* stream) {
  if (!block_scores) return FTK_ERR_BAD_ARG;
  if (bh_count <= 0 || N <= 0) return FTK_ERR_BAD_ARG;
  if (!workspace || workspace_bytes < ftk_block_score_workspace(bh_count, N))
    return FTK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return FTK_ERR_BAD_ARG;
  ScoreWs ws;
  score_ws_layout(bh_count, N, 0, false, static_cast<char*>(workspace), &ws);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int e = run_score(q, k, dtype, B, H, N, D, sq_b, sq_n, sq_h, sk_b, sk_n, sk_h, bh_begin,
                    bh_count, score_block_size, pad_head, pad_tail, scale, block_scores, ws, status,
                    st);
  if (e) return e;
  const int M = static_cast<int>((pad_head + N + pad_tail) / score_block_size);
  const int64_t rows = bh_count * N;
  const int grid = static_cast<int>(std::min<int64_t>((rows * M + 255) / 256, 148 * 16));
  score_normalize_kernel<<<grid, 256, 0, st>>>(block_scores, ws.row_total, block_scores, rows, M);
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" size_t ftk_score_topk_workspace(int64_t bh_count, int64_t N, int64_t M) {
  return score_ws_layout(bh_count, N, M, true, nullptr, nullptr);
}

extern "C" int ftk_score_topk(const void* q, const void* k, int dtype, int64_t B, int64_t H,
                              int64_t N, int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h,
                              int64_t sk_b, int64_t sk_n, int64_t sk_h, int64_t bh_begin,
                              int64_t bh_count, int score_block_size, int pad_head, int pad_tail,
                              float scale, int topk, float threshold, int32_t* topk_idx, float* topk_raw,
                              float* topk_avg, void* workspace, size_t workspace_bytes,
                              int32_t* status, void* stream) {
  if (!topk_idx || !topk_raw || !topk_avg || topk < 0) return FTK_ERR_BAD_ARG;
  if (bh_count <= 0 || N <= 0 || score_block_size <= 0) return FTK_ERR_BAD_ARG;
  const int64_t M = (pad_head + N + pad_tail) / score_block_size;
  if (M > 4096) return FTK_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < ftk_score_topk_workspace(bh_count, N, M))
    return FTK_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return FTK_ERR_BAD_ARG;
  ScoreWs ws;
  score_ws_layout(bh_count, N, M, true, static_cast<char*>(workspace), &ws);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int e = run_score(q, k, dtype, B, H, N, D, sq_b, sq_n, sq_h, sk_b, sk_n, sk_h, bh_begin,
                    bh_count, score_block_size, pad_head, pad_tail, scale, ws.sums, ws, status, st);
  if (e) return e;
  return select_launch(ws.sums, ws.row_total, bh_count * N, static_cast<int>(M), topk,
                       score_block_size, pad_head, pad_tail, threshold, topk_idx, topk_raw,
                       topk_avg, st);
}
