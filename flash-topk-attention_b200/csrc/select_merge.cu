// HBM-bound integer / fp32 kernels of the path: top-k select, q-block merge,
// reverse index, count sort.  No tensor cores here; the rules that matter are
// coalesced row reads, warp-level reductions and a fixed summation order so
// that every result is reproducible bit for bit.
#include <algorithm>

#include "ftk_host.cuh"
#include "ftk_sm100.cuh"
#include "select_row.cuh"

namespace ftk {

// ------------------------------------------------------------------ select
// One warp per row.  Replaces topk_select_kernel
// (flash_topk_attn_v2/csrc/topk_select_kernel.cu:7-131): average = raw /
// valid_count (IEEE division), order by (average descending, block id
// ascending), sequential fp32 running sum of the raw scores, keep positions up
// to and including the first whose running sum reaches the threshold.
// The row's averages and raw scores sit in shared memory (block id = index);
// lane l owns ids l, l+32, ...  Each round takes the warp-wide best of the
// per-lane bests with two redux instructions and the owning lane rescans its
// own ids.  Scores are non-negative, so their bit patterns order as integers;
// consumed / absent entries hold -1.0f.
constexpr int SEL_WARPS = 8;

__global__ void __launch_bounds__(SEL_WARPS * 32)
topk_select_kernel(const float* __restrict__ scores, const float* __restrict__ row_scale,
                   int64_t rows, int M, int M_out, int bsz, int pad_head, int pad_tail,
                   float threshold, int32_t* __restrict__ out_idx, float* __restrict__ out_raw,
                   float* __restrict__ out_avg) {
  extern __shared__ float sel_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * SEL_WARPS + warp;
  if (row >= rows) return;
  const int Mp = (M + 31) & ~31;
  float* savg = sel_smem + static_cast<size_t>(warp) * 2 * Mp;
  float* sraw = savg + Mp;
  const float* in = scores + row * M;
  // unnormalised sums of the fused path are scaled by one reciprocal per row
  const float inv_total = row_scale ? __frcp_rn(row_scale[row]) : 1.f;
  // dividing by a power of two is exact as a multiplication: same bits, no divide
  const bool pow2 = (bsz & (bsz - 1)) == 0;
  const float inv_bsz = 1.f / static_cast<float>(bsz);

  int best_bits = __float_as_int(-1.f);
  int best_j = 0x7fffffff;
  for (int j = lane; j < Mp; j += 32) {
    float raw = 0.f, avg = -1.f;
    if (j < M) {
      raw = in[j];
      if (row_scale) raw *= inv_total;
      int n = bsz;
      if (j == 0) n -= pad_head;
      if (j == M - 1) n -= pad_tail;
      avg = (pow2 && n == bsz) ? raw * inv_bsz : __fdiv_rn(raw, static_cast<float>(n));
      if (!(avg >= 0.f)) avg = 0.f;  // NaN / negative input: rank last among real blocks
    }
    savg[j] = avg;
    sraw[j] = raw;
    const int bits = __float_as_int(avg);
    if (bits > best_bits) { best_bits = bits; best_j = j; }
  }
  __syncwarp();

  float cum = 0.f;
  bool cut = false;
  int32_t* oi = out_idx + row * M_out;
  float* orw = out_raw + row * M_out;
  float* oav = out_avg + row * M_out;
  int hold_idx = -1;
  float hold_raw = 0.f, hold_avg = 0.f;
  for (int r = 0; r < M_out; r++) {
    int w_idx = -1;
    float w_raw = 0.f, w_avg = 0.f;
    if (!cut) {
      const int mx = redux_max_s32(best_bits);
      const unsigned cand = (best_bits == mx) ? static_cast<unsigned>(best_j) : 0xffffffffu;
      const unsigned win = redux_min_u32(cand);
      w_idx = static_cast<int>(win);
      w_raw = sraw[win];
      w_avg = __int_as_float(mx);
      cum += w_raw;
      if (cum >= threshold) cut = true;
      if ((win & 31u) == static_cast<unsigned>(lane)) {
        savg[win] = -1.f;
        best_bits = __float_as_int(-1.f);
        best_j = 0x7fffffff;
        for (int j = lane; j < Mp; j += 32) {
          const int bits = __float_as_int(savg[j]);
          if (bits > best_bits) { best_bits = bits; best_j = j; }
        }
      }
    }
    if ((r & 31) == lane) { hold_idx = w_idx; hold_raw = w_raw; hold_avg = w_avg; }
    if ((r & 31) == 31 || r == M_out - 1) {
      const int base = r & ~31;
      if (base + lane <= r) {
        oi[base + lane] = hold_idx;
        orw[base + lane] = hold_raw;
        oav[base + lane] = hold_avg;
      }
    }
  }
}

// (bitonic_desc, sorted_emit and the per-row register select live in select_row.cuh)
// warps (= rows) per CTA: 8, or 4 where a row's scratch takes 6 KB
template <int IPT>
__host__ __device__ constexpr int sel_wpc() { return IPT >= 32 ? 4 : SEL_WARPS; }

template <int IPT>
__global__ void __launch_bounds__(sel_wpc<IPT>() * 32, IPT == 16 ? 3 : (IPT == 32 ? 4 : 1))
topk_select_reg_kernel(const float* __restrict__ scores, const float* __restrict__ row_scale,
                       int64_t rows, int M, int M_out, int bsz, int pad_head, int pad_tail,
                       float threshold, int32_t* __restrict__ out_idx,
                       float* __restrict__ out_raw, float* __restrict__ out_avg) {
  constexpr int WPC = sel_wpc<IPT>();
  constexpr int CAP = IPT >= 4 ? 256 : 128;
  __shared__ float sraw_all[WPC][32 * IPT];
  __shared__ unsigned long long scand_all[IPT >= 2 ? WPC : 1][CAP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a warp walks rows warp_id, warp_id + warps, ...; the loads of its next row are in
  // flight while it works on the current one (the kernel is otherwise bound by their latency)
  const int64_t nwarps = static_cast<int64_t>(gridDim.x) * WPC;
  int64_t row = static_cast<int64_t>(blockIdx.x) * WPC + warp;
  auto fetch = [&](int64_t r, float (&v)[IPT]) {
    const float* in = scores + r * M;
#pragma unroll
    for (int i = 0; i < IPT; i++) {
      const int j = i * 32 + lane;
      v[i] = (r < rows && j < M) ? __ldg(in + j) : 0.f;
    }
  };
  float cur[IPT], nxt[IPT];
  fetch(row, cur);
  for (; row < rows; row += nwarps) {
    fetch(row + nwarps, nxt);
    const float inv_total = row_scale ? __frcp_rn(row_scale[row]) : 1.f;
    select_row_reg<IPT>(cur, row_scale != nullptr, inv_total, M, M_out, bsz, pad_head, pad_tail,
                        threshold, sraw_all[warp], scand_all[IPT >= 2 ? warp : 0], lane,
                        out_idx + row * M_out, out_raw + row * M_out, out_avg + row * M_out);
    __syncwarp();   // the warp's scratch is free again
#pragma unroll
    for (int i = 0; i < IPT; i++) cur[i] = nxt[i];
  }
}

template <int IPT>
static void launch_select_reg(const float* block_scores, const float* row_scale, int64_t rows,
                              int M, int M_out, int bsz, int pad_head, int pad_tail,
                              float threshold, int32_t* topk_idx, float* topk_raw,
                              float* topk_avg, cudaStream_t st) {
  constexpr int WPC = sel_wpc<IPT>();
  // a few CTAs per SM, each warp looping over rows
  const int64_t want = (rows + WPC - 1) / WPC;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(want, sm_count() * 16LL));
  topk_select_reg_kernel<IPT><<<grid, WPC * 32, 0, st>>>(
      block_scores, row_scale, rows, M, M_out, bsz, pad_head, pad_tail, threshold, topk_idx,
      topk_raw, topk_avg);
}

int select_launch(const float* block_scores, const float* row_scale, int64_t rows, int M,
                  int max_topk, int bsz, int pad_head, int pad_tail, float threshold,
                  int32_t* topk_idx, float* topk_raw, float* topk_avg, cudaStream_t st) {
  if (!block_scores || !topk_idx || !topk_raw || !topk_avg) return FTK_ERR_BAD_ARG;
  if (rows <= 0 || M <= 0 || bsz <= 0 || max_topk < 0) return FTK_ERR_BAD_ARG;
  if (pad_head < 0 || pad_tail < 0 || pad_head >= bsz || pad_tail >= bsz) return FTK_ERR_BAD_ARG;
  if (M > 4096) return FTK_ERR_UNSUPPORTED;
  const int M_out = max_topk > 0 ? std::min(max_topk, M) : M;
  const int64_t grid = (rows + SEL_WARPS - 1) / SEL_WARPS;
  if (2 * grid > 0x7fffffffLL) return FTK_ERR_BAD_ARG;
  const unsigned g = static_cast<unsigned>(grid);
#define FTK_SEL_REG(IPT)                                                                        \
  launch_select_reg<IPT>(block_scores, row_scale, rows, M, M_out, bsz, pad_head, pad_tail,     \
                         threshold, topk_idx, topk_raw, topk_avg, st)
  if (M <= 32) FTK_SEL_REG(1);
  else if (M <= 64) FTK_SEL_REG(2);
  else if (M <= 128) FTK_SEL_REG(4);
  else if (M <= 256) FTK_SEL_REG(8);
  else if (M <= 512) FTK_SEL_REG(16);
  else if (M <= 1024) FTK_SEL_REG(32);
  else {
    const int Mp = (M + 31) & ~31;
    const size_t smem = static_cast<size_t>(SEL_WARPS) * 2 * Mp * sizeof(float);
    if (smem > 48 * 1024) {
      if (cudaFuncSetAttribute(topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem)) != cudaSuccess)
        return FTK_ERR_CUDA;
    }
    topk_select_kernel<<<g, SEL_WARPS * 32, smem, st>>>(
        block_scores, row_scale, rows, M, M_out, bsz, pad_head, pad_tail, threshold, topk_idx,
        topk_raw, topk_avg);
  }
#undef FTK_SEL_REG
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

// ------------------------------------------------------------------- merge
// One CTA (4 warps) per q-block.  Replaces qblock_merge_kernel
// (flash_topk_attn_v2/csrc/qblock_merge_kernel.cu:7-89).  The reference adds
// with shared-memory float atomics in arbitrary order; here warp w owns the
// block ids congruent to w mod 4 and walks every entry of the q-block in
// (row, rank) order, so each aggregate is an fp32 sum in one fixed order.
// Entries of one 32-wide step that name the same block (possible when K < 32)
// are applied in lane order.  The table is then sorted as 64-bit keys
// (aggregate bits : ~block id), largest first, with a bitonic network.
constexpr int MG_THREADS = 128;

__global__ void __launch_bounds__(MG_THREADS)
qblock_merge_kernel(const int32_t* __restrict__ idx, const float* __restrict__ scr, int64_t N,
                    int K, int g, int q_pad_head, int QM, int Mtot, int Mp, int W,
                    int32_t* __restrict__ out_idx, float* __restrict__ out_scr,
                    int32_t* __restrict__ counts, int* status) {
  extern __shared__ unsigned long long mg_keys[];
  float* agg = reinterpret_cast<float*>(mg_keys + Mp);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t qb = blockIdx.x;  // bh * QM + m
  const int64_t bh = qb / QM;
  const int m = static_cast<int>(qb - bh * QM);

  __shared__ int cnt_s;
  if (tid == 0) cnt_s = 0;
  for (int j = tid; j < Mp; j += MG_THREADS) agg[j] = 0.f;
  __syncthreads();

  const int t0 = m * g - q_pad_head;
  const int r0 = max(t0, 0);
  const int r1 = static_cast<int>(min(static_cast<long long>(N), static_cast<long long>(t0) + g));
  if (r1 > r0) {
    const int64_t base = (bh * N + r0) * K;
    const int total = (r1 - r0) * K;
    for (int e0 = 0; e0 < total; e0 += 32) {
      const int e = e0 + lane;
      int j = -1;
      float s = 0.f;
      if (e < total) {
        j = idx[base + e];
        s = scr ? scr[base + e] : 1.f;
      }
      if (j >= Mtot) {
        if (status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
        j = -1;
      }
      const bool mine = (j >= 0) && ((j & 3) == warp);
      const unsigned grp = __match_any_sync(0xffffffffu, mine ? j : -1 - lane);
      const int rank = __popc(grp & ((1u << lane) - 1u));
      const int rounds = redux_max_s32(mine ? __popc(grp) : 0);
      for (int rd = 0; rd < rounds; rd++) {
        if (mine && rank == rd) agg[j] += s;
        __syncwarp();
      }
    }
  }
  __syncthreads();

  for (int j = tid; j < Mp; j += MG_THREADS) {
    const float a = agg[j];
    unsigned long long key = 0ull;
    if (j < Mtot && a > 0.f)
      key = (static_cast<unsigned long long>(__float_as_uint(a)) << 32) |
            static_cast<unsigned long long>(0xffffffffu - static_cast<unsigned>(j));
    mg_keys[j] = key;
  }
  __syncthreads();
  // bitonic sort, descending
  for (int k = 2; k <= Mp; k <<= 1) {
    for (int s = k >> 1; s > 0; s >>= 1) {
      for (int i = tid; i < Mp; i += MG_THREADS) {
        const int p = i ^ s;
        if (p > i) {
          const unsigned long long a = mg_keys[i], b = mg_keys[p];
          const bool desc = ((i & k) == 0);
          if (desc ? (a < b) : (a > b)) { mg_keys[i] = b; mg_keys[p] = a; }
        }
      }
      __syncthreads();
    }
  }
  int local = 0;
  int32_t* oi = out_idx + qb * W;
  float* os = out_scr ? out_scr + qb * W : nullptr;
  for (int r = tid; r < W; r += MG_THREADS) {
    int id = -1;
    float sc = 0.f;
    if (r < Mp) {
      const unsigned long long key = mg_keys[r];
      if (key != 0ull) {
        id = static_cast<int>(0xffffffffu - static_cast<unsigned>(key & 0xffffffffull));
        sc = __uint_as_float(static_cast<unsigned>(key >> 32));
        local++;
      }
    }
    oi[r] = id;
    if (os) os[r] = sc;
  }
  // count = number of valid entries written (they form a prefix of the row)
  if (local) atomicAdd(&cnt_s, local);
  __syncthreads();
  if (tid == 0 && counts) counts[qb] = cnt_s;
}

// Bitonic network over 32*E values held E per lane in BLOCKED order (position
// p = lane*E + r), sorted largest first.  Strides below E stay inside a lane
// (registers only); only the log2(32) largest strides of each merge cross
// lanes, so a 512-key sort needs 15 shuffle stages where the striped layout of
// bitonic_desc needs 35.
template <int E, typename T>
__device__ __forceinline__ void bitonic_desc_blocked(T (&v)[E], int lane) {
  constexpr int N = 32 * E;
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j < E) {
#pragma unroll
        for (int r = 0; r < E; r++) {
          if ((r & j) == 0) {
            // k < E: the direction bit is a bit of r, else a bit of the lane
            const bool desc = (k < E) ? ((r & k) == 0) : ((lane & (k / E)) == 0);
            const T x = v[r], y = v[r | j];
            const bool sw = desc ? (x < y) : (x > y);
            v[r] = sw ? y : x;
            v[r | j] = sw ? x : y;
          }
        }
      } else {
        const int jl = j / E;
        const bool lower = (lane & jl) == 0;
        const bool desc = (lane & (k / E)) == 0;
        const bool take_max = (desc == lower);
#pragma unroll
        for (int r = 0; r < E; r++) {
          const T o = __shfl_xor_sync(0xffffffffu, v[r], jl);
          const bool o_gt = o > v[r];
          v[r] = (take_max == o_gt) ? o : v[r];
        }
      }
    }
  }
}

// Merge with ONE WARP per q-block, for tables of up to 32*E <= 1024 block ids
// (every BASELINE shape).  Same arithmetic as qblock_merge_kernel: the entries
// of the q-block are walked in (row, rank) order, 32 at a time, entries of one
// step that name the same block are applied in lane order, so every aggregate
// is the same fp32 sum in the same order.  No block-wide barrier: the warp
// zeroes its own table in shared memory, adds into it (repeats inside a step
// are found with a tag table, see below), builds 64-bit keys (aggregate bits : ~block id) in registers,
// sorts them with the blocked bitonic network and writes its row, the -1 / 0
// tail with 16-byte stores.
constexpr int MGW_WARPS = 4;

template <int E>
__global__ void __launch_bounds__(MGW_WARPS * 32)
qblock_merge_warp_kernel(const int32_t* __restrict__ idx, const float* __restrict__ scr, int64_t N,
                         int K, int g, int q_pad_head, int QM, int64_t total_qb, int Mtot, int W,
                         int32_t* __restrict__ out_idx, float* __restrict__ out_scr,
                         int32_t* __restrict__ counts, int* status) {
  constexpr int MP = 32 * E;
  constexpr int U = 4;   // steps fetched and checked together
  __shared__ float agg_all[MGW_WARPS][MP];
  __shared__ uint8_t tag_all[MGW_WARPS][U * MP];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t qb = static_cast<int64_t>(blockIdx.x) * MGW_WARPS + warp;  // bh * QM + m
  if (qb >= total_qb) return;
  float* agg = agg_all[warp];
  uint8_t* tag = tag_all[warp];
  const int64_t bh = qb / QM;
  const int m = static_cast<int>(qb - bh * QM);
#pragma unroll
  for (int r = 0; r < E; r++) agg[r * 32 + lane] = 0.f;
  __syncwarp();

  const int t0 = m * g - q_pad_head;
  const int r0 = max(t0, 0);
  const int r1 = static_cast<int>(min(static_cast<long long>(N), static_cast<long long>(t0) + g));
  if (r1 > r0) {
    const int64_t base = (bh * N + r0) * K;
    const int total = (r1 - r0) * K;
    // A step is up to 32 consecutive entries; when a row holds fewer than 32
    // picks a step is one row, so that entries of a step come from one row and
    // (top-k picks of a row being distinct) name distinct blocks.
    const int step = K < 32 ? K : 32;
    // the next batch of U steps is in flight while this one is applied
    int jn[U];
    float sn[U];
    auto fetch = [&](int e0) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int e = e0 + u * step + lane;
        jn[u] = -1;
        sn[u] = 0.f;
        if (lane < step && e < total) {
          jn[u] = __ldg(idx + base + e);
          sn[u] = scr ? __ldg(scr + base + e) : 1.f;
        }
      }
    };
    fetch(0);
    for (int e0 = 0; e0 < total; e0 += step * U) {
      int jj[U];
      float ss[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        jj[u] = jn[u];
        ss[u] = sn[u];
      }
      if (e0 + step * U < total) fetch(e0 + step * U);
      // Do two entries of one step name the same block?  Each lane writes its
      // lane number into the step's tag table at its block id and reads it
      // back: a lane that finds another lane's number shares its id with it.
      // (A match instruction answers the same question at many times the cost.)
      bool lost = false;
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (jj[u] >= Mtot) {
          if (status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
          jj[u] = -1;
        }
        if (jj[u] >= 0) tag[u * MP + jj[u]] = static_cast<uint8_t>(lane);
      }
      __syncwarp();
#pragma unroll
      for (int u = 0; u < U; u++)
        if (jj[u] >= 0) lost |= tag[u * MP + jj[u]] != static_cast<uint8_t>(lane);
      const bool repeats = __any_sync(0xffffffffu, lost);
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (e0 + u * step >= total) break;   // warp-uniform
        const int j = jj[u];
        const bool act = j >= 0;
        if (!repeats) {
          if (act) agg[j] += ss[u];
        } else {
          // entries of the step that share a block are applied in lane order
          const unsigned grp = __match_any_sync(0xffffffffu, act ? j : -1 - lane);
          const int rank = __popc(grp & ((1u << lane) - 1u));
          const int rounds = redux_max_s32(act ? __popc(grp) : 1);
          for (int rd = 0; rd < rounds; rd++) {
            if (act && rank == rd) agg[j] += ss[u];
            __syncwarp();
          }
        }
        __syncwarp();
      }
    }
  }
  __syncwarp();

  // any assignment of ids to sort positions will do: read the table bank by bank
  unsigned long long key[E];
  int nz = 0;
#pragma unroll
  for (int r = 0; r < E; r++) {
    const int j = r * 32 + lane;
    const float a = agg[j];
    key[r] = 0ull;
    if (j < Mtot && a > 0.f) {
      key[r] = (static_cast<unsigned long long>(__float_as_uint(a)) << 32) |
               static_cast<unsigned long long>(0xffffffffu - static_cast<unsigned>(j));
      nz++;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) nz += __shfl_xor_sync(0xffffffffu, nz, d);
  bitonic_desc_blocked<E>(key, lane);

  int32_t* oi = out_idx + qb * W;
  float* os = out_scr ? out_scr + qb * W : nullptr;
  int ids[E];
  float scs[E];
#pragma unroll
  for (int r = 0; r < E; r++) {
    ids[r] = key[r] ? static_cast<int>(0xffffffffu - static_cast<unsigned>(key[r] & 0xffffffffull))
                    : -1;
    scs[r] = __uint_as_float(static_cast<unsigned>(key[r] >> 32));
  }
  const bool vec = (W & 3) == 0 && (reinterpret_cast<uintptr_t>(out_idx) & 15) == 0 &&
                   (!out_scr || (reinterpret_cast<uintptr_t>(out_scr) & 15) == 0);
  const int p0 = lane * E;   // first rank held by this lane
  if (E >= 4 && vec) {
#pragma unroll
    for (int r = 0; r < E; r += 4) {
      if (p0 + r < W) {      // W % 4 == 0: the whole quad is inside the row
        *reinterpret_cast<int4*>(oi + p0 + r) = make_int4(ids[r], ids[r + 1], ids[r + 2], ids[r + 3]);
        if (os)
          *reinterpret_cast<float4*>(os + p0 + r) =
              make_float4(scs[r], scs[r + 1], scs[r + 2], scs[r + 3]);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < E; r++) {
      if (p0 + r < W) {
        oi[p0 + r] = ids[r];
        if (os) os[p0 + r] = scs[r];
      }
    }
  }
  if (W > MP) {
    if (vec) {
      int4* o4 = reinterpret_cast<int4*>(oi);
      float4* s4 = reinterpret_cast<float4*>(os);
      for (int x = (MP >> 2) + lane; x < (W >> 2); x += 32) {
        o4[x] = make_int4(-1, -1, -1, -1);
        if (os) s4[x] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      for (int x = MP + lane; x < W; x += 32) {
        oi[x] = -1;
        if (os) os[x] = 0.f;
      }
    }
  }
  // valid entries form a prefix of the row
  if (lane == 0 && counts) counts[qb] = min(nz, W);
}

// Exact union of a q-block's per-row picks, ascending by block id.  Replaces
// _build_qblock_indices_kernel of the first-generation operators
// (flash_topk_attn/attention.py:23-67: load, sort, drop repeats, compact).
// One CTA per q-block: the picks set bits of a shared-memory bitmap (order
// free), then each warp lists the set bits of its words behind an exclusive
// prefix of the word popcounts.  Rows beyond `W` entries cannot occur when W
// >= min(g * K, blocks); a longer union is cut and reported.
constexpr int UN_THREADS = 128;
constexpr int UN_MAX_WORDS = 2048;   // 65536 block ids

__global__ void __launch_bounds__(UN_THREADS)
qblock_union_kernel(const int32_t* __restrict__ idx, int64_t N, int K, int g, int q_pad_head,
                    int QM, int Mtot, int W, int32_t* __restrict__ out_idx,
                    int32_t* __restrict__ counts, int* status) {
  __shared__ unsigned bits[UN_MAX_WORDS];
  __shared__ int wsum[UN_THREADS / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t qb = blockIdx.x;
  const int64_t bh = qb / QM;
  const int m = static_cast<int>(qb - bh * QM);
  const int words = (Mtot + 31) >> 5;
  for (int j = tid; j < words; j += UN_THREADS) bits[j] = 0u;
  __syncthreads();
  const int t0 = m * g - q_pad_head;
  const int r0 = max(t0, 0);
  const int r1 = static_cast<int>(min(static_cast<long long>(N), static_cast<long long>(t0) + g));
  if (r1 > r0) {
    const int64_t base = (bh * N + r0) * K;
    const int total = (r1 - r0) * K;
    auto mark = [&](int j) {
      if (j >= Mtot) {
        if (status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
      } else if (j >= 0) {
        atomicOr(&bits[j >> 5], 1u << (j & 31));
      }
    };
    const int32_t* src = idx + base;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (total & 3) == 0) {
      // 16-byte loads, four in flight per thread
      const int4* src4 = reinterpret_cast<const int4*>(src);
      const int quads = total >> 2;
      for (int e0 = 0; e0 < quads; e0 += 4 * UN_THREADS) {
        int4 t[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int e = e0 + u * UN_THREADS + tid;
          t[u] = e < quads ? __ldg(src4 + e) : make_int4(-1, -1, -1, -1);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          mark(t[u].x);
          mark(t[u].y);
          mark(t[u].z);
          mark(t[u].w);
        }
      }
    } else {
      for (int e = tid; e < total; e += UN_THREADS) mark(src[e]);
    }
  }
  __syncthreads();
  // each thread owns a contiguous run of words: ascending ids stay ascending
  const int per = (words + UN_THREADS - 1) / UN_THREADS;
  const int w0 = min(tid * per, words), w1 = min(w0 + per, words);
  int mine = 0;
  for (int j = w0; j < w1; j++) mine += __popc(bits[j]);
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += t;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  int before = incl - mine, total_cnt = 0;
  for (int x = 0; x < UN_THREADS / 32; x++) {
    if (x < warp) before += wsum[x];
    total_cnt += wsum[x];
  }
  int32_t* oi = out_idx + qb * W;
  for (int j = w0; j < w1; j++) {
    unsigned b = bits[j];
    while (b) {
      const int bit = __ffs(b) - 1;
      b &= b - 1;
      if (before < W) oi[before] = j * 32 + bit;
      before++;
    }
  }
  const int kept = min(total_cnt, W);
  if ((reinterpret_cast<uintptr_t>(oi) & 15) == 0 && (W & 3) == 0) {
    const int a = min((kept + 3) & ~3, W);
    if (tid < a - kept) oi[kept + tid] = -1;
    int4* o4 = reinterpret_cast<int4*>(oi);
    for (int r = (a >> 2) + tid; r < (W >> 2); r += UN_THREADS) o4[r] = make_int4(-1, -1, -1, -1);
  } else {
    for (int r = kept + tid; r < W; r += UN_THREADS) oi[r] = -1;
  }
  if (tid == 0) {
    if (counts) counts[qb] = kept;
    if (total_cnt > W && status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
  }
}

__global__ void max_index_kernel(const int32_t* __restrict__ idx, int64_t n, int32_t* result) {
  int mx = 0;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    mx = max(mx, idx[i] + 1);
  mx = redux_max_s32(mx);
  if ((threadIdx.x & 31) == 0) atomicMax(result, mx);
}
__global__ void set_one_kernel(int32_t* p) { *p = 1; }

// ----------------------------------------------------------- reverse index
// Replaces build_reverse_indices_kernel / argsort_reverse_counts_kernel
// (flash_topk_attn_v2/csrc/build_reverse_indices_kernel.cu:6-62).  The
// reference hands out slots with global atomicAdd (arbitrary order); here a
// bitmap [bh][kv block][q-block bit] is OR-ed together first (order-free),
// then one warp per kv block lists its set bits in ascending q-block order.
__global__ void reverse_mark_kernel(const int32_t* __restrict__ merged,
                                    const int32_t* __restrict__ counts, int64_t total_qb, int QM,
                                    int W, int M, int words, unsigned* __restrict__ bits,
                                    int* status) {
  // one warp per q-block row
  const int64_t qb = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (qb >= total_qb) return;
  const int64_t bh = qb / QM;
  const int m = static_cast<int>(qb - bh * QM);
  const int cnt = counts ? min(counts[qb], W) : W;
  const int32_t* row = merged + qb * W;
  for (int e = lane; e < cnt; e += 32) {
    const int j = row[e];
    if (j < 0) continue;
    if (j >= M) {
      if (status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
      continue;
    }
    atomicOr(&bits[(bh * M + j) * words + (m >> 5)], 1u << (m & 31));
  }
}

__global__ void reverse_list_kernel(const unsigned* __restrict__ bits, int64_t total_kv, int QM,
                                    int words, int32_t* __restrict__ rev,
                                    int32_t* __restrict__ rcount) {
  const int64_t kv = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (kv >= total_kv) return;
  const unsigned* wrow = bits + kv * words;
  int32_t* out = rev + kv * QM;
  int base = 0;
  for (int w0 = 0; w0 < words; w0 += 32) {
    const int wi = w0 + lane;
    const unsigned word = wi < words ? wrow[wi] : 0u;
    const int c = __popc(word);
    // exclusive prefix over lanes
    int pre = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, pre, d);
      if (lane >= d) pre += v;
    }
    const int tot = __shfl_sync(0xffffffffu, pre, 31);
    int pos = base + pre - c;
    unsigned wbits = word;
    while (wbits) {
      const int b = __ffs(wbits) - 1;
      wbits &= wbits - 1;
      out[pos++] = wi * 32 + b;
    }
    base += tot;
  }
  for (int i = base + lane; i < QM; i += 32) out[i] = -1;
  if (lane == 0) rcount[kv] = base;
}

// per-(b,h) stable descending argsort of the M counts (bitonic on 64-bit keys)
__global__ void reverse_sort_kernel(const int32_t* __restrict__ rcount, int M, int Mp,
                                    int32_t* __restrict__ sorted_kv) {
  extern __shared__ unsigned long long rs_keys[];
  const int tid = threadIdx.x;
  const int64_t bh = blockIdx.x;
  for (int j = tid; j < Mp; j += blockDim.x) {
    unsigned long long key = 0ull;
    if (j < M)
      key = (static_cast<unsigned long long>(static_cast<unsigned>(rcount[bh * M + j]) + 1u) << 32) |
            static_cast<unsigned long long>(0xffffffffu - static_cast<unsigned>(j));
    rs_keys[j] = key;
  }
  __syncthreads();
  for (int k = 2; k <= Mp; k <<= 1) {
    for (int s = k >> 1; s > 0; s >>= 1) {
      for (int i = tid; i < Mp; i += blockDim.x) {
        const int p = i ^ s;
        if (p > i) {
          const unsigned long long a = rs_keys[i], b = rs_keys[p];
          const bool desc = ((i & k) == 0);
          if (desc ? (a < b) : (a > b)) { rs_keys[i] = b; rs_keys[p] = a; }
        }
      }
      __syncthreads();
    }
  }
  for (int r = tid; r < M; r += blockDim.x)
    sorted_kv[bh * M + r] =
        static_cast<int>(0xffffffffu - static_cast<unsigned>(rs_keys[r] & 0xffffffffull));
}

// ------------------------------------------------------------ count sort
// Replaces sort_by_count_launch (flash_topk_attn_v2/csrc/sort_by_count_kernel.cu:12-52,
// a CUB device radix sort): stable counting sort, descending.  Chunks of the
// input are histogrammed, a single CTA turns the [key][chunk] table into start
// offsets (key descending, chunk ascending), and each chunk is then placed by
// one warp walking it in order so equal counts keep ascending flat id.
constexpr int SBC_CHUNK = 2048;

__global__ void sbc_hist_kernel(const int32_t* __restrict__ counts, int64_t total, int range,
                                int nchunk, unsigned* __restrict__ table) {
  const int chunk = blockIdx.x;
  const int64_t b0 = static_cast<int64_t>(chunk) * SBC_CHUNK;
  const int64_t b1 = min(static_cast<long long>(total), static_cast<long long>(b0) + SBC_CHUNK);
  for (int64_t i = b0 + threadIdx.x; i < b1; i += blockDim.x) {
    int key = counts[i];
    key = min(max(key, 0), range - 1);
    atomicAdd(&table[static_cast<size_t>(key) * nchunk + chunk], 1u);
  }
}
// exclusive scan of the table read in (key descending, chunk ascending) order
constexpr int SBC_SCAN_THREADS = 512;
__global__ void __launch_bounds__(SBC_SCAN_THREADS)
sbc_scan_kernel(unsigned* __restrict__ table, int range, int nchunk) {
  __shared__ unsigned warp_tot[SBC_SCAN_THREADS / 32];
  __shared__ unsigned carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  const int64_t n = static_cast<int64_t>(range) * nchunk;
  for (int64_t b = 0; b < n; b += SBC_SCAN_THREADS) {
    const int64_t i = b + tid;
    int64_t src = 0;
    unsigned v = 0;
    if (i < n) {
      const int64_t key = range - 1 - i / nchunk, chunk = i % nchunk;
      src = key * nchunk + chunk;
      v = table[src];
    }
    unsigned inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned u = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += u;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    unsigned woff = 0, btot = 0;
    for (int wv = 0; wv < SBC_SCAN_THREADS / 32; wv++) {
      const unsigned t = warp_tot[wv];
      if (wv < warp) woff += t;
      btot += t;
    }
    const unsigned carry = carry_s;
    if (i < n) table[src] = carry + woff + inc - v;
    __syncthreads();
    if (tid == 0) carry_s = carry + btot;
    __syncthreads();
  }
}
__global__ void sbc_place_kernel(const int32_t* __restrict__ counts, int64_t total, int range,
                                 int nchunk, unsigned* __restrict__ table,
                                 int32_t* __restrict__ sorted_counts,
                                 int32_t* __restrict__ sorted_ids) {
  const int chunk = blockIdx.x;
  const int lane = threadIdx.x;
  const int64_t b0 = static_cast<int64_t>(chunk) * SBC_CHUNK;
  const int64_t b1 = min(static_cast<long long>(total), static_cast<long long>(b0) + SBC_CHUNK);
  for (int64_t i0 = b0; i0 < b1; i0 += 32) {
    const int64_t i = i0 + lane;
    const bool act = i < b1;
    int raw = act ? counts[i] : 0;
    int key = act ? min(max(raw, 0), range - 1) : -1 - lane;
    const unsigned grp = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(grp & ((1u << lane) - 1u));
    unsigned base = 0;
    if (act) base = table[static_cast<size_t>(key) * nchunk + chunk];
    __syncwarp();
    if (act) {
      sorted_counts[base + rank] = raw;
      sorted_ids[base + rank] = static_cast<int32_t>(i);
      if (rank == __popc(grp) - 1) table[static_cast<size_t>(key) * nchunk + chunk] = base + rank + 1;
    }
    __syncwarp();
  }
}

}  // namespace ftk

using namespace ftk;

extern "C" int ftk_topk_select(const float* block_scores, const float* row_scale, int64_t rows,
                               int M, int max_topk, int score_block_size, int pad_head,
                               int pad_tail, float threshold, int32_t* topk_idx, float* topk_raw,
                               float* topk_avg, int32_t* status, void* stream) {
  (void)status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return select_launch(block_scores, row_scale, rows, M, max_topk, score_block_size, pad_head,
                       pad_tail, threshold, topk_idx, topk_raw, topk_avg, st);
}

static int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

extern "C" int ftk_qblock_merge(const int32_t* topk_idx, const float* topk_scores, int64_t BH,
                                int64_t N, int K, int q_block_size, int q_pad_head,
                                int q_pad_tail, int num_score_blocks, int qblock_topk,
                                int32_t* merged_idx, float* merged_scores, int32_t* counts,
                                int32_t* status, void* stream) {
  if (!topk_idx || !merged_idx || BH <= 0 || N <= 0 || K <= 0) return FTK_ERR_BAD_ARG;
  if (q_block_size <= 0 || qblock_topk <= 0 || num_score_blocks <= 0) return FTK_ERR_BAD_ARG;
  if (q_pad_head < 0 || q_pad_tail < 0 || q_pad_head >= q_block_size ||
      q_pad_tail >= q_block_size)
    return FTK_ERR_BAD_ARG;
  if ((q_pad_head + N + q_pad_tail) % q_block_size != 0) return FTK_ERR_BAD_ARG;
  if (num_score_blocks > 4096) return FTK_ERR_UNSUPPORTED;
  const int64_t QM = (q_pad_head + N + q_pad_tail) / q_block_size;
  if (BH * QM > 0x7fffffffLL || QM > 0x7fffffffLL) return FTK_ERR_BAD_ARG;
  const int Mp = std::max(32, next_pow2(num_score_blocks));
  const size_t smem = static_cast<size_t>(Mp) * 12;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (Mp <= 1024) {
    // one warp per q-block
    const int64_t total_qb = BH * QM;
    const unsigned grid = static_cast<unsigned>((total_qb + MGW_WARPS - 1) / MGW_WARPS);
#define FTK_MGW(E)                                                                          \
  qblock_merge_warp_kernel<E><<<grid, MGW_WARPS * 32, 0, st>>>(                             \
      topk_idx, topk_scores, N, K, q_block_size, q_pad_head, static_cast<int>(QM), total_qb, \
      num_score_blocks, qblock_topk, merged_idx, merged_scores, counts, status)
    switch (Mp) {
      case 32: FTK_MGW(1); break;
      case 64: FTK_MGW(2); break;
      case 128: FTK_MGW(4); break;
      case 256: FTK_MGW(8); break;
      case 512: FTK_MGW(16); break;
      default: FTK_MGW(32); break;
    }
#undef FTK_MGW
    return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
  }
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(qblock_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return FTK_ERR_CUDA;
  qblock_merge_kernel<<<static_cast<unsigned>(BH * QM), MG_THREADS, smem, st>>>(
      topk_idx, topk_scores, N, K, q_block_size, q_pad_head, static_cast<int>(QM),
      num_score_blocks, Mp, qblock_topk, merged_idx, merged_scores, counts, status);
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" int ftk_qblock_union(const int32_t* topk_idx, int64_t BH, int64_t N, int K,
                                int q_block_size, int q_pad_head, int q_pad_tail,
                                int num_score_blocks, int width, int32_t* merged_idx,
                                int32_t* counts, int32_t* status, void* stream) {
  if (!topk_idx || !merged_idx || BH <= 0 || N <= 0 || K <= 0) return FTK_ERR_BAD_ARG;
  if (q_block_size <= 0 || width <= 0 || num_score_blocks <= 0) return FTK_ERR_BAD_ARG;
  if (q_pad_head < 0 || q_pad_tail < 0 || q_pad_head >= q_block_size ||
      q_pad_tail >= q_block_size)
    return FTK_ERR_BAD_ARG;
  if ((q_pad_head + N + q_pad_tail) % q_block_size != 0) return FTK_ERR_BAD_ARG;
  if (num_score_blocks > UN_MAX_WORDS * 32) return FTK_ERR_UNSUPPORTED;
  const int64_t QM = (q_pad_head + N + q_pad_tail) / q_block_size;
  if (BH * QM > 0x7fffffffLL) return FTK_ERR_BAD_ARG;
  qblock_union_kernel<<<static_cast<unsigned>(BH * QM), UN_THREADS, 0,
                        static_cast<cudaStream_t>(stream)>>>(
      topk_idx, N, K, q_block_size, q_pad_head, static_cast<int>(QM), num_score_blocks, width,
      merged_idx, counts, status);
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" int ftk_max_index_plus1(const int32_t* idx, int64_t count, int32_t* result,
                                   void* stream) {
  if (!idx || !result || count < 0) return FTK_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  set_one_kernel<<<1, 1, 0, st>>>(result);
  if (count > 0) {
    const int grid = static_cast<int>(std::min<int64_t>((count + 255) / 256, 148 * 8));
    max_index_kernel<<<grid, 256, 0, st>>>(idx, count, result);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" size_t ftk_build_reverse_workspace(int64_t BH, int QM, int M) {
  const size_t words = static_cast<size_t>((QM + 31) / 32);
  return ((static_cast<size_t>(BH) * M * words * 4) + 255) & ~static_cast<size_t>(255);
}

extern "C" int ftk_build_reverse(const int32_t* merged_idx, const int32_t* counts, int64_t BH,
                                 int QM, int W, int M, int32_t* reverse_idx,
                                 int32_t* reverse_counts, int32_t* sorted_kv, void* workspace,
                                 size_t workspace_bytes, int32_t* status, void* stream) {
  if (!merged_idx || !reverse_idx || !reverse_counts) return FTK_ERR_BAD_ARG;
  if (BH <= 0 || QM <= 0 || W <= 0 || M <= 0) return FTK_ERR_BAD_ARG;
  if (sorted_kv && M > 8192) return FTK_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < ftk_build_reverse_workspace(BH, QM, M))
    return FTK_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int words = (QM + 31) / 32;
  unsigned* bits = static_cast<unsigned*>(workspace);
  if (cudaMemsetAsync(bits, 0, static_cast<size_t>(BH) * M * words * 4, st) != cudaSuccess)
    return FTK_ERR_CUDA;
  const int64_t total_qb = BH * QM, total_kv = BH * M;
  reverse_mark_kernel<<<static_cast<unsigned>((total_qb * 32 + 255) / 256), 256, 0, st>>>(
      merged_idx, counts, total_qb, QM, W, M, words, bits, status);
  reverse_list_kernel<<<static_cast<unsigned>((total_kv * 32 + 255) / 256), 256, 0, st>>>(
      bits, total_kv, QM, words, reverse_idx, reverse_counts);
  if (sorted_kv) {
    const int Mp = std::max(32, next_pow2(M));
    const size_t smem = static_cast<size_t>(Mp) * 8;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(reverse_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    reverse_sort_kernel<<<static_cast<unsigned>(BH), 256, smem, st>>>(reverse_counts, M, Mp,
                                                                     sorted_kv);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

extern "C" size_t ftk_sort_by_count_workspace(int64_t total, int max_count) {
  const size_t nchunk = static_cast<size_t>((total + SBC_CHUNK - 1) / SBC_CHUNK);
  return ((static_cast<size_t>(max_count) + 1) * nchunk * 4 + 255) & ~static_cast<size_t>(255);
}

extern "C" int ftk_sort_by_count(const int32_t* counts, int64_t total, int max_count,
                                 int32_t* sorted_counts, int32_t* sorted_ids, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  if (!counts || !sorted_counts || !sorted_ids || total <= 0 || max_count < 0)
    return FTK_ERR_BAD_ARG;
  if (total > 0x7fffffffLL) return FTK_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < ftk_sort_by_count_workspace(total, max_count))
    return FTK_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int range = max_count + 1;
  const int nchunk = static_cast<int>((total + SBC_CHUNK - 1) / SBC_CHUNK);
  unsigned* table = static_cast<unsigned*>(workspace);
  if (cudaMemsetAsync(table, 0, static_cast<size_t>(range) * nchunk * 4, st) != cudaSuccess)
    return FTK_ERR_CUDA;
  sbc_hist_kernel<<<nchunk, 256, 0, st>>>(counts, total, range, nchunk, table);
  sbc_scan_kernel<<<1, SBC_SCAN_THREADS, 0, st>>>(table, range, nchunk);
  sbc_place_kernel<<<nchunk, 32, 0, st>>>(counts, total, range, nchunk, table, sorted_counts,
                                          sorted_ids);
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}

// ------------------------------------------------- reverse index, no allocation
// Some callers of this library cannot hand it a workspace because they cannot
// allocate device memory at the point of the call: code running inside a
// memory-pool callback, a plugin whose host gives it fixed input/output
// buffers only, or a latency-critical loop that must never enter the
// allocator.  For them this entry point does what ftk_build_reverse does, with
// the membership bitmap kept in a fixed array that is part of the loaded
// library image (FTK_NOALLOC_REVERSE_BYTES on every GPU that loads the
// library, held until the process exits).
//
// In host code the array's name is only a handle, not a device address, so
// the address is looked up per device with cudaGetSymbolAddress the first time
// the entry point runs on that device (with that device current) and cached.
// That first call should come before any stream capture.  The array is shared
// by every call and keeps the previous call's bits: the part a call needs is
// cleared on the caller's stream first.  Two calls whose GPU work overlaps
// (different streams, or different host threads) race on it.
constexpr size_t FTK_NOALLOC_REVERSE_BYTES = 4u << 20;  // 4 MiB
constexpr int FTK_NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) unsigned g_noalloc_reverse_bits[FTK_NOALLOC_REVERSE_BYTES / 4];

static std::mutex g_noalloc_mutex;
static unsigned* g_noalloc_ptr[FTK_NOALLOC_MAX_DEVICES] = {nullptr};

extern "C" size_t ftk_build_reverse_noalloc_capacity(void) { return FTK_NOALLOC_REVERSE_BYTES; }

extern "C" int ftk_build_reverse_noalloc(const int32_t* merged_idx, const int32_t* counts,
                                         int64_t BH, int QM, int W, int M, int32_t* reverse_idx,
                                         int32_t* reverse_counts, int32_t* sorted_kv,
                                         int32_t* status, void* stream) {
  if (!merged_idx || !reverse_idx || !reverse_counts) return FTK_ERR_BAD_ARG;
  if (BH <= 0 || QM <= 0 || W <= 0 || M <= 0) return FTK_ERR_BAD_ARG;
  if (sorted_kv && M > 8192) return FTK_ERR_UNSUPPORTED;
  const int words = (QM + 31) / 32;
  const size_t need = static_cast<size_t>(BH) * M * words * 4;
  // larger problems must use ftk_build_reverse with a caller-owned workspace
  if (need > FTK_NOALLOC_REVERSE_BYTES) return FTK_ERR_CAPACITY;

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FTK_ERR_CUDA;
  if (dev < 0 || dev >= FTK_NOALLOC_MAX_DEVICES) return FTK_ERR_UNSUPPORTED;
  unsigned* bits = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_reverse_bits) != cudaSuccess || !p)
        return FTK_ERR_CUDA;
      g_noalloc_ptr[dev] = static_cast<unsigned*>(p);
    }
    bits = g_noalloc_ptr[dev];
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(bits, 0, need, st) != cudaSuccess) return FTK_ERR_CUDA;
  const int64_t total_qb = BH * QM, total_kv = BH * M;
  reverse_mark_kernel<<<static_cast<unsigned>((total_qb * 32 + 255) / 256), 256, 0, st>>>(
      merged_idx, counts, total_qb, QM, W, M, words, bits, status);
  reverse_list_kernel<<<static_cast<unsigned>((total_kv * 32 + 255) / 256), 256, 0, st>>>(
      bits, total_kv, QM, words, reverse_idx, reverse_counts);
  if (sorted_kv) {
    const int Mp = std::max(32, next_pow2(M));
    const size_t smem = static_cast<size_t>(Mp) * 8;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(reverse_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return FTK_ERR_CUDA;
    reverse_sort_kernel<<<static_cast<unsigned>(BH), 256, smem, st>>>(reverse_counts, M, Mp,
                                                                     sorted_kv);
  }
  return cudaGetLastError() == cudaSuccess ? FTK_OK : FTK_ERR_CUDA;
}
