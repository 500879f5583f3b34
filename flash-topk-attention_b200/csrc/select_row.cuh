// Top-k select of one row by one warp (used by topk_select_reg_kernel).
#pragma once

#include "ftk_sm100.cuh"

namespace ftk {

__device__ __forceinline__ int redux_max_s32(int v) {
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ unsigned redux_min_u32(unsigned v) {
  unsigned r;
  asm volatile("redux.sync.min.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}

// Bitonic network over 32*E values held E per lane (position p = r*32 + lane),
// sorted largest first.  Distances below 32 exchange across lanes, the others
// between registers of one lane; every index is a compile-time constant.
template <int E, typename T>
__device__ __forceinline__ void bitonic_desc(T (&v)[E], int lane) {
  constexpr int LOGN = (E == 1 ? 5 : E == 2 ? 6 : E == 4 ? 7 : 8);
#pragma unroll
  for (int lk = 1; lk <= LOGN; lk++) {
    const int k = 1 << lk;
#pragma unroll
    for (int lj = lk - 1; lj >= 0; lj--) {
      const int j = 1 << lj;
      if (j >= 32) {
        const int jr = j >> 5;
#pragma unroll
        for (int r = 0; r < E; r++) {
          if ((r & jr) == 0) {
            const bool desc = (((r * 32) & k) == 0);
            const T x = v[r], y = v[r | jr];
            const bool sw = desc ? (x < y) : (x > y);
            v[r] = sw ? y : x;
            v[r | jr] = sw ? x : y;
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < E; r++) {
          const T o = __shfl_xor_sync(0xffffffffu, v[r], j);
          const bool desc = (((r * 32 + lane) & k) == 0);
          const bool lower = (lane & j) == 0;
          const bool take_max = (desc == lower);
          const bool o_gt = o > v[r];
          v[r] = (take_max == o_gt) ? o : v[r];
        }
      }
    }
  }
}

// Sort the compacted candidates (64-bit keys: average bits high, inverted block
// id low, so larger key = better score, then lower id) and write the first
// M_out <= 64 of them.  The running sum of raw scores is accumulated in rank
// order, one addition per rank, exactly like a sequential scan.
template <int E>
__device__ __forceinline__ void sorted_emit(const unsigned long long* cand, int count, int lane,
                                            const float* sraw, int M_out, float threshold,
                                            int32_t* oi, float* orw, float* oav) {
  unsigned long long v[E];
#pragma unroll
  for (int r = 0; r < E; r++) v[r] = (r * 32 + lane < count) ? cand[r * 32 + lane] : 0ull;
  bitonic_desc<E>(v, lane);
  // ranks lane (slot 0) and 32 + lane (slot 1, only when more than 32 are wanted)
  constexpr int SLOTS = E >= 2 ? 2 : 1;
  int id[SLOTS];
  float avg[SLOTS], raw[SLOTS], mycum[SLOTS];
#pragma unroll
  for (int q = 0; q < SLOTS; q++) {
    id[q] = static_cast<int>(0xffffffffu - static_cast<unsigned>(v[q]));
    avg[q] = __int_as_float(static_cast<int>(v[q] >> 32));
    raw[q] = (q * 32 + lane < M_out) ? sraw[id[q]] : 0.f;
    mycum[q] = 0.f;
  }
  float cum = 0.f;
  for (int p = 0; p < min(M_out, 32); p++) {
    cum += __shfl_sync(0xffffffffu, raw[0], p);
    if (p == lane) mycum[0] = cum;
  }
  if (SLOTS > 1)
    for (int p = 32; p < M_out; p++) {
      cum += __shfl_sync(0xffffffffu, raw[SLOTS - 1], p - 32);
      if (p - 32 == lane) mycum[SLOTS - 1] = cum;
    }
  // first rank whose running sum reaches the threshold
  int cutpos = 64;
#pragma unroll
  for (int q = SLOTS - 1; q >= 0; q--) {
    const unsigned m = __ballot_sync(0xffffffffu, (q * 32 + lane < M_out) && (mycum[q] >= threshold));
    if (m) cutpos = q * 32 + __ffs(m) - 1;
  }
#pragma unroll
  for (int q = 0; q < SLOTS; q++) {
    const int rank = q * 32 + lane;
    if (rank < M_out) {
      const bool keep = rank <= cutpos;
      oi[rank] = keep ? id[q] : -1;
      orw[rank] = keep ? raw[q] : 0.f;
      oav[rank] = keep ? avg[q] : 0.f;
    }
  }
}

// Register variant for M <= 32 * IPT (IPT a compile-time constant): the lane's
// IPT averages stay in registers, so the rescan after a pop is a fully
// unrolled compare/select chain with no shared-memory traffic, and the lane
// caches its runner-up so that most pops need no rescan at all.  Raw scores
// still sit in shared memory (one broadcast read per extracted element).
//
// When at most 32 entries are wanted (64 with at least 128 blocks) the kernel first tries a filter-and-sort
// path: every lane splits its slots into two groups and takes each group's
// maximum; the 64 maxima are 64 distinct entries, so the M_out-th largest of
// them (T) is a lower bound of the M_out-th largest entry overall, and
// {average >= T} holds every entry the result can contain (ties with T
// included).  That set is compacted with ballots (about 40 entries for
// M = 512), sorted as 64-bit keys and written.  The extraction loop below only
// runs when the set does not fit 128 candidates.
//
// `rawv` = the lane's slots of the row's M block sums (slot i = block i * 32 +
// lane, loaded by the caller so that it can have the next row's loads in
// flight); `scaled`: multiply by `inv_total` first (scoring hands over
// unnormalised sums and one total per row).  `sraw` (32 * IPT floats) and `cand`
// (128 keys, 256 when IPT >= 4, unused when IPT == 1) are the warp's own
// shared-memory scratch.
template <int IPT>
__device__ __forceinline__ void select_row_reg(const float (&rawv)[IPT], bool scaled,
                                               float inv_total, int M, int M_out, int bsz,
                                               int pad_head, int pad_tail, float threshold,
                                               float* sraw, unsigned long long* cand, int lane,
                                               int32_t* oi, float* orw, float* oav) {
  const bool pow2 = (bsz & (bsz - 1)) == 0;
  const float inv_bsz = 1.f / static_cast<float>(bsz);
  const int NEG = __float_as_int(-1.f);

  int a[IPT];   // average bit patterns (non-negative floats order as ints); NEG = absent
#pragma unroll
  for (int i = 0; i < IPT; i++) {
    const int j = i * 32 + lane;
    float raw = 0.f, avg = -1.f;
    if (j < M) {
      raw = rawv[i];
      if (scaled) raw *= inv_total;
      int n = bsz;
      if (j == 0) n -= pad_head;
      if (j == M - 1) n -= pad_tail;
      avg = (pow2 && n == bsz) ? raw * inv_bsz : __fdiv_rn(raw, static_cast<float>(n));
      if (!(avg >= 0.f)) avg = 0.f;
    }
    sraw[j] = raw;
    a[i] = __float_as_int(avg);
  }
  // best and runner-up of the lane; ties keep the lower slot (= lower id)
  int b1 = NEG, i1 = IPT, b2 = NEG, i2 = IPT;
  auto rescan = [&]() {
    b1 = NEG; i1 = IPT; b2 = NEG; i2 = IPT;
#pragma unroll
    for (int i = 0; i < IPT; i++) {
      const int v = a[i];
      if (v > b1) { b2 = b1; i2 = i1; b1 = v; i1 = i; }
      else if (v > b2) { b2 = v; i2 = i; }
    }
  };
  __syncwarp();

  // G group maxima per lane: 2 when at most 32 entries are wanted, 4 (with at
  // least 4 slots per lane) when at most 64 are: 32 * G distinct entries, so
  // their M_out-th largest bounds the M_out-th largest entry from below
  if constexpr (IPT >= 2) {
    constexpr int CAP = IPT >= 4 ? 256 : 128;     // candidate keys the warp's scratch holds
    const int G = M_out <= 32 ? 2 : 4;
    if (M_out <= 32 || (IPT >= 4 && M_out <= 64)) {
      int T;
      if (G == 2) {
        int gm[2] = {NEG, NEG};
#pragma unroll
        for (int i = 0; i < IPT; i++) gm[i >= IPT / 2] = max(gm[i >= IPT / 2], a[i]);
        bitonic_desc<2>(gm, lane);
        T = __shfl_sync(0xffffffffu, gm[0], M_out - 1);
      } else {
        int gm[4] = {NEG, NEG, NEG, NEG};
#pragma unroll
        for (int i = 0; i < IPT; i++) gm[(4 * i) / IPT] = max(gm[(4 * i) / IPT], a[i]);
        if constexpr (IPT >= 4) bitonic_desc<4>(gm, lane);
        const int hi = __shfl_sync(0xffffffffu, gm[1], (M_out - 1) & 31);
        const int lo = __shfl_sync(0xffffffffu, gm[0], (M_out - 1) & 31);
        T = (M_out - 1) >= 32 ? hi : lo;
      }
      if (T >= 0) {
        const unsigned lt = (1u << lane) - 1u;
        int count = 0;
#pragma unroll
        for (int i = 0; i < IPT; i++) {
          const bool c = a[i] >= T;
          const unsigned bal = __ballot_sync(0xffffffffu, c);
          const int pos = count + __popc(bal & lt);
          if (c && pos < CAP)
            cand[pos] = (static_cast<unsigned long long>(static_cast<unsigned>(a[i])) << 32) |
                        (0xffffffffu - static_cast<unsigned>(i * 32 + lane));
          count += __popc(bal);
        }
        __syncwarp();
        if (count <= CAP) {
          if (count <= 32 && M_out <= 32)
            sorted_emit<1>(cand, count, lane, sraw, M_out, threshold, oi, orw, oav);
          else if (count <= 64)
            sorted_emit<2>(cand, count, lane, sraw, M_out, threshold, oi, orw, oav);
          else if (count <= 128)
            sorted_emit<4>(cand, count, lane, sraw, M_out, threshold, oi, orw, oav);
          else
            sorted_emit<8>(cand, count, lane, sraw, M_out, threshold, oi, orw, oav);
          return;
        }
      }
    }
  }
  rescan();

  float cum = 0.f;
  bool cut = false;
  int hold_idx = -1;
  float hold_raw = 0.f, hold_avg = 0.f;
  for (int r = 0; r < M_out; r++) {
    int w_idx = -1;
    float w_raw = 0.f, w_avg = 0.f;
    if (!cut) {
      const int mx = redux_max_s32(b1);
      const unsigned mine =
          (b1 == mx) ? static_cast<unsigned>(i1 * 32 + lane) : 0xffffffffu;
      const unsigned win = redux_min_u32(mine);
      w_idx = static_cast<int>(win);
      w_raw = sraw[win];
      w_avg = __int_as_float(mx);
      cum += w_raw;
      if (cum >= threshold) cut = true;
      if ((win & 31u) == static_cast<unsigned>(lane)) {
        // pop: the slot is consumed; promote the runner-up, rescan only when
        // there is none cached
#pragma unroll
        for (int i = 0; i < IPT; i++)
          if (i == i1) a[i] = NEG;
        if (i2 < IPT) {
          b1 = b2; i1 = i2; b2 = NEG; i2 = IPT;
        } else {
          rescan();
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

}  // namespace ftk
