// Pieces shared by the sparse-attention kernels (forward, dQ, dK/dV).
//
// A CTA works on a 128-row tile made of G "groups" (q-blocks in the forward
// and dQ kernels, kv-blocks in the dK/dV kernel).  Each group brings its own
// list of partner blocks; the CTA walks the UNION of those lists in ascending
// block order and masks, per row, the partners its group does not list.  With
// 64-row blocks this fills the 128-row UMMA tile; where neighbouring groups
// list the same partners (the common case) no work is wasted.
#pragma once

#include "ftk_sm100.cuh"

namespace ftk {

constexpr int AT_MAX_GROUPS = 8;      // groups per 128-row tile
constexpr int AT_MAX_BLOCKS = 4096;   // partner blocks per slice
constexpr int AT_WORDS = AT_MAX_BLOCKS / 32;

struct UnionScratch {
  unsigned bm[AT_MAX_GROUPS][AT_WORDS];  // membership bitmaps
  uint16_t ids[AT_MAX_BLOCKS];           // union, ascending
  uint8_t masks[AT_MAX_BLOCKS];          // bit g set: group g lists the block
  int warp_tot[4];
  int total;
};

// All threads of the CTA call this.  `rows` points at the first group's list,
// consecutive groups `row_stride` entries apart; each list is read up to
// `width` entries (or counts[g] when given), negative ids skipped, ids >=
// num_blocks reported through `status`.  Returns the union size.
__device__ __forceinline__ int build_union(UnionScratch& u, const int32_t* rows, int64_t row_stride,
                                           int groups, int width, const int32_t* counts,
                                           int num_blocks, int* status) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int words = (num_blocks + 31) >> 5;
  for (int i = tid; i < AT_MAX_GROUPS * AT_WORDS; i += nthr) (&u.bm[0][0])[i] = 0u;
  __syncthreads();
  for (int g = 0; g < groups; g++) {
    const int cnt = counts ? min(counts[g], width) : width;
    const int32_t* row = rows + g * row_stride;
    for (int e = tid; e < cnt; e += nthr) {
      const int j = row[e];
      if (j < 0) continue;
      if (j >= num_blocks) {
        if (status) atomicCAS(status, 0, FTK_DEV_BAD_INDEX);
        continue;
      }
      atomicOr(&u.bm[g][j >> 5], 1u << (j & 31));
    }
  }
  __syncthreads();
  // 128 threads: one bitmap word each, block-wide exclusive scan of popcounts
  unsigned uni = 0;
  int c = 0;
  if (tid < AT_WORDS && tid < words) {
#pragma unroll
    for (int g = 0; g < AT_MAX_GROUPS; g++) uni |= u.bm[g][tid];
    c = __popc(uni);
  }
  if (tid < 128) {
    const int lane = tid & 31, wp = tid >> 5;
    int inc = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += v;
    }
    if (lane == 31) u.warp_tot[wp] = inc;
    __syncwarp();
    // stash the inclusive value; offsets added after the barrier below
    c = inc - c;  // exclusive within warp
  }
  __syncthreads();
  if (tid < 128) {
    const int wp = tid >> 5;
    int off = 0;
    for (int q = 0; q < wp; q++) off += u.warp_tot[q];
    int pos = off + c;
    unsigned bits = uni;
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      unsigned mk = 0;
#pragma unroll
      for (int g = 0; g < AT_MAX_GROUPS; g++) mk |= ((u.bm[g][tid] >> b) & 1u) << g;
      u.ids[pos] = static_cast<uint16_t>(tid * 32 + b);
      u.masks[pos] = static_cast<uint8_t>(mk);
      pos++;
    }
    if (tid == 127) u.total = u.warp_tot[0] + u.warp_tot[1] + u.warp_tot[2] + u.warp_tot[3];
  }
  __syncthreads();
  return u.total;
}

// two fp32 -> one 32-bit word of two 16-bit floats (element 0 in the low half)
__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
  if (fmt == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack2(uint32_t w, int fmt) {
  if (fmt == 1) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  }
  return __half22float2(*reinterpret_cast<__half2*>(&w));
}

}  // namespace ftk
