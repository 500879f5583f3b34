// Host-side helpers shared by the launchers: error codes, tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda, so the
// library also loads on machines without a driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace ftk {

// C-ABI return codes (mirrored in include/ftk_api.h)
enum : int {
  FTK_OK = 0,
  FTK_ERR_BAD_ARG = -1,
  FTK_ERR_UNSUPPORTED = -2,
  FTK_ERR_WORKSPACE = -3,
  FTK_ERR_CUDA = -4,
  FTK_ERR_DRIVER = -5,
  FTK_ERR_CAPACITY = -6,
};

enum : int { FTK_DTYPE_F16 = 0, FTK_DTYPE_BF16 = 1 };

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tensor map over a 16-bit tensor addressed as [b][n][h][d] with element
// strides (sb, sn, sh) and unit stride along d.  Box = box_d x 1 x box_rows x 1
// (d, h, n, b), 128-byte swizzle, out-of-range elements read as zero.
// Coordinates at load time are (d0, h, n0, b).
inline int encode_tmap_bnhd(CUtensorMap* out, const void* base, int dtype, int64_t B, int64_t N,
                            int64_t H, int64_t D, int64_t sb, int64_t sn, int64_t sh, int box_d,
                            int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return FTK_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return FTK_ERR_BAD_ARG;
  if (((sb * 2) & 15) || ((sn * 2) & 15) || ((sh * 2) & 15)) return FTK_ERR_BAD_ARG;
  if (box_d * 2 > 128 || box_rows > 256 || box_rows < 1) return FTK_ERR_BAD_ARG;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)N, (cuuint64_t)B};
  // a stride of an extent-1 dimension is never used for addressing but must
  // still be a legal value
  cuuint64_t strides[3] = {(cuuint64_t)(sh > 0 ? sh : D) * 2, (cuuint64_t)(sn > 0 ? sn : D) * 2,
                           (cuuint64_t)(sb > 0 ? sb : D) * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_d, 1u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUtensorMapDataType dt =
      dtype == FTK_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FTK_OK : FTK_ERR_DRIVER;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace ftk
