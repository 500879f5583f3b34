// Version and error-text entry points of the C ABI.
#include "ftk_host.cuh"
#include "ftk_sm100.cuh"

extern "C" int ftk_version(void) { return 100; }  // 0.1.0

extern "C" const char* ftk_error_string(int code) {
  switch (code) {
    case ftk::FTK_OK: return "ok";
    case ftk::FTK_ERR_BAD_ARG: return "bad argument (shape, range or alignment)";
    case ftk::FTK_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case ftk::FTK_ERR_WORKSPACE: return "workspace missing or too small";
    case ftk::FTK_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
    case ftk::FTK_ERR_DRIVER: return "tensor-map encoding unavailable or failed";
    case ftk::FTK_ERR_CAPACITY:
      return "problem exceeds the fixed buffer of a no-allocation entry point";
    case ftk::FTK_DEV_TIMEOUT_TMA: return "device: TMA producer wait timed out";
    case ftk::FTK_DEV_TIMEOUT_MMA: return "device: UMMA issuer wait timed out";
    case ftk::FTK_DEV_TIMEOUT_CONSUMER: return "device: consumer wait timed out";
    case ftk::FTK_DEV_TIMEOUT_EPILOGUE: return "device: epilogue wait timed out";
    case ftk::FTK_DEV_BAD_INDEX: return "device: block index out of range";
    default: return "unknown code";
  }
}
