// Test-only translation unit (not part of libftk_sm100.so): drives the bounded
// waits of csrc/ftk_sm100.cuh until they give up.  Built with a short
// FTK_WAIT_CYCLES so a wait runs out after ~0.1 ms.  One CTA, no TMA and no
// tcgen05 instruction in flight: a wait that runs out records its code, raises
// the CTA's abort flag and returns, and the kernel ends normally.
#include "ftk_sm100.cuh"

using namespace ftk;

// trace[0]: warp 0's wait result      (expected 0: ran out or saw the flag)
// trace[1]: abort flag after the waits (expected 1)
// trace[2]: warp 1's wait result      (expected 0)
// trace[3]: mbar_wait_all over {completed, never completed} (expected 0)
// trace[4]: wait on a barrier that did complete (expected 1)
// trace[5]: clock ticks warp 0 spent in its wait
__global__ void wait_probe_kernel(int* status, int* trace) {
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  const uint32_t never = smem_u32(&bars[0]), done = smem_u32(&bars[1]);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(never, 1);
    mbar_init(done, 1);
    mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_arrive(done);   // phase 0 of `done` completes
  __syncthreads();
  WaitCtx w{&abort_flag, status};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    const long long t0 = clock64();
    // nobody ever arrives on `never`
    const bool ok = mbar_wait(never, 0, w, warp == 0 ? FTK_DEV_TIMEOUT_TMA : FTK_DEV_TIMEOUT_CONSUMER);
    if (warp == 0) {
      trace[0] = ok ? 1 : 0;
      trace[5] = static_cast<int>(clock64() - t0);
    } else {
      trace[2] = ok ? 1 : 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    trace[1] = abort_flag;
    const uint32_t b[2] = {done, never};
    const uint32_t ph[2] = {0u, 0u};
    trace[3] = mbar_wait_all<2>(b, ph, w, FTK_DEV_TIMEOUT_MMA) ? 1 : 0;
    trace[4] = mbar_wait(done, 0, w, FTK_DEV_TIMEOUT_EPILOGUE) ? 1 : 0;
  }
}

// status may be null: the waits must still give up cleanly (only the code is lost)
extern "C" int ftk_wait_probe(int32_t* status, int32_t* trace, void* stream) {
  if (!trace) return -1;
  wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, trace);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" long long ftk_wait_probe_cycles(void) { return FTK_WAIT_CYCLES; }
