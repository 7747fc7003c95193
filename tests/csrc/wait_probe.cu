// Test-only translation unit (never linked into libbeam_b200.so): makes the kernels' bounded waits run out.
//
// Every wait in the product kernels goes through bounded_wait / bounded_wait_warp (csrc/umma_common.cuh), which
// give up after a time limit, raise the CTA-wide abort flag, record a fault code and return so that the common
// teardown still runs.  In the product that limit is two seconds and is never reached.  This probe calls the same
// functions with a limit passed by the host (about a millisecond) on mbarriers that are initialised and that
// nothing ever arrives on: each role's wait expires, the fault word is written, the teardown (drain delay, CTA
// barrier, TMEM release) completes and the kernel returns.  It is a wait with a short limit that gives up: no
// trap, no assert, no endless loop, and the context stays usable.
#include <cuda_runtime.h>

#include "../../general-nvgpu-testing_b200/csrc/umma_common.cuh"

namespace {

// words of `out`: [0] producer wait returned (1 = barrier completed, 0 = gave up), [1] same for the warp-wide
// wait of warp 2, [2] CTAs that reached the end of the teardown, [3] longest wait in microseconds
__global__ void __launch_bounds__(128, 1) wait_probe_kernel(int* status_word, int* out, unsigned long long limit_ns) {
  using namespace beam;
  __shared__ __align__(8) unsigned long long bars[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int cta_abort_flag;
  volatile int* cta_abort = &cta_abort_flag;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar0 = ptx::smem_u32(&bars[0]), bar1 = ptx::smem_u32(&bars[1]);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar0, 1);  // one arrival expected; nobody arrives
    ptx::mbar_init(bar1, 1);
    cta_abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {  // the same TMEM life cycle as the GEMM kernels: allocated at set-up, freed in the teardown
    ptx::tmem_alloc<1>(ptx::smem_u32(&tmem_slot), 32);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const uint64_t t0 = ptx::globaltimer_ns();
  if (warp == 0) {
    if (lane == 0) {  // the producer's wait for a free stage
      const bool ok = bounded_wait(bar0, 0, cta_abort, status_word, kFaultProducerWait, limit_ns);
      atomicExch(out + 0, ok ? 1 : 0);
      atomicMax(out + 3, static_cast<int>((ptx::globaltimer_ns() - t0) / 1000));
    }
  } else if (warp == 2) {  // an epilogue warp's wait for a finished accumulator
    const bool ok = bounded_wait_warp(bar1, 0, cta_abort, status_word, kFaultEpilogueWait, lane, limit_ns);
    if (lane == 0) {
      atomicExch(out + 1, ok ? 1 : 0);
      atomicMax(out + 3, static_cast<int>((ptx::globaltimer_ns() - t0) / 1000));
    }
  }
  // common teardown, as at the end of every product kernel
  __syncwarp();
  if (*cta_abort) abort_drain_delay();
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, 32);
  }
  if (threadIdx.x == 0) atomicAdd(out + 2, 1);
}

}  // namespace

// Launches `ctas` CTAs of the probe on `stream` with the given wait limit.  status_word and out are device
// pointers (1 and 4 ints, zeroed by the caller).  Returns the cudaError_t of the launch.
extern "C" __attribute__((visibility("default"))) int wait_probe_launch(int* status_word, int* out, int ctas,
                                                                        unsigned long long limit_ns, void* stream) {
  if (ctas < 1 || ctas > 1024) return static_cast<int>(cudaErrorInvalidValue);
  wait_probe_kernel<<<ctas, 128, 0, static_cast<cudaStream_t>(stream)>>>(status_word, out, limit_ns);
  return static_cast<int>(cudaGetLastError());
}
