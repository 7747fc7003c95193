// Device-side helpers shared by the UMMA kernels: bounded mbarrier waits that turn a
// would-be hang into a status code, and the status codes themselves.
#pragma once

#include "sm100_ptx.cuh"

namespace beam {

// Values written to the device status word (0 = healthy). The host maps any non-zero
// value to BEAM_ERR_DEVICE_TIMEOUT and reports the raw word through beam_device_status().
enum DeviceFault : int {
  kFaultNone = 0,
  kFaultProducerWait = 0x101,  // TMA producer gave up waiting for a free pipeline stage
  kFaultMmaWaitFull = 0x102,   // MMA issuer gave up waiting for operand bytes
  kFaultMmaWaitAcc = 0x103,    // MMA issuer gave up waiting for a drained accumulator
  kFaultEpilogueWait = 0x104,  // epilogue gave up waiting for a finished accumulator
  kFaultReduceWait = 0x105,    // split-K / LayerNorm exchange wait ran out
};

// Every spin in these kernels goes through here. A wait gives up after kWaitLimitNs of wall
// time (or at once when another role of this CTA already gave up): it raises the CTA-wide
// abort flag, records `fault` in the global status word and returns false; callers then leave
// their role loops and fall through to the common teardown, which still frees TMEM.
constexpr uint64_t kWaitLimitNs = 2000ull * 1000ull * 1000ull;
constexpr uint32_t kSpinSuspendNs = 4000u;

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* cta_abort,
                                             int* status_word, int fault, uint64_t limit_ns = kWaitLimitNs) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spin = 1;; ++spin) {
    // suspended in hardware until the phase completes or kSpinSuspendNs pass: few instructions while waiting
    if (ptx::mbar_try_wait_suspend(bar, parity, kSpinSuspendNs)) return true;
    if ((spin & 0x3Fu) == 0) {
      if (*cta_abort) return false;
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *cta_abort = 1;
        if (status_word) atomicCAS(status_word, 0, fault);
        return false;
      }
    }
  }
}

// The same wait for whole warps (the epilogue, which sleeps through a tile's main loop): only lane 0 waits, suspended
// in hardware on the barrier for up to kSuspendNs at a time instead of polling, and the rest of the warp parks at
// the shuffle.  Returns the same value in every lane.
constexpr uint32_t kSuspendNs = 50000u;

__device__ __forceinline__ bool bounded_wait_warp(uint32_t bar, uint32_t parity, volatile int* cta_abort,
                                                  int* status_word, int fault, uint32_t lane,
                                                  uint64_t limit_ns = kWaitLimitNs) {
  int ok = 1;
  if (lane == 0) {
    if (!ptx::mbar_try_wait(bar, parity)) {
      uint64_t t0 = 0;
      for (uint32_t spin = 1;; ++spin) {
        if (ptx::mbar_try_wait_suspend(bar, parity, kSuspendNs)) break;
        if ((spin & 0xFu) == 0) {
          if (*cta_abort) {
            ok = 0;
            break;
          }
          const uint64_t now = ptx::globaltimer_ns();
          if (t0 == 0) {
            t0 = now;
          } else if (now - t0 > limit_ns) {
            *cta_abort = 1;
            if (status_word) atomicCAS(status_word, 0, fault);
            ok = 0;
            break;
          }
        }
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// After an abort, give asynchronous work this CTA already issued (TMA copies into its shared
// memory, UMMAs into its TMEM) time to land before shared memory and TMEM are released.
__device__ __forceinline__ void abort_drain_delay() {
  const uint64_t t0 = ptx::globaltimer_ns();
  while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
}

}  // namespace beam
