// Device side of the expert-parallel hand-shakes (EpSync, common.cuh): system-scope flag words
// in the ranks' symmetric buffers, bounded waits, "last block raises the flag".
#pragma once
#include "common.cuh"

namespace moe {
namespace epsync {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *flag >= epoch (epochs only grow). False on timeout, with
// MOE_B200_DEV_TIMEOUT and the wait site in the status words.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, int32_t* status,
                                          int where) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  // an earlier wait of this call already gave up: do not stack time-outs
  if (*reinterpret_cast<const volatile int32_t*>(status) != MOE_B200_DEV_OK) return false;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((it & 63u) == 0) {
      if (global_ns() - t0 > kWaitLimitNs) {
        atomicMax(&status[0], MOE_B200_DEV_TIMEOUT);
        status[1] = where;
        return false;
      }
      __nanosleep(200);
    }
  }
}

// Threads 0 .. world-1 of the block wait for one flag each; returns (to every thread, after a
// block barrier) whether all arrived. No-op (true) when the kernel was given nothing to wait for.
__device__ __forceinline__ bool block_wait(const EpSync& sy, int32_t* status, int where) {
  if (sy.wait_flags == nullptr) return true;
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < sy.world) {
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(sy.epoch);
    if (!wait_flag(sy.wait_flags + threadIdx.x, epoch, status, where)) s_ok = 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// Called by every thread of every block at the end of the kernel, after its peer stores: the
// last block to arrive raises this rank's word on every rank. No-op without a counter.
__device__ __forceinline__ void grid_signal(const EpSync& sy) {
  if (sy.done_counter == nullptr) return;
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(sy.done_counter, 1u);
    s_last = (prev == gridDim.x - 1);
    __threadfence_system();
  }
  __syncthreads();
  if (s_last && (int)threadIdx.x < sy.world) {
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(sy.epoch);
    st_release_sys(sy.signal_flags[threadIdx.x], epoch);
  }
}

}  // namespace epsync
}  // namespace moe
