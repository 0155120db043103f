// Cross-GPU epoch flags: 32-bit words in the owner's symmetric arena, written by peers with
// system-scope release stores and polled with acquire loads. Every wait is bounded twice (a time limit
// on the global timer and a poll count); a wait that runs out returns false and the caller records a
// status code and carries on, so a missing peer ends in a host-side error instead of a hung GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mtb {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag >= epoch (wrap-safe) for at most `limit_us` microseconds.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint32_t limit_us) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  const unsigned long long budget = static_cast<unsigned long long>(limit_us) * 1000ull;
  for (uint32_t i = 0; i < 0x7fffffffu; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    __nanosleep(200);
    if ((i & 31u) == 31u) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > budget) return false;
    }
  }
  return false;
}

// Default bound of a wait on a peer's flag, in microseconds. It has to cover legitimate skew between
// ranks (one rank holding an over-length sample, a first-touch allocation of pinned memory), which at 70B
// scale is tens of seconds; a peer that is really gone still ends the wait, just later. Tests pass a
// bound of a few milliseconds.
constexpr uint32_t FLAG_SPIN_LIMIT = 180u * 1000u * 1000u;

}  // namespace mtb
