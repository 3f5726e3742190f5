// Flagged-word hand-off ("LL" protocol): data and its ready flag travel in one 8-byte
// store, so a producer needs no fence and no separate event, and a consumer's poll is
// already its load.  Word = {two 16-bit values, 32-bit tag}; an aligned 8-byte access is
// single-copy atomic, so a word is either old or new, never torn.  The tag is
// (iterations since the library was created << 8) | producing operator, which differs from
// whatever the same buffer held before (the previous layer's or iteration's words).
//
// The reference hands every intermediate over through its event queue
// (persistent_kernel.cuh:454-974); this replaces that for edges whose readers are all
// LINEAR (or ALLREDUCE) tasks, when at most 8 tokens are in flight.
#pragma once
#include "device_common.cuh"

namespace ypk {

__device__ __forceinline__ uint32_t ll_tag(const Runtime &rt, long long iter, int id) {
  return (static_cast<uint32_t>(rt.ll_epoch + static_cast<unsigned long long>(iter)) << 8) |
         (static_cast<uint32_t>(id) & 255u);
}
__device__ __forceinline__ unsigned long long ll_word(uint32_t data, uint32_t tag) {
  return static_cast<unsigned long long>(data) | (static_cast<unsigned long long>(tag) << 32);
}
__device__ __forceinline__ void ll_store(unsigned long long *p, unsigned long long w) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_store_sys(unsigned long long *p, unsigned long long w) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Two neighbouring words (16-byte aligned).  Each is atomic on its own.
__device__ __forceinline__ void ll_load2(const unsigned long long *p, unsigned long long &a,
                                         unsigned long long &b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ bool ll_ok(unsigned long long w, uint32_t tag) {
  return static_cast<uint32_t>(w >> 32) == tag;
}

// Bounded polling state of one thread.
struct LLPoll {
  uint32_t spins = 0;
  unsigned long long t0 = 0;
  bool failed = false;
  // Call after an unsuccessful try; returns false when the thread should give up.
  __device__ __forceinline__ bool again(const WaitCtx &wc) {
    if (failed) return false;
    ++spins;
    if (spins > 16u) __nanosleep(32);
    if ((spins & 127u) == 0u) {
      if (t0 == 0) t0 = globaltimer();
      const bool seen = abort_seen(wc);
      if (seen || globaltimer() - t0 > wc.rt->budget_ns) {
        if (!seen) raise_abort(wc, YPK_ERR_TIMEOUT, -6);
        failed = true;
        return false;
      }
    }
    return true;
  }
};

}  // namespace ypk
