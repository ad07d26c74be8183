// Host instantiation of the protocol environment: GCC atomics on memory shared
// between threads or processes (POSIX shared memory).
#pragma once
#include <stdint.h>
#include <time.h>
#include <sched.h>

namespace esgd {

struct HostEnv {
  static inline uint64_t ld_acq64(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
  static inline void st_rel64(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
  // On the host a release store costs nothing extra (x86: a plain store), and ThreadSanitizer does not
  // model "fence, then relaxed stores": the grouped stores of the protocol are release stores here.
  static inline void st_rlx64(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
  static inline void st_rlx32(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
  static inline uint32_t ld_acq32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
  static inline void st_rel32(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
  static inline uint64_t cas64(uint64_t* p, uint64_t expect, uint64_t desired) {
    __atomic_compare_exchange_n(p, &expect, desired, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
    return expect;
  }
  static inline uint32_t cas32(uint32_t* p, uint32_t expect, uint32_t desired) {
    __atomic_compare_exchange_n(p, &expect, desired, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
    return expect;
  }
  static inline uint32_t add32(uint32_t* p, uint32_t v) { return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL); }
  static inline void fence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
  static inline void fence_sc() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
  static inline uint64_t now_ns() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
  }
  static inline void pause() { sched_yield(); }
};

}  // namespace esgd
