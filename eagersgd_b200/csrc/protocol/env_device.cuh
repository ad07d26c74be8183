// Device instantiation of the protocol environment: system-scope PTX atomics on
// peer-mapped memory (own HBM and the other GPUs' HBM over NVLink / NVSwitch).
#pragma once
#include <stdint.h>

namespace esgd {

struct DevEnv {
  static __device__ __forceinline__ uint64_t ld_acq64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st_rel64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  }
  static __device__ __forceinline__ void st_rlx64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
  }
  static __device__ __forceinline__ void st_rlx32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  }
  static __device__ __forceinline__ uint32_t ld_acq32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st_rel32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  }
  static __device__ __forceinline__ uint64_t cas64(uint64_t* p, uint64_t expect, uint64_t desired) {
    uint64_t old;
    asm volatile("atom.acq_rel.sys.global.cas.b64 %0, [%1], %2, %3;"
                 : "=l"(old) : "l"(p), "l"(expect), "l"(desired) : "memory");
    return old;
  }
  static __device__ __forceinline__ uint32_t cas32(uint32_t* p, uint32_t expect, uint32_t desired) {
    uint32_t old;
    asm volatile("atom.acq_rel.sys.global.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old) : "l"(p), "r"(expect), "r"(desired) : "memory");
    return old;
  }
  static __device__ __forceinline__ uint32_t add32(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
  }
  static __device__ __forceinline__ void fence() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
  static __device__ __forceinline__ void fence_sc() { asm volatile("fence.sc.sys;" ::: "memory"); }
  static __device__ __forceinline__ uint64_t now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
  }
  static __device__ __forceinline__ void pause() { __nanosleep(100); }
};

}  // namespace esgd
