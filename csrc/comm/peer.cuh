// Cross-GPU signalling over peer-mapped memory: system-scope release stores and
// acquire loads on 32-bit sequence words, with bounded spins.  Every rank owns a
// small "flag page" that all peers map; word [slot * kMaxRanks + r] of rank d's
// page is written only by rank r.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ft {
namespace peer {

constexpr int kMaxRanks = 8;
constexpr long long kSpinCycles = 20000000000LL;   // ~10 s at 1.9 GHz: ranks are at most one unit apart

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sequence numbers only grow; (a - b) as signed handles wrap-around.
__device__ __forceinline__ bool seq_reached(uint32_t have, uint32_t want) {
  return (int32_t)(have - want) >= 0;
}

// Spin until *p >= want.  False when the budget (clock cycles) ran out.
__device__ __forceinline__ bool wait_seq(const uint32_t* p, uint32_t want, long long budget) {
  if (seq_reached(ld_acquire_sys(p), want)) return true;
  const long long t0 = clock64();
  while (!seq_reached(ld_acquire_sys(p), want)) {
    if (clock64() - t0 > budget) return false;
    __nanosleep(64);
  }
  return true;
}

struct Peers {
  int world;
  int rank;
  uint32_t* flags[kMaxRanks];   // flag page of every rank (own page included), peer-mapped
};

}  // namespace peer
}  // namespace ft
