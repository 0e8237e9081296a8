// Definitions shared by the causal flash-attention kernels (attention_fwd2.cuh,
// attention_bwd.cuh): tile sizes, the forward parameter block and the
// 128-byte swizzle of a [rows][64] shared-memory chunk.
#pragma once
#include "common.cuh"
#include "tcgen05.cuh"

namespace ft {
namespace attn {

using namespace ft::sm100;

constexpr int BQ = 128, BKV = 128, KV_STAGES = 2;

struct FwdParams {
  void* o;                 // [B, S, Hq, D] contiguous
  float* lse;              // [B, Hq, S]: natural log of sum exp(scale * s) per query row
  int B, S, Hq, Hkv;
  float scale_log2;        // softmax scale * log2(e)
  float scale_ln;          // softmax scale
  int q_col0, k_col0, v_col0;   // column of head 0 inside the respective tensor map rows
  int* err;
  // timeline capture (TRACE instantiation only): clock64() of CTA trace_cta at the hand-over points
  // of K/V blocks trace_it0 .. trace_it0 + 7, as trace[(role * 8 + site) * 8 + block]
  long long* trace;
  int trace_cta, trace_it0;
};

// byte offset of 16-byte unit `u` (0..7) of row `r` inside a 128B-swizzled [rows][64] chunk
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t u) {
  return (r >> 3) * 1024 + (r & 7) * 128 + ((u ^ (r & 7)) << 4);
}

}  // namespace attn
}  // namespace ft
