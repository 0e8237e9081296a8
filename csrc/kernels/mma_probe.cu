// Rate of 128-deep tcgen05 products (eight 128xNx16 instructions) as a single CTA sees it, measured
// in SM clocks by the issuing warp itself.  One CTA per SM holds fixed zero-filled tiles in shared
// memory and issues `rounds` products back to back; clock64() around them gives the time per
// product.  benchmarks/mma_rate.py runs the modes; what they showed on a B200:
//   * the pipe executes 128-wide instructions at its full rate (64 clocks each) wherever the
//     operands are - shared memory in either major, A in tensor memory - as long as the issuing
//     thread does nothing else between them;
//   * its queue covers about two instructions, so whatever the issuing thread does between two
//     products beyond ~128 clocks (a barrier wait, a fence, a commit, branches) is time the pipe
//     stands still: 150-220 clocks per product in the form a pipelined kernel needs;
//   * a whole warp that runs the loop and elects one lane to issue loses less than a lone
//     thread inside `if (lane == 0)`.
//
// Operands (OPS):  0  A, B K-major in shared memory, N = 128      (S = Q K^T, dP = dO V^T)
//                  1  A, B MN-major in shared memory, N = 128     (dV = P^T dO, dK = dS^T Q)
//                  2  A K-major, B MN-major in shared memory      (dQ = dS K)
//                  3  A in tensor memory, B MN-major, N = 128     (O += P V)
//                  4  A, B K-major in shared memory, N = 256
//                  5  a pair per round, as the attention forward issues them: O += P V with P read from
//                     tensor-memory columns 0-63, then S = Q K^T written over columns 0-127 (the
//                     columns P was just read from)      6  the same pair with S written elsewhere
// Issue (STYLE):   0  elected lane of a whole warp, nothing between the products
//                  1  per product: barrier wait (succeeds at once), tcgen05 fence, product, commit;
//                     issued inside `if (lane == 0)`
//                  2  the same, whole warp with an elected issuer
//                  3  as 2, but the barrier of the NEXT product is looked at (mbarrier.test_wait)
//                     between the sixth and the seventh instruction of this one, while the pipe
//                     still has queued work; the blocking wait remains only for a miss
// Others (DISTURB): 0 idle   1 four warps keep loading tensor memory   2 four warps keep storing
//                     to shared memory   3 eight warps keep computing exponentials (special-function
//                     unit and fma pipe, no memory)   4 four warps keep storing to tensor memory
//                     (the columns the A operand of OPS 3 is read from)
//   mode = OPS (0-4, STYLE 0, idle) | 5, 6 = OPS 0 with STYLE 1, 2 | 7, 8 = OPS 0, STYLE 0 with
//   DISTURB 1, 2 | 9 = OPS 3, STYLE 0, DISTURB 1 | 10 = OPS 0 with STYLE 3 |
//   11, 12 = OPS 0, 3 with DISTURB 3 | 13 = OPS 3 with DISTURB 4 | 14, 15 = OPS 5, 6 (clocks per pair)
#include "common.cuh"
#include "gemm_host.h"
#include "tcgen05.cuh"

namespace {

using namespace ft;
using namespace ft::sm100;

constexpr int kProbeThreads = 320;                   // warp 0 issues, warp 1 owns tensor memory, 2-9 disturb
constexpr int kChunk = 128 * 128;                    // [128 rows][64 columns] of 16-bit values
constexpr int kSmem = 2 * kChunk /* A */ + 4 * kChunk /* B, up to 256 rows */ + 32 * 1024 /* scratch */ + 2048;

struct ProbeBars {
  uint64_t done, idle, fresh;
  uint32_t tmem_base;
  volatile uint32_t stop;
};

// One product: eight instructions on the tiles at offsets a_off / b_off (bytes, uniform).
template <int OPS, int KK0 = 0, int KK1 = 8>
__device__ __forceinline__ void issue_product(uint32_t acc, uint32_t tmem_a, uint32_t aA, uint32_t aB, bool first);

// OPS 5 / 6: the pair PV, QK
template <int OPS>
__device__ __forceinline__ void issue_pair(uint32_t tmem, uint32_t aA, uint32_t aB, bool first) {
  issue_product<3>(tmem + 256, tmem, aA, aB, first);
  issue_product<0>(tmem + (OPS == 5 ? 0 : 128), tmem, aA, aB, true);
}

template <int OPS, int KK0, int KK1>
__device__ __forceinline__ void issue_product(uint32_t acc, uint32_t tmem_a, uint32_t aA, uint32_t aB, bool first) {
  constexpr uint32_t hi = smem_desc_hi(1024);
  constexpr uint32_t idesc = make_idesc_f16(1, OPS == 1, OPS == 1 || OPS == 2 || OPS == 3, 128, OPS == 4 ? 256 : 128);
  const uint32_t a_lo = smem_desc_lo(aA, OPS == 1 ? kChunk : 16);
  const uint32_t b_lo = smem_desc_lo(aB, (OPS == 0 || OPS == 4) ? 16 : kChunk);
#pragma unroll
  for (int kk = KK0; kk < KK1; ++kk) {
    const uint32_t k_off = ((kk / 4) * kChunk + (kk % 4) * 32) >> 4;            // K-major, 128 rows
    const uint32_t k_off256 = ((kk / 4) * 2 * kChunk + (kk % 4) * 32) >> 4;     // K-major, 256 rows
    const uint32_t mn_off = (kk * 2048) >> 4;                                    // MN-major
    const uint64_t ad = smem_desc_join(a_lo + (OPS == 1 ? mn_off : k_off), hi);
    const uint64_t bd = smem_desc_join(b_lo + (OPS == 0 ? k_off : OPS == 4 ? k_off256 : mn_off), hi);
    if constexpr (OPS == 3) umma_f16_ts(acc, tmem_a + kk * 8, bd, idesc, !first || kk != 0);
    else umma_f16(acc, ad, bd, idesc, !first || kk != 0);
  }
}

template <int OPS, int STYLE, int DISTURB>
__global__ void __launch_bounds__(kProbeThreads, 1)
mma_probe_kernel(int rounds, int wobble, long long* __restrict__ out, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + 2 * kChunk;
  uint8_t* sX = sB + 4 * kChunk;
  ProbeBars* bars = reinterpret_cast<ProbeBars*>(sX + 32 * 1024);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < (6 * kChunk + 32 * 1024) / 16; i += kProbeThreads)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(&bars->done, 1);
    mbar_init(&bars->idle, 1);                       // receives commits, nobody waits
    mbar_init(&bars->fresh, 1);                      // never completes: waiting for parity 1 succeeds at once
    bars->stop = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    // the tile addresses change from round to round (by an offset that is zero at run time, which
    // the compiler cannot know), as a kernel's stages do: no descriptor is loop-invariant
    const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
    if constexpr (STYLE == 1) {
      if (lane == 0) {
        const long long t0 = clock64();
        bool ok = true;
        for (int r = 0; r < rounds; ++r) {
          if (!mbar_wait(&bars->fresh, 1)) { ok = false; break; }
          tc_fence_after();
          issue_product<OPS>(tmem + 256, tmem, aA + (r & 1) * wobble, aB + (r & 1) * wobble, r == 0);
          umma_commit(&bars->idle);
        }
        umma_commit(&bars->done);
        ok = ok && mbar_wait(&bars->done, 0);
        const long long t1 = clock64();
        if (!ok) atomicCAS(err, 0, 501);
        out[blockIdx.x] = t1 - t0;
        bars->stop = 1;
      }
    } else if constexpr (STYLE == 3) {
      const long long t0 = clock64();
      bool ok = true, ready = false;
      for (int r = 0; r < rounds && ok; ++r) {
        if (!ready) ok = __all_sync(0xffffffffu, mbar_wait(&bars->fresh, 1)) != 0;
        tc_fence_after();
        if (elect_one())
          issue_product<OPS, 0, 6>(tmem + 256, tmem, aA + (r & 1) * wobble, aB + (r & 1) * wobble, r == 0);
        __syncwarp();
        ready = __all_sync(0xffffffffu, mbar_test(&bars->fresh, 1)) != 0;     // next product's barrier
        if (elect_one()) {
          issue_product<OPS, 6, 8>(tmem + 256, tmem, aA + (r & 1) * wobble, aB + (r & 1) * wobble, false);
          umma_commit(&bars->idle);
        }
        __syncwarp();
      }
      if (elect_one()) {
        umma_commit(&bars->done);
        ok = mbar_wait(&bars->done, 0) && ok;
        const long long t1 = clock64();
        if (!ok) atomicCAS(err, 0, 501);
        out[blockIdx.x] = t1 - t0;
        bars->stop = 1;
      }
      __syncwarp();
    } else {
      const long long t0 = clock64();
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        if constexpr (STYLE == 2) {
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->fresh, 1)) != 0;
          tc_fence_after();
        }
        if (elect_one()) {
          if constexpr (OPS >= 5) issue_pair<OPS>(tmem, aA + (r & 1) * wobble, aB + (r & 1) * wobble, r == 0);
          else issue_product<OPS>(tmem + 256, tmem, aA + (r & 1) * wobble, aB + (r & 1) * wobble, r == 0);
          if constexpr (STYLE == 2) umma_commit(&bars->idle);
        }
        __syncwarp();
      }
      if (elect_one()) {
        umma_commit(&bars->done);
        ok = mbar_wait(&bars->done, 0) && ok;
        const long long t1 = clock64();
        if (!ok) atomicCAS(err, 0, 501);
        out[blockIdx.x] = t1 - t0;
        bars->stop = 1;
      }
      __syncwarp();
    }
  } else if (warp >= 2 && DISTURB != 0 && (DISTURB == 3 || warp < 6)) {
    // the disturbing warps: bounded by the issuing warp's stop flag and by a turn count
    const int quarter = warp & 3;
    const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16);
    uint32_t sink = 0;
    for (int turn = 0; turn < (1 << 22) && !bars->stop; ++turn) {
      if constexpr (DISTURB == 3) {
        float x = __uint_as_float(0x3f000000u + (turn & 0xffff) + lane);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float y;
          asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
          x = fmaf(y, 0.25f, -0.125f);
        }
        sink ^= __float_as_uint(x);
      } else if constexpr (DISTURB == 4) {
        if (warp < 6) {
          uint32_t v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = turn + i;
          tmem_st_32x32(taddr, v);
          tmem_st_32x32(taddr + 32, v);
          tmem_st_wait();
        }
      } else if constexpr (DISTURB == 2) {
        uint4* p = reinterpret_cast<uint4*>(sX) + ((turn * 128 + (warp - 2) * 32 + lane) & 2047);
        *p = make_uint4(turn, sink, 0, 0);
      } else {
        uint32_t v[32];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tmem_ld_32x32(taddr + c * 32, v);          // columns 0-127: not the accumulator
          tmem_ld_wait();
          sink ^= v[0] ^ v[31];
        }
      }
    }
    if (sink == 0x12345678u) out[gridDim.x] = sink;  // keeps the loads alive
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int OPS, int STYLE, int DISTURB>
void launch_probe(int rounds, long long* out, int dev, cudaStream_t stream) {
  auto kern = mma_probe_kernel<OPS, STYLE, DISTURB>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  // the second argument is a tile offset the compiler cannot see is zero
  kern<<<ft::gemm::sm_count(dev), kProbeThreads, kSmem, stream>>>(rounds, 0, out, ft::gemm::error_word(dev));
}

}  // namespace

extern "C" {

// out: device buffer of (number of SMs + 1) clock counts, one per CTA.  rounds <= 4096.
int ft_mma_probe(int mode, int rounds, long long* out, cudaStream_t stream) {
  if (mode < 0 || mode > 15 || rounds < 1 || rounds > 4096) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  switch (mode) {
    case 0: launch_probe<0, 0, 0>(rounds, out, dev, stream); break;
    case 1: launch_probe<1, 0, 0>(rounds, out, dev, stream); break;
    case 2: launch_probe<2, 0, 0>(rounds, out, dev, stream); break;
    case 3: launch_probe<3, 0, 0>(rounds, out, dev, stream); break;
    case 4: launch_probe<4, 0, 0>(rounds, out, dev, stream); break;
    case 5: launch_probe<0, 1, 0>(rounds, out, dev, stream); break;
    case 6: launch_probe<0, 2, 0>(rounds, out, dev, stream); break;
    case 7: launch_probe<0, 0, 1>(rounds, out, dev, stream); break;
    case 8: launch_probe<0, 0, 2>(rounds, out, dev, stream); break;
    case 9: launch_probe<3, 0, 1>(rounds, out, dev, stream); break;
    case 10: launch_probe<0, 3, 0>(rounds, out, dev, stream); break;
    case 11: launch_probe<0, 0, 3>(rounds, out, dev, stream); break;
    case 12: launch_probe<3, 0, 3>(rounds, out, dev, stream); break;
    case 13: launch_probe<3, 0, 4>(rounds, out, dev, stream); break;
    case 14: launch_probe<5, 0, 0>(rounds, out, dev, stream); break;
    default: launch_probe<6, 0, 0>(rounds, out, dev, stream); break;
  }
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

}  // extern "C"
