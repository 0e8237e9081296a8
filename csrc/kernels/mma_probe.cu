// Rate of 128-deep tcgen05 products (eight 128xNx16 instructions) for the operand placements the
// attention kernels use, measured in SM clocks by the issuing thread itself.  One CTA per SM
// holds fixed zero-filled tiles in shared memory; one thread issues `rounds` products back to
// back (the tensor pipe's queue holds it back, so the time per round is the pipe's time per
// product) and records clock64() around them.  Used by benchmarks/mma_rate.py to tell what a
// kernel can expect from the tensor pipe before any of its own overheads.
//
//   mode 0  A, B K-major in shared memory, N = 128          (S = Q K^T, dP = dO V^T)
//   mode 1  A, B MN-major in shared memory, N = 128         (dV = P^T dO, dK = dS^T Q)
//   mode 2  A K-major, B MN-major in shared memory, N = 128 (dQ = dS K)
//   mode 3  A in tensor memory, B MN-major, N = 128         (O += P V)
//   mode 4  A, B K-major in shared memory, N = 256
//   mode 5  mode 0 while four warps keep loading 128 columns of tensor memory
//   mode 6  mode 0 while four warps keep storing to shared memory (16 bytes per thread and turn)
//   mode 7  mode 3 while four warps keep loading 128 columns of tensor memory
//   mode 8  mode 0 with the instructions of two independent products interleaved (two accumulators):
//           clocks per PAIR of products
//   mode 9  mode 1 likewise          mode 10  mode 3 likewise
//   mode 11 mode 0 with each instruction's descriptors built from the tile address inside the loop
//           (every other mode adds a constant to a descriptor half prepared before the loop)
//   mode 12 mode 0 with tile addresses that change from round to round (as a kernel's stages do),
//           issued from inside `if (lane == 0)`
//   modes 14-18: mode 12 plus, per product, what a pipelined kernel does around it:
//           14 a tcgen05.commit to a barrier nobody waits on   15 a tcgen05.fence::after_thread_sync
//           16 an mbarrier try_wait that succeeds at once      17 all three
//           18 all three, and the accumulator rotating over four regions of tensor memory
//   mode 19 wait + fence + product + commit, accumulator rotating, written without run-time switches,
//           inside `if (lane == 0)`        mode 20 the same, whole warp with an elected issuer
//   mode 13 the same issued by an elected lane of a warp that runs the loop as a whole, so that the
//           descriptor arithmetic is warp-uniform
#include "common.cuh"
#include "gemm_host.h"
#include "tcgen05.cuh"

namespace {

using namespace ft;
using namespace ft::sm100;

constexpr int kProbeThreads = 192;                   // warp 0 issues, warp 1 owns tensor memory, 2-5 disturb
constexpr int kChunk = 128 * 128;                    // [128 rows][64 columns] of 16-bit values
constexpr int kSmem = 2 * kChunk /* A */ + 4 * kChunk /* B, up to 256 rows */ + 32 * 1024 /* scratch */ + 2048;

struct ProbeBars {
  uint64_t done, idle, fresh;
  uint32_t tmem_base;
  volatile uint32_t stop;
};

__global__ void __launch_bounds__(kProbeThreads, 1)
mma_probe_kernel(int mode, int rounds, int wobble, long long* __restrict__ out, int* __restrict__ err) {
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

  if (warp == 0 && mode == 20) {
    const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
    constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, 128, 128);
    constexpr uint32_t hi = smem_desc_hi(1024);
    const long long t0 = clock64();
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const uint32_t a_lo = smem_desc_lo(aA + (r & 1) * wobble, 16), b_lo = smem_desc_lo(aB + (r & 1) * wobble, 16);
      const uint32_t acc = tmem + (r & 3) * 128;
      ok = mbar_wait(&bars->fresh, 1);               // every lane waits: uniform
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk / 4) * kChunk + (kk % 4) * 32) >> 4;
          umma_f16(acc, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi), idesc, (r | kk) != 0);
        }
        umma_commit(&bars->idle);
      }
      __syncwarp();
    }
    if (elect_one()) {
      umma_commit(&bars->done);
      ok = ok && mbar_wait(&bars->done, 0);
      const long long t1 = clock64();
      if (!ok) atomicCAS(err, 0, 501);
      out[blockIdx.x] = t1 - t0;
      bars->stop = 1;
    }
    __syncwarp();
  } else if (warp == 0 && mode == 19) {
    if (lane == 0) {
      const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
      constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, 128, 128);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const long long t0 = clock64();
      bool ok = true;
      for (int r = 0; r < rounds; ++r) {
        const uint32_t a_lo = smem_desc_lo(aA + (r & 1) * wobble, 16), b_lo = smem_desc_lo(aB + (r & 1) * wobble, 16);
        const uint32_t acc = tmem + (r & 3) * 128;
        if (!mbar_wait(&bars->fresh, 1)) { atomicCAS(err, 0, 502); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk / 4) * kChunk + (kk % 4) * 32) >> 4;
          umma_f16(acc, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi), idesc, (r | kk) != 0);
        }
        umma_commit(&bars->idle);
      }
      umma_commit(&bars->done);
      ok = ok && mbar_wait(&bars->done, 0);
      const long long t1 = clock64();
      if (!ok) atomicCAS(err, 0, 501);
      out[blockIdx.x] = t1 - t0;
      bars->stop = 1;
    }
  } else if (warp == 0 && mode == 13) {
    // the whole warp runs the loop; one elected lane issues
    const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
    constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, 128, 128);
    constexpr uint32_t hi = smem_desc_hi(1024);
    const long long t0 = clock64();
    for (int r = 0; r < rounds; ++r) {
      const uint32_t a_lo = smem_desc_lo(aA + (r & 1) * wobble, 16), b_lo = smem_desc_lo(aB + (r & 1) * wobble, 16);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = ((kk / 4) * kChunk + (kk % 4) * 32) >> 4;
        if (elect_one())
          umma_f16(tmem + 256, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi), idesc, (r | kk) != 0);
        __syncwarp();
      }
    }
    bool ok = true;
    if (elect_one()) {
      umma_commit(&bars->done);
      ok = mbar_wait(&bars->done, 0);
      const long long t1 = clock64();
      if (!ok) atomicCAS(err, 0, 501);
      out[blockIdx.x] = t1 - t0;
      bars->stop = 1;
    }
    __syncwarp();
  } else if (warp == 0) {
    if (lane == 0 && mode >= 12 && mode != 13) {
      const bool with_commit = mode == 14 || mode >= 17, with_fence = mode == 15 || mode >= 17,
                 with_wait = mode == 16 || mode >= 17, rotate = mode == 18;
      const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
      constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, 128, 128);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const long long t0 = clock64();
      for (int r = 0; r < rounds; ++r) {
        const uint32_t a_lo = smem_desc_lo(aA + (r & 1) * wobble, 16), b_lo = smem_desc_lo(aB + (r & 1) * wobble, 16);
        const uint32_t acc = tmem + (rotate ? (r & 3) * 128 : 256);
        if (with_wait && !mbar_wait(&bars->fresh, 1)) break;
        if (with_fence) tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk / 4) * kChunk + (kk % 4) * 32) >> 4;
          umma_f16(acc, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi), idesc, (r | kk) != 0);
        }
        if (with_commit) umma_commit(&bars->idle);
      }
      umma_commit(&bars->done);
      const bool ok = mbar_wait(&bars->done, 0);
      const long long t1 = clock64();
      if (!ok) atomicCAS(err, 0, 501);
      out[blockIdx.x] = t1 - t0;
      bars->stop = 1;
    } else if (lane == 0) {
      const uint32_t aA = smem_u32(sA), aB = smem_u32(sB);
      const bool two = mode >= 8 && mode <= 10;      // two accumulators, instructions alternating
      const bool rebuilt = mode == 11;               // mode 0 with every descriptor built from scratch
      const int base = (mode == 5 || mode == 6 || mode == 8 || mode == 11) ? 0
                       : (mode == 7 || mode == 10) ? 3 : (mode == 9 ? 1 : mode);
      const int n = base == 4 ? 256 : 128;
      const uint32_t idesc = make_idesc_f16(1, base == 1, base == 1 || base == 2 || base == 3, 128, n);
      // descriptors of the eight instructions of a product, low halves; the tiles never move
      uint32_t a_lo[8], b_lo[8];
      const uint32_t hi = smem_desc_hi(1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t k_off = (kk / 4) * kChunk + (kk % 4) * 32;            // K-major, 128 rows
        const uint32_t k_off256 = (kk / 4) * 2 * kChunk + (kk % 4) * 32;     // K-major, 256 rows
        const uint32_t mn_off = kk * 2048;                                    // MN-major
        a_lo[kk] = base == 1 ? smem_desc_lo(aA, kChunk) + (mn_off >> 4) : smem_desc_lo(aA, 16) + (k_off >> 4);
        b_lo[kk] = base == 0 ? smem_desc_lo(aB, 16) + (k_off >> 4)
                   : base == 4 ? smem_desc_lo(aB, 16) + (k_off256 >> 4)
                               : smem_desc_lo(aB, kChunk) + (mn_off >> 4);
      }
      const long long t0 = clock64();
      if (rebuilt) {
        for (int r = 0; r < rounds; ++r) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t k_off = (kk / 4) * kChunk + (kk % 4) * 32;
            umma_f16(tmem + 256, make_smem_desc(aA + k_off, 16, 1024), make_smem_desc(aB + k_off, 16, 1024),
                     idesc, (r | kk) != 0);
          }
        }
      } else if (base == 3) {
        for (int r = 0; r < rounds; ++r) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            umma_f16_ts(tmem + 256, tmem + kk * 8, smem_desc_join(b_lo[kk], hi), idesc, (r | kk) != 0);
            if (two) umma_f16_ts(tmem + 384, tmem + 64 + kk * 8, smem_desc_join(b_lo[kk], hi), idesc, (r | kk) != 0);
          }
        }
      } else {
        for (int r = 0; r < rounds; ++r) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            umma_f16(tmem + 256, smem_desc_join(a_lo[kk], hi), smem_desc_join(b_lo[kk], hi), idesc, (r | kk) != 0);
            if (two) umma_f16(tmem + 384, smem_desc_join(a_lo[kk], hi), smem_desc_join(b_lo[kk], hi), idesc, (r | kk) != 0);
          }
        }
      }
      umma_commit(&bars->done);
      const bool ok = mbar_wait(&bars->done, 0);
      const long long t1 = clock64();
      if (!ok) atomicCAS(err, 0, 501);
      out[blockIdx.x] = t1 - t0;
      bars->stop = 1;
    }
  } else if (warp >= 2 && (mode == 5 || mode == 6 || mode == 7)) {
    // the disturbing warps: bounded by the issuing thread's stop flag and by a turn count
    const int quarter = warp & 3;
    const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16);
    uint32_t sink = 0;
    for (int turn = 0; turn < (1 << 22) && !bars->stop; ++turn) {
      if (mode == 6) {
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

}  // namespace

extern "C" {

// out: device buffer of (number of SMs + 1) clock counts, one per CTA.  rounds <= 4096.
int ft_mma_probe(int mode, int rounds, long long* out, cudaStream_t stream) {
  if (mode < 0 || mode > 20 || rounds < 1 || rounds > 4096) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    configured = true;
  }
  // the third argument is a tile offset the compiler cannot see is zero (modes 12 and 13)
  mma_probe_kernel<<<ft::gemm::sm_count(dev), kProbeThreads, kSmem, stream>>>(mode, rounds, 0, out,
                                                                              ft::gemm::error_word(dev));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

}  // extern "C"
