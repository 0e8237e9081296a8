// CTA-pair tcgen05 GEMM with the SwiGLU activation in its epilogue:
//
//     act[M, F] = silu(X W_gate^T) * (X W_up^T),      W = [W_gate ; W_up] stored [2F, K]
//
// Same pipeline and barrier protocol as gemm_pair_kernel (gemm2_kernel.cuh); the
// difference is which rows of W a pair stages and what the epilogue does.  For the
// output columns [128 nb, 128 nb + 128) the leader CTA stages the gate rows
// [128 nb, +128) and its partner the up rows [F + 128 nb, +128), so the 256-column
// accumulator of every CTA holds gate in columns 0..127 and up in columns 128..255 of
// the SAME output columns: the epilogue thread that owns a row reads both, applies the
// activation on the fp32 accumulators and stores one 16-bit value.  The [M, 2F]
// intermediate is neither written nor read again (two passes over it, 4 x the size of
// the output, disappear); when the backward pass needs it (`gu` not null) it is stored
// from the same registers.  F must be a multiple of 128.  X and W are K-major.
#pragma once
#include "gemm2_kernel.cuh"

namespace ft {
namespace gemm {

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_pair_swiglu_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        void* __restrict__ act, int64_t ld_act, void* __restrict__ gu, int64_t ld_gu, int M,
                        int F, int K, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + P_STAGES * P_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();            // 0 = leader
  const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
  const int mt = (M + P_BM - 1) / P_BM, nt = F / 128, kt = (K + BK - 1) / BK;
  const int num_tiles = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);            // 4 epilogue warps in each of the two CTAs
    }
    bars->abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs) {
        int mb, nb;
        tile_coords(t, mt, nt, mb, nb);
        const int m0 = mb * P_BM + (int)cta * 128;   // this CTA's rows of X
        const int n0 = nb * 128 + (int)cta * F;      // gate rows (leader) or up rows (partner) of W
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 21);
            break;
          }
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          if (cta == 0) mbar_expect_tx(&bars->full[stage], 2 * P_STAGE_BYTES);
          tma_load_2d_pair(sa, &tmap_a, &bars->full[stage], kb * BK, m0);
          tma_load_2d_pair(sb, &tmap_b, &bars->full[stage], kb * BK, n0);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, 0, 0, P_BM, P_BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicCAS(err, 0, 22);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * P_BN;
        bool failed = false;
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 23);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * P_STAGE_BYTES);
          const uint32_t sb = sa + P_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k)
            umma_f16_pair(tmem_d, make_smem_desc(sa + k * (UK * 2), 16, 1024),
                          make_smem_desc(sb + k * (UK * 2), 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&bars->empty[stage]);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit_pair(&bars->tmem_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    int it = 0;
    for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++it) {
      int mb, nb;
      tile_coords(t, mt, nt, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase)) {
        *abort_flag = 1;
        atomicCAS(err, 0, 24);
        break;
      }
      tc_fence_after();
      const int row = mb * P_BM + (int)cta * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * P_BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        const int col0 = nb * 128 + c * 32;          // output column (and gate column of gu)
        uint32_t g[32], u[32];
        tmem_ld_32x32(taddr + c * 32, g);
        tmem_ld_32x32(taddr + 128 + c * 32, u);
        tmem_ld_wait();
        if (gu != nullptr) {
          store_chunk<T, kStore16>(g, gu, ld_gu, row, col0, M, 2 * F);
          store_chunk<T, kStore16>(u, gu, ld_gu, row, F + col0, M, 2 * F);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float gv = __uint_as_float(g[j]);
          g[j] = __float_as_uint(__fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[j]));
        }
        store_chunk<T, kStore16>(g, act, ld_act, row, col0, M, F);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  cluster_sync_all();                                // the peer may still read this CTA's shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace gemm
}  // namespace ft
