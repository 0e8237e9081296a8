// Device side of the tcgen05 GEMM: persistent warp-specialised kernel shared by
// the plain GEMM (gemm_tcgen05.cu) and the all-gather-fused GEMM (comm/ag_gemm.cu).
// See gemm_tcgen05.cu for the description of the pipeline.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"
#include "../comm/peer.cuh"

namespace ft {
namespace gemm {

using namespace ft::sm100;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

enum OutMode : int { kStore16 = 0, kStore32 = 1, kAcc16 = 2, kAcc32 = 3 };

// Arguments of the all-gather role of the CTA-pair kernel (gemm2_kernel.cuh, GATHER = true) and
// of the stand-alone gather (comm/ag_gemm.cu).  The gathered bytes are a window
// [w_off_bytes, w_off_bytes + w_bytes) of a flat buffer that the ranks shard in contiguous
// pieces of `shard_bytes` (rank r owns flat bytes [r * shard_bytes, (r+1) * shard_bytes));
// w_peer / w_local point at the window's first byte in every rank's / this rank's buffer.
// A row-sharded matrix is the case w_off_bytes = 0, shard_bytes = rows_per_rank * row_bytes.
// The copy warps count finished chunks per 256-row block in `ready`; the TMA producers wait for
// a block's count before they load it.
struct GatherArgs {
  peer::Peers peers;
  uint32_t seq;
  int start_slot, done_slot;
  long long spin_budget;
  const void* w_peer[peer::kMaxRanks];
  void* w_local;
  int64_t shard_bytes;     // bytes of the flat buffer each rank owns
  int64_t block_bytes;     // bytes covered by one `ready` counter
  int num_copiers;
  uint32_t* ready;
  unsigned int* block_counter;
  int64_t w_off_bytes;
  int64_t w_bytes;
  int group_m;             // CTA-pair GEMM, with or without gather: row blocks per group of the tile walk (0: GROUP_M)
  // accumulating epilogues (kAcc16 / kAcc32), with or without gather: the matrix that is added to
  // the product, of C's type and shape with row stride add_ld; nullptr = C itself (in-place +=)
  const void* add_src;
  int64_t add_ld;
};

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};

// Tile t of the walk: groups of `group_m` row blocks, inside a group column by column, so that
// the tiles in flight at one time share few A and few B blocks (L2 reuse).
__device__ __forceinline__ void tile_coords(int t, int mt, int nt, int& mb, int& nb, int group_m = GROUP_M) {
  const int group_size = group_m * nt;
  const int group = t / group_size;
  const int first_m = group * group_m;
  const int gm = min(mt - first_m, group_m);
  const int in_group = t - group * group_size;
  mb = first_m + in_group % gm;
  nb = in_group / gm;
}

template <typename T, int MODE>
__device__ __forceinline__ void store_chunk(const uint32_t (&acc)[32], void* C, int64_t ldc, int row,
                                            int col0, int M, int N, const void* R = nullptr,
                                            int64_t ldr = 0) {
  if (row >= M) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
  if constexpr (MODE == kStore32 || MODE == kAcc32) {
    float* p = reinterpret_cast<float*>(C) + (int64_t)row * ldc + col0;
    const float* rp = p;                             // what an accumulating mode adds to the product
    if constexpr (MODE == kAcc32) rp = reinterpret_cast<const float*>(R) + (int64_t)row * ldr + col0;
    if (col0 + 32 <= N && (ldc % 4 == 0) && (MODE != kAcc32 || ldr % 4 == 0)) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if constexpr (MODE == kAcc32) {
          float4 old = reinterpret_cast<const float4*>(rp)[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(p)[q] = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j) p[j] = (MODE == kAcc32 ? rp[j] : 0.f) + v[j];
    }
  } else {
    T* p = reinterpret_cast<T*>(C) + (int64_t)row * ldc + col0;
    const T* rp = p;
    if constexpr (MODE == kAcc16) rp = reinterpret_cast<const T*>(R) + (int64_t)row * ldr + col0;
    if (col0 + 32 <= N && (ldc % 8 == 0) && (MODE != kAcc16 || ldr % 8 == 0)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[8 * q + j];
        if constexpr (MODE == kAcc16) {
          float old[8];
          unpack8<T>(reinterpret_cast<const uint4*>(rp)[q], old);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += old[j];
        }
        reinterpret_cast<uint4*>(p)[q] = pack8<T>(o);
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j)
        p[j] = from_float<T>((MODE == kAcc16 ? to_float(rp[j]) : 0.f) + v[j]);
    }
  }
}

// ---- bulk (untiled) async copies, used by the gather role; never multicast
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                   reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all_but_1() {
  asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Of `gather` this kernel uses only the add source of its accumulating epilogue (it shares the
// launch signature of the CTA-pair kernel).
template <typename T, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            void* __restrict__ C, int64_t ldc, int M, int N, int K, int* __restrict__ err,
            const __grid_constant__ GatherArgs gather) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (M + BM - 1) / BM, nt = (N + BN - 1) / BN, kt = (K + BK - 1) / BK;
  const int num_tiles = mt * nt;
  const int first_tile = (int)blockIdx.x;
  const int tile_step = (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step) {
        int mb, nb;
        tile_coords(t, mt, nt, mb, nb);
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 1);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tmap_a, &bars->full[stage], mb * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &bars->full[stage], kb * BK, mb * BM);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tmap_b, &bars->full[stage], nb * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &bars->full[stage], kb * BK, nb * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc =
          make_idesc_f16(sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0, A_MN ? 1 : 0,
                         B_MN ? 1 : 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicCAS(err, 0, 2);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 3);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sa + k * (UK * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sb + k * (UK * 2), 16, 1024);
            umma_f16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);          // frees the stage once the MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&bars->tmem_full[acc]);          // accumulator complete
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue
    const int quarter = warp & 3;                    // TMEM lane quarter this warp may read
    const void* add_src = gather.add_src ? gather.add_src : C;
    const int64_t add_ld = gather.add_src ? gather.add_ld : ldc;
    int it = 0;
    for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step, ++it) {
      int mb, nb;
      tile_coords(t, mt, nt, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase)) {
        *abort_flag = 1;
        atomicCAS(err, 0, 4);
        break;
      }
      tc_fence_after();
      const int row = mb * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = nb * BN + c * 32;
        if (col0 >= N) break;                        // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_chunk<T, MODE>(r, C, ldc, row, col0, M, N, add_src, add_ld);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


}  // namespace gemm
}  // namespace ft
