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

// Arguments of the all-gather role (used only when the kernel is instantiated with
// GATHER = true).  B is row-sharded over `peers.world` ranks: rank r owns rows
// [r * rows_per_rank, (r+1) * rows_per_rank) of every rank's [N, K] buffer.
// CTAs [0, num_copiers) pull the remote shards into the local buffer with bulk
// copies (peer global -> shared -> local global) and count finished chunks per
// 256-row block in `ready`; the TMA producers of the other CTAs wait for a block's
// count before they load it.  Tiles are walked starting with the local shard and
// then in the order the shards arrive.
struct GatherArgs {
  peer::Peers peers;
  uint32_t seq;
  int start_slot, done_slot;
  long long spin_budget;
  const void* w_peer[peer::kMaxRanks];
  void* w_local;
  int64_t row_bytes;       // GEMM use: bytes of one row of B
  int rows_per_rank;       // GEMM use: rows of B owned by each rank
  int64_t shard_bytes;     // bytes each rank owns (multiple of 16)
  int64_t block_bytes;     // bytes covered by one `ready` counter
  int num_copiers;
  uint32_t* ready;
  unsigned int* block_counter;
  int lagged;              // 1: announce a chunk NSTAGE-1 store groups late (keeps the copy stream
                           //    full); 0: wait for each store before the next (the first form)
  // CTA-pair GEMM (gather_role_w): B is a window [w_off_bytes, w_off_bytes + w_bytes) of a flat
  // buffer that is sharded in contiguous pieces of `shard_bytes` (rank r owns flat bytes
  // [r * shard_bytes, (r+1) * shard_bytes)); w_peer / w_local point at the window's first byte.
  // A row-sharded matrix is the case w_off_bytes = 0, shard_bytes = rows_per_rank * row_bytes.
  int64_t w_off_bytes;
  int64_t w_bytes;
  int group_m;             // CTA-pair GEMM, with or without gather: row blocks per group of the tile walk (0: GROUP_M)
};

constexpr int COPY_CHUNK = 32768;

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
                                            int col0, int M, int N) {
  if (row >= M) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
  if constexpr (MODE == kStore32 || MODE == kAcc32) {
    float* p = reinterpret_cast<float*>(C) + (int64_t)row * ldc + col0;
    if (col0 + 32 <= N && (ldc % 4 == 0)) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if constexpr (MODE == kAcc32) {
          float4 old = reinterpret_cast<float4*>(p)[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(p)[q] = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j) p[j] = (MODE == kAcc32 ? p[j] : 0.f) + v[j];
    }
  } else {
    T* p = reinterpret_cast<T*>(C) + (int64_t)row * ldc + col0;
    if (col0 + 32 <= N && (ldc % 8 == 0)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[8 * q + j];
        if constexpr (MODE == kAcc16) {
          float old[8];
          unpack8<T>(reinterpret_cast<uint4*>(p)[q], old);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += old[j];
        }
        reinterpret_cast<uint4*>(p)[q] = pack8<T>(o);
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j)
        p[j] = from_float<T>((MODE == kAcc16 ? to_float(p[j]) : 0.f) + v[j]);
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

// The copier role of one CTA: thread 0 streams this CTA's share of the remote
// chunks through the shared-memory ring, STAGES - 1 loads in flight.
// CHUNK bytes per bulk copy, NSTAGE ring slots of STRIDE bytes, one mbarrier per slot.
template <int CHUNK, int NSTAGE, int STRIDE>
__device__ __forceinline__ void gather_role(const GatherArgs& G, uint8_t* smem, uint64_t* full_bars, int* err) {
  const int W = G.peers.world, R = G.peers.rank;
  if (W <= 1) return;
  uint32_t* mine = G.peers.flags[R];
  if (blockIdx.x == 0) {                      // tell every peer that the local shard is in place
    __threadfence_system();
    for (int p = 0; p < W; ++p)
      if (p != R) peer::st_release_sys(G.peers.flags[p] + G.start_slot * peer::kMaxRanks + R, G.seq);
  }
  bool ok = true;
  for (int p = 0; p < W && ok; ++p)
    if (p != R && !peer::wait_seq(mine + G.start_slot * peer::kMaxRanks + p, G.seq, G.spin_budget)) ok = false;
  if (!ok) {
    atomicCAS(err, 0, 201);
  } else {
    const int64_t shard_bytes = G.shard_bytes;
    const int64_t chunks_per_shard = (shard_bytes + CHUNK - 1) / CHUNK;
    const int64_t total = chunks_per_shard * (W - 1);
    const int64_t block_bytes = G.block_bytes;
    // chunk q of this CTA: global index blockIdx.x + q * num_copiers (the last chunk of a
    // shard may be short)
    auto locate = [&](int64_t q, const uint8_t*& src, uint8_t*& dst, int& nblk, uint32_t& bytes) {
      const int64_t gq = blockIdx.x + q * G.num_copiers;
      const int k = (int)(gq / chunks_per_shard);
      const int p = (R + 1 + k) % W;
      const int64_t in_shard = (gq % chunks_per_shard) * CHUNK;
      const int64_t off = (int64_t)p * shard_bytes + in_shard;
      const int64_t left = shard_bytes - in_shard;
      bytes = (uint32_t)(left < CHUNK ? left : CHUNK);
      src = reinterpret_cast<const uint8_t*>(G.w_peer[p]) + off;
      dst = reinterpret_cast<uint8_t*>(G.w_local) + off;
      nblk = (int)(off / block_bytes);
    };
    const int64_t n = total > blockIdx.x ? (total - blockIdx.x + G.num_copiers - 1) / G.num_copiers : 0;
    uint32_t phase[NSTAGE];
    for (int s = 0; s < NSTAGE; ++s) phase[s] = 0;
    for (int64_t q = 0; q < n && q < NSTAGE - 1; ++q) {
      const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
      locate(q, src, dst, nb, bytes);
      const int s = (int)(q % NSTAGE);
      mbar_expect_tx(&full_bars[s], bytes);
      bulk_load(smem + s * STRIDE, src, bytes, &full_bars[s]);
    }
    if (G.lagged) {
      // Stage reuse only needs the previous store to have *read* shared memory; a chunk is
      // announced once its store group has fully completed, which is checked LAG groups late
      // so that the completion latency never stalls the copy stream.
      constexpr int LAG = NSTAGE - 1;
      int pending[NSTAGE];
      for (int64_t q = 0; q < n; ++q) {
        const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
        locate(q, src, dst, nb, bytes);
        const int s = (int)(q % NSTAGE);
        if (!mbar_wait(&full_bars[s], phase[s])) { atomicCAS(err, 0, 202); break; }
        phase[s] ^= 1;
        bulk_store(dst, smem + s * STRIDE, bytes);
        bulk_commit();
        pending[s] = nb;
        asm volatile("cp.async.bulk.wait_group %0;" ::"n"(LAG) : "memory");
        if (q >= LAG) {                         // chunk q - LAG is in local memory
          fence_proxy_async_all();
          __threadfence();
          red_release_add(G.ready + pending[(int)((q - LAG) % NSTAGE)], 1u);
        }
        const int64_t nq = q + NSTAGE - 1;
        if (nq < n) {
          const uint8_t* src2; uint8_t* dst2; int nb2; uint32_t bytes2;
          locate(nq, src2, dst2, nb2, bytes2);
          const int s2 = (int)(nq % NSTAGE);    // stage of chunk q - 1
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          mbar_expect_tx(&full_bars[s2], bytes2);
          bulk_load(smem + s2 * STRIDE, src2, bytes2, &full_bars[s2]);
        }
      }
      bulk_wait_all();
      fence_proxy_async_all();
      __threadfence();
      for (int64_t q = (n > LAG ? n - LAG : 0); q < n; ++q) {
        const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
        locate(q, src, dst, nb, bytes);
        red_release_add(G.ready + nb, 1u);
      }
    } else {
      int prev_nb = -1;
      for (int64_t q = 0; q < n; ++q) {
        const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
        locate(q, src, dst, nb, bytes);
        const int s = (int)(q % NSTAGE);
        if (!mbar_wait(&full_bars[s], phase[s])) { atomicCAS(err, 0, 202); break; }
        phase[s] ^= 1;
        bulk_store(dst, smem + s * STRIDE, bytes);
        bulk_commit();
        bulk_wait_all_but_1();                  // every chunk before this one is in local memory
        if (q >= 1) {
          fence_proxy_async_all();
          __threadfence();
          red_release_add(G.ready + prev_nb, 1u);
        }
        prev_nb = nb;
        const int64_t nq = q + NSTAGE - 1;
        if (nq < n) {
          const uint8_t* src2; uint8_t* dst2; int nb2; uint32_t bytes2;
          locate(nq, src2, dst2, nb2, bytes2);
          const int s2 = (int)(nq % NSTAGE);    // stage of chunk q - 1, whose store has completed
          mbar_expect_tx(&full_bars[s2], bytes2);
          bulk_load(smem + s2 * STRIDE, src2, bytes2, &full_bars[s2]);
        }
      }
      bulk_wait_all();
      if (prev_nb >= 0) {
        fence_proxy_async_all();
        __threadfence();
        red_release_add(G.ready + prev_nb, 1u);
      }
    }
  }
  // end barrier: the last copier tells the peers that this rank reads their shards no more
  __threadfence_system();
  const unsigned int done = atomicAdd(G.block_counter, 1u);
  if (done == (unsigned int)G.num_copiers - 1) {
    *G.block_counter = 0;
    for (int p = 0; p < W; ++p)
      if (p != R) peer::st_release_sys(G.peers.flags[p] + G.done_slot * peer::kMaxRanks + R, G.seq);
    for (int p = 0; p < W; ++p)
      if (p != R && !peer::wait_seq(mine + G.done_slot * peer::kMaxRanks + p, G.seq, G.spin_budget))
        atomicCAS(err, 0, 203);
  }
}

template <typename T, bool A_MN, bool B_MN, int MODE, bool GATHER = false>
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
  // with GATHER the first CTAs copy and the rest share the tiles among themselves
  const int copiers = GATHER ? gather.num_copiers : 0;
  const int first_tile = (int)blockIdx.x - copiers;
  const int tile_step = (int)gridDim.x - copiers;
  const int nt_local = GATHER ? gather.rows_per_rank / BN : 0;
  const int n_rot = GATHER ? gather.peers.rank * nt_local : 0;

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

  if (GATHER && first_tile < 0) {
    // ------------------------------------------------------- gather role
    if (threadIdx.x == 0) gather_role<COPY_CHUNK, STAGES, STAGE_BYTES>(gather, smem, bars->full, err);
  } else if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step) {
        int mb, nb;
        tile_coords(t, mt, nt, mb, nb);
        if constexpr (GATHER) {
          nb = (nb + n_rot) % nt;
          if (nb < n_rot || nb >= n_rot + nt_local) {      // rows that come from a peer
            const uint32_t need = (uint32_t)(gather.block_bytes / COPY_CHUNK);
            const long long t0 = clock64();
            bool ok = true;
            while (ld_acquire_gpu(gather.ready + nb) < need) {
              if (clock64() - t0 > gather.spin_budget) { ok = false; break; }
              __nanosleep(128);
            }
            if (!ok) { *abort_flag = 1; atomicCAS(err, 0, 204); break; }
            fence_proxy_async_all();
          }
        }
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
    int it = 0;
    for (int t = first_tile; t < num_tiles && !*abort_flag; t += tile_step, ++it) {
      int mb, nb;
      tile_coords(t, mt, nt, mb, nb);
      if constexpr (GATHER) nb = (nb + n_rot) % nt;
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
        store_chunk<T, MODE>(r, C, ldc, row, col0, M, N);
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
