// tcgen05 GEMM with CTA pairs (cta_group::2): two CTAs of a 2-CTA cluster, on the
// two SMs of a TPC, compute one 256 x 256 output tile.  Each CTA stages its own
// 128 rows of A and one 128-row half of B per k-block (32 KB instead of 48 KB), the
// leader CTA's single MMA thread issues tcgen05.mma.cta_group::2 (M = 256, N = 256,
// K = 16) that reads both CTAs' shared memory, and each CTA's tensor memory
// receives the 128 x 256 accumulator of its own rows.  Compared with the
// single-CTA kernel of gemm_kernel.cuh this cuts shared-memory traffic per FLOP
// (that kernel is bound by it) and deepens the TMA ring to 6 stages.
//
// Barrier protocol per pipeline stage s
//   full[s]   lives in the leader; the leader's producer arms it with the bytes of
//             BOTH CTAs, every TMA load (cta_group::2 form, no multicast) signals the
//             leader's barrier;
//   empty[s]  one per CTA; the leader's tcgen05.commit multicasts its arrival to both;
//   tmem_full[a]   one per CTA, arrival multicast by the leader's commit;
//   tmem_empty[a]  lives in the leader; the epilogue warps of both CTAs arrive on it.
// All waits are bounded; on expiry an error code is recorded and the CTA leaves
// through the common exit (cluster barrier, tensor-memory release).
#pragma once
#include "gemm_kernel.cuh"

namespace ft {
namespace gemm {

constexpr int P_BM = 256, P_BN = 256;               // tile of a CTA pair
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = 128 * BK * 2, P_B_BYTES = 128 * BK * 2, P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;       // clears the CTA-rank bit of a shared::cluster address
// All-gather variant: one more warp per CTA streams remote rows of B through a small
// ring of its own, so every SM keeps computing while the weight arrives.
constexpr int G2_CHUNK = 8192, G2_STAGES = 4;
constexpr int P_SMEM_BYTES_GATHER = P_SMEM_BYTES + G2_STAGES * G2_CHUNK;
constexpr int P_THREADS_GATHER = NUM_THREADS + 32;

struct PairBarriers {
  uint64_t full[P_STAGES];
  uint64_t empty[P_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
  uint64_t gather_full[G2_STAGES];                   // ring of the copy warp (all-gather variant)
};
static_assert(sizeof(PairBarriers) <= 256, "barrier block outgrew its slot");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Warps arrive after divergent role code, so the non-aligned forms are used and every
// warp reconverges first.
__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// TMA tile load of a CTA pair: data lands in this CTA, completion bytes go to the
// barrier at the same offset in the leader CTA.  Not a multicast load.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                                 int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & kPeerBitMask),
      "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrival on the barrier at this offset in both CTAs of the pair once all MMAs issued
// so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

// Arrive on the barrier at this offset in the leader CTA (from either CTA).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerBitMask) : "memory");
}

// Ownership arithmetic of the gathered window (see GatherArgs), in chunks of G2_CHUNK bytes.
// Host code guarantees that shard_bytes and w_off_bytes are multiples of the chunk, so a
// chunk has exactly one owner and this rank's part of the window is one run of whole chunks.
struct WindowOwnership {
  int64_t n_total;         // chunks of the window (the last one may be short)
  int64_t oc_lo, oc_hi;    // this rank's chunks [oc_lo, oc_hi); empty when equal
  int64_t start;           // first remote chunk in copy order: right behind the own run
  __device__ __forceinline__ int64_t n_remote() const { return n_total - (oc_hi - oc_lo); }
};

__device__ __forceinline__ WindowOwnership window_ownership(const GatherArgs& G) {
  WindowOwnership w;
  const int64_t R = G.peers.rank, W = G.peers.world;
  w.n_total = (G.w_bytes + G2_CHUNK - 1) / G2_CHUNK;
  int64_t lo = R * G.shard_bytes - G.w_off_bytes, hi = (R + 1) * G.shard_bytes - G.w_off_bytes;
  lo = lo < 0 ? 0 : (lo > G.w_bytes ? G.w_bytes : lo);
  hi = hi < 0 ? 0 : (hi > G.w_bytes ? G.w_bytes : hi);
  w.oc_lo = lo / G2_CHUNK;
  w.oc_hi = (hi + G2_CHUNK - 1) / G2_CHUNK;
  if (hi <= lo) { w.oc_lo = w.oc_hi = 0; }
  // nothing of the window here: every rank starts at a different place, so that the owners'
  // links are loaded evenly
  w.start = w.oc_hi > w.oc_lo ? w.oc_hi % w.n_total : (R * w.n_total) / W;
  return w;
}

// chunks of 256-row block `nb` that come from a peer
__device__ __forceinline__ uint32_t remote_chunks_in_block(const GatherArgs& G, const WindowOwnership& w,
                                                           int nb) {
  const int64_t per_block = G.block_bytes / G2_CHUNK;
  int64_t c0 = (int64_t)nb * per_block, c1 = c0 + per_block;
  if (c1 > w.n_total) c1 = w.n_total;
  if (c1 <= c0) return 0;
  const int64_t a = c0 > w.oc_lo ? c0 : w.oc_lo, b = c1 < w.oc_hi ? c1 : w.oc_hi;
  return (uint32_t)((c1 - c0) - (b > a ? b - a : 0));
}

// Copy role of the CTA-pair all-gather GEMM: one thread per CTA pulls its share of the
// window's remote chunks (peer HBM -> shared memory -> local HBM, bulk copies, never multicast),
// completion announced per 256-row block NSTAGE-1 store groups late so that the copy stream
// never waits for a store to land.  Start / end barriers as in gather_role.
__device__ __forceinline__ void gather_role_w(const GatherArgs& G, uint8_t* smem, uint64_t* full_bars, int* err) {
  constexpr int NSTAGE = G2_STAGES, CHUNK = G2_CHUNK, LAG = NSTAGE - 1;
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
    const WindowOwnership own = window_ownership(G);
    const int64_t total = own.n_remote();
    auto locate = [&](int64_t q, const uint8_t*& src, uint8_t*& dst, int& nblk, uint32_t& bytes) {
      const int64_t c = (own.start + blockIdx.x + q * G.num_copiers) % own.n_total;
      const int64_t off = c * CHUNK;
      const int64_t left = G.w_bytes - off;
      bytes = (uint32_t)(left < CHUNK ? left : CHUNK);
      const int p = (int)((G.w_off_bytes + off) / G.shard_bytes);
      src = reinterpret_cast<const uint8_t*>(G.w_peer[p]) + off;
      dst = reinterpret_cast<uint8_t*>(G.w_local) + off;
      nblk = (int)(off / G.block_bytes);
    };
    const int64_t n = total > blockIdx.x ? (total - blockIdx.x + G.num_copiers - 1) / G.num_copiers : 0;
    uint32_t phase[NSTAGE];
    for (int s = 0; s < NSTAGE; ++s) phase[s] = 0;
    for (int64_t q = 0; q < n && q < NSTAGE - 1; ++q) {
      const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
      locate(q, src, dst, nb, bytes);
      const int s = (int)(q % NSTAGE);
      mbar_expect_tx(&full_bars[s], bytes);
      bulk_load(smem + s * CHUNK, src, bytes, &full_bars[s]);
    }
    int pending[NSTAGE];
    int64_t q = 0;
    for (; q < n; ++q) {
      const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
      locate(q, src, dst, nb, bytes);
      const int s = (int)(q % NSTAGE);
      if (!mbar_wait(&full_bars[s], phase[s])) { atomicCAS(err, 0, 202); break; }
      phase[s] ^= 1;
      bulk_store(dst, smem + s * CHUNK, bytes);
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
        bulk_load(smem + s2 * CHUNK, src2, bytes2, &full_bars[s2]);
      }
    }
    bulk_wait_all();
    fence_proxy_async_all();
    __threadfence();
    // the chunks stored but not yet announced: the last LAG of those that were stored
    for (int64_t r = (q > LAG ? q - LAG : 0); r < q; ++r) {
      const uint8_t* src; uint8_t* dst; int nb; uint32_t bytes;
      locate(r, src, dst, nb, bytes);
      red_release_add(G.ready + nb, 1u);
    }
  }
  // end barrier: the last copier tells the peers that this rank reads their shards no more
  __threadfence_system();
  const unsigned int done = atomicAdd(G.block_counter, 1u);
  if (done == (unsigned int)G.num_copiers - 1) {
    *G.block_counter = 0;
    for (int p = 0; p < W; ++p)
      if (p != R) peer::st_release_sys(G.peers.flags[p] + G.done_slot * peer::kMaxRanks + R, G.seq);
    for (int p = 0; p < W && ok; ++p)
      if (p != R && !peer::wait_seq(mine + G.done_slot * peer::kMaxRanks + p, G.seq, G.spin_budget))
        atomicCAS(err, 0, 203);
  }
}

// With GATHER, B is a window of a flat buffer sharded over the ranks of `gather.peers` (see GatherArgs): warp 6
// of every CTA copies its share of the remote rows into the local buffer (peer HBM ->
// shared memory -> local HBM, bulk copies without multicast) and counts finished
// chunks per 256-row block; tiles are walked from the local shard outwards and each
// producer waits (bounded) for the block it is about to load.
template <typename T, bool A_MN, bool B_MN, int MODE, bool GATHER = false>
__global__ void __launch_bounds__(GATHER ? P_THREADS_GATHER : NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 void* __restrict__ C, int64_t ldc, int M, int N, int K, int* __restrict__ err,
                 const __grid_constant__ GatherArgs gather) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + P_STAGES * P_STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();            // 0 = leader
  const int pair = (int)(blockIdx.x >> 1), num_pairs = (int)(gridDim.x >> 1);
  const int mt = (M + P_BM - 1) / P_BM, nt = (N + P_BN - 1) / P_BN, kt = (K + BK - 1) / BK;
  const int num_tiles = mt * nt;
  const int group_m = gather.group_m > 0 ? gather.group_m : GROUP_M;
  // with GATHER the columns are walked from this rank's own rows outwards, in copy order
  WindowOwnership own = {};
  int n_rot = 0;
  if constexpr (GATHER) {
    own = window_ownership(gather);
    n_rot = (int)((own.start * G2_CHUNK) / gather.block_bytes) % nt;
    if (own.oc_hi > own.oc_lo) n_rot = (int)((own.oc_lo * G2_CHUNK) / gather.block_bytes);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    if constexpr (GATHER)
      for (int s = 0; s < G2_STAGES; ++s) mbar_init(&bars->gather_full[s], 1);
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
        tile_coords(t, mt, nt, mb, nb, group_m);
        if constexpr (GATHER) {
          nb = (nb + n_rot) % nt;
          const uint32_t need = remote_chunks_in_block(gather, own, nb);
          if (need > 0) {                                  // rows that come from a peer
            const long long t0 = clock64();
            bool ok = true;
            while (ld_acquire_gpu(gather.ready + nb) < need) {
              if (clock64() - t0 > gather.spin_budget) { ok = false; break; }
              __nanosleep(128);
            }
            if (!ok) { *abort_flag = 1; atomicCAS(err, 0, 15); break; }
            fence_proxy_async_all();
          }
        }
        const int m0 = mb * P_BM + (int)cta * 128;   // this CTA's rows of A
        const int n0 = nb * P_BN + (int)cta * 128;   // this CTA's half of B
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 11);
            break;
          }
          uint8_t* sa = smem + stage * P_STAGE_BYTES;
          uint8_t* sb = sa + P_A_BYTES;
          if (cta == 0) mbar_expect_tx(&bars->full[stage], 2 * P_STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sa + j * (64 * BK * 2), &tmap_a, &bars->full[stage], m0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(sa, &tmap_a, &bars->full[stage], kb * BK, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d_pair(sb + j * (64 * BK * 2), &tmap_b, &bars->full[stage], n0 + j * 64, kb * BK);
          } else {
            tma_load_2d_pair(sb, &tmap_b, &bars->full[stage], kb * BK, n0);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc =
          make_idesc_f16(std::is_same<T, __nv_bfloat16>::value ? 1 : 0, A_MN ? 1 : 0, B_MN ? 1 : 0, P_BM, P_BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicCAS(err, 0, 12);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * P_BN;
        bool failed = false;
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 13);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * P_STAGE_BYTES);
          const uint32_t sb = sa + P_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sa + k * (UK * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sb + k * (UK * 2), 16, 1024);
            umma_f16_pair(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&bars->empty[stage]);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit_pair(&bars->tmem_full[acc]);
      }
    }
  } else if (GATHER && warp == 6) {
    // ------------------------------------------------------------ copy warp (both CTAs)
    if (lane == 0) {
      uint8_t* ring = smem + P_STAGES * P_STAGE_BYTES + 256;
      gather_role_w(gather, ring, bars->gather_full, err);
    }
  } else {
    // ---------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const void* add_src = gather.add_src ? gather.add_src : C;
    const int64_t add_ld = gather.add_src ? gather.add_ld : ldc;
    int it = 0;
    for (int t = pair; t < num_tiles && !*abort_flag; t += num_pairs, ++it) {
      int mb, nb;
      tile_coords(t, mt, nt, mb, nb, group_m);
      if constexpr (GATHER) nb = (nb + n_rot) % nt;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase)) {
        *abort_flag = 1;
        atomicCAS(err, 0, 14);
        break;
      }
      tc_fence_after();
      const int row = mb * P_BM + (int)cta * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * P_BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < P_BN / 32; ++c) {
        const int col0 = nb * P_BN + c * 32;
        if (col0 >= N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_chunk<T, MODE>(r, C, ldc, row, col0, M, N, add_src, add_ld);
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
