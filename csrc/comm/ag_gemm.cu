// Parameter all-gather over NVSwitch peer memory fused with the GEMM that
// consumes the gathered weight, and the stand-alone peer gather the engine uses
// for whole units.
//
// ft_ag_gemm: y[M,N] = x[M,K] * W[N,K]^T where W is row-sharded over `world`
// ranks (rank r owns rows [r*N/world, (r+1)*N/world) of every rank's peer-mapped
// [N,K] buffer).  One persistent launch.  Default form (M > 128): the CTA-pair
// tcgen05 pipeline of kernels/gemm2_kernel.cuh on every SM, with one more warp
// per CTA that pulls its share of the remote shards into the local buffer with
// non-multicast bulk copies (peer HBM -> shared memory -> local HBM) and
// publishes one counter per 256-row block.  Fallback form: the first
// `num_copiers` CTAs only copy and the others run the single-CTA pipeline of
// kernels/gemm_kernel.cuh.  Either way the output tiles are walked from the
// local shard outwards in arrival order, the TMA producers waiting (bounded) for
// a block's counter before loading it, so the transfer overlaps the math tile by
// tile and the weight crosses NVLink exactly once.
//
// ft_peer_gather: the copier role alone, for any flat sharded buffer.
//
// Both replace the NCCL all_gather_into_tensor of
// flextrain/memory/coordinator/parameter.py:516 (and, for ft_ag_gemm, the cuBLAS
// GEMM that follows it).
#include <cstdio>
#include <cstring>

#include "../kernels/gemm_host.h"
#include "../kernels/gemm2_kernel.cuh"
#include "../kernels/gemm_kernel.cuh"

namespace {

using namespace ft;
using namespace ft::gemm;

constexpr int kReadyWords = 8192;
// one "copiers finished" counter per call site (indexed by the start slot), so gathers issued
// from different streams never count each other's CTAs
constexpr int kCounters = 64;

uint32_t* g_ready[16] = {nullptr};
unsigned int* g_counter[16] = {nullptr};
long long g_spin_budget = 0;
int g_gather_lag = 1;   // see ft_gather_set_lag

int ensure_state(int dev) {
  if (!g_ready[dev]) {
    // first half: ft_ag_gemm (reset per call); second half: ft_peer_gather (write-only there)
    if (cudaMalloc(&g_ready[dev], 2 * kReadyWords * sizeof(uint32_t)) != cudaSuccess) return -1;
    cudaMemset(g_ready[dev], 0, 2 * kReadyWords * sizeof(uint32_t));
    if (cudaMalloc(&g_counter[dev], kCounters * sizeof(unsigned int)) != cudaSuccess) return -1;
    cudaMemset(g_counter[dev], 0, kCounters * sizeof(unsigned int));
  }
  return 0;
}

// Small footprint on purpose (3 x 8 KiB of shared memory, one warp): these CTAs
// must fit on an SM beside a resident GEMM CTA, otherwise a gather that runs on
// a side stream would take whole SMs away from the compute stream.
constexpr int PG_CHUNK = 8192, PG_STAGES = 3;

__global__ void __launch_bounds__(32)
peer_gather_kernel(const __grid_constant__ GatherArgs gather, int* __restrict__ err) {
  __shared__ __align__(128) uint8_t ring[PG_STAGES * PG_CHUNK];
  __shared__ uint64_t full_bars[PG_STAGES];
  if (threadIdx.x == 0) {
    for (int s = 0; s < PG_STAGES; ++s) mbar_init(&full_bars[s], 1);
    fence_barrier_init();
    gather_role<PG_CHUNK, PG_STAGES, PG_CHUNK>(gather, ring, full_bars, err);
  }
}

// The same gather with plain 16-byte peer loads and local stores issued by every thread
// (four loads in flight per thread), no shared memory: one CTA per SM keeps ~4.8 MB of
// requests in flight, more than the link's bandwidth-delay product, and the CTAs fit beside
// any resident kernel.  Start / end barriers as in gather_role; CTAs never wait for each other.
constexpr int LS_THREADS = 512;
constexpr int LS_UNROLL = 4;

__global__ void __launch_bounds__(LS_THREADS)
peer_gather_ldst_kernel(const __grid_constant__ GatherArgs G, int* __restrict__ err) {
  __shared__ int s_ok;
  const int W = G.peers.world, R = G.peers.rank;
  uint32_t* mine = G.peers.flags[R];
  if (blockIdx.x == 0 && threadIdx.x < W && (int)threadIdx.x != R) {
    __threadfence_system();
    peer::st_release_sys(G.peers.flags[threadIdx.x] + G.start_slot * peer::kMaxRanks + R, G.seq);
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int p = 0; p < W && ok; ++p)
      if (p != R && !peer::wait_seq(mine + G.start_slot * peer::kMaxRanks + p, G.seq, G.spin_budget)) ok = 0;
    if (!ok) atomicCAS(err, 0, 201);
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    // 16-byte vectors; vector q of the call: peer (R + 1 + q_chunk % (W-1)) so that consecutive
    // chunks of LS_THREADS vectors go to different links
    const int64_t vec_per_shard = G.shard_bytes / 16;
    const int64_t chunks_per_shard = (vec_per_shard + LS_THREADS - 1) / LS_THREADS;
    const int64_t total_chunks = chunks_per_shard * (W - 1);
    for (int64_t c0 = (int64_t)blockIdx.x * LS_UNROLL; c0 < total_chunks; c0 += (int64_t)gridDim.x * LS_UNROLL) {
      uint4 v[LS_UNROLL];
      int64_t off[LS_UNROLL];
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u) {
        const int64_t c = c0 + u;
        off[u] = -1;
        if (c < total_chunks) {
          const int p = (R + 1 + (int)(c % (W - 1))) % W;
          const int64_t iv = (c / (W - 1)) * LS_THREADS + threadIdx.x;
          if (iv < vec_per_shard) {
            off[u] = (int64_t)p * vec_per_shard + iv;
            v[u] = __ldcg(reinterpret_cast<const uint4*>(G.w_peer[p]) + off[u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u)
        if (off[u] >= 0) reinterpret_cast<uint4*>(G.w_local)[off[u]] = v[u];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int done = atomicAdd(G.block_counter, 1u);
    if (done == gridDim.x - 1) {
      *G.block_counter = 0;
      for (int p = 0; p < W; ++p)
        if (p != R) peer::st_release_sys(G.peers.flags[p] + G.done_slot * peer::kMaxRanks + R, G.seq);
      for (int p = 0; p < W && s_ok; ++p)
        if (p != R && !peer::wait_seq(mine + G.done_slot * peer::kMaxRanks + p, G.seq, G.spin_budget))
          atomicCAS(err, 0, 203);
    }
  }
}

int g_gather_mode = -1;   // -1: read FLEXTRAIN_PEER_GATHER on first use; 0 bulk copies, 1 loads / stores

int fill_gather(GatherArgs& G, int world, int rank, const void* const* w_ptrs, uint32_t* const* flags,
                uint32_t seq, int start_slot, int done_slot, int num_copiers, int dev) {
  memset(&G, 0, sizeof(G));
  G.peers.world = world;
  G.peers.rank = rank;
  for (int r = 0; r < world; ++r) {
    G.peers.flags[r] = flags ? flags[r] : nullptr;
    G.w_peer[r] = w_ptrs[r];
  }
  G.w_local = const_cast<void*>(w_ptrs[rank]);
  G.seq = seq;
  G.start_slot = start_slot;
  G.done_slot = done_slot;
  G.spin_budget = g_spin_budget > 0 ? g_spin_budget : peer::kSpinCycles;
  G.num_copiers = num_copiers;
  G.ready = g_ready[dev];
  G.lagged = g_gather_lag;
  G.block_counter = g_counter[dev] + (start_slot & (kCounters - 1));
  return 0;
}

// CTA-pair form (kernels/gemm2_kernel.cuh with GATHER): every CTA computes and its
// seventh warp copies, so no SM is given up to the transfer.
template <typename T, int MODE>
int launch_pair_gather(const CUtensorMap& ta, const CUtensorMap& tb, void* y, int64_t ldc, int M, int N,
                       int K, int* err, int grid, const GatherArgs& G, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<T, false, false, MODE, true>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES_GATHER);
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(P_THREADS_GATHER, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_BYTES_GATHER;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, y, ldc, M, N, K, err, G);
  return e == cudaSuccess ? 0 : (int)e;
}

int g_ag_pair = -1;   // -1: read FLEXTRAIN_AG_GEMM_PAIR on first use (default on)

}  // namespace

extern "C" {

// Selects the CTA-pair form (1, default) or the single-CTA form with dedicated copy
// CTAs (0) for later ft_ag_gemm calls.
void ft_ag_gemm_set_pair(int on) { g_ag_pair = on ? 1 : 0; }

void ft_ag_set_spin_budget(long long cycles) { g_spin_budget = cycles; }

// Form of ft_peer_gather: 1 = loads / stores by every thread (default), 0 = bulk copies through
// shared memory by one thread per CTA.
void ft_gather_set_mode(int mode) { g_gather_mode = mode ? 1 : 0; }

// Completion signalling of the copy role for later ft_ag_gemm / ft_peer_gather calls:
// 1 = lagged by NSTAGE-1 store groups (default), 0 = one store at a time.
void ft_gather_set_lag(int on) { g_gather_lag = on ? 1 : 0; }

// y[M,N] = x[M,K] * W^T with W gathered from its row shards inside the same launch.
// w_ptrs[r]: this process's mapping of rank r's [N,K] buffer (16-bit dtype `ab_dtype`).
// Requires N % (world * 256) == 0 and K % 64 == 0.  Returns 0, <0 for bad arguments,
// >0 for a CUDA error.
int ft_ag_gemm(int world, int rank, const void* const* w_ptrs, uint32_t* const* flags, uint32_t seq,
               int start_slot, int done_slot, const void* x, int64_t lda, void* y, int64_t ldc,
               int c_dtype, int M, int N, int K, int ab_dtype, int num_copiers, cudaStream_t stream) {
  if (world < 1 || world > peer::kMaxRanks || rank < 0 || rank >= world) return -1;
  if (N % (world * BN) || K % 64 || M <= 0) return -2;
  if (ab_dtype != kBF16 && ab_dtype != kF16) return -3;
  if (c_dtype != ab_dtype && c_dtype != kF32) return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -4;
  const int nt = N / BN;
  if (nt > kReadyWords) return -5;
  const int sms = sm_count(dev);
  if (world == 1) num_copiers = 0;
  if (num_copiers < 0 || num_copiers >= sms) return -6;
  if (world > 1 && num_copiers == 0) return -6;
  GatherArgs G;
  fill_gather(G, world, rank, w_ptrs, flags, seq, start_slot, done_slot, num_copiers, dev);
  G.row_bytes = (int64_t)K * 2;
  G.rows_per_rank = N / world;
  G.shard_bytes = (int64_t)G.rows_per_rank * G.row_bytes;
  G.block_bytes = (int64_t)BN * G.row_bytes;
  if (g_ag_pair < 0) {
    const char* e = getenv("FLEXTRAIN_AG_GEMM_PAIR");
    g_ag_pair = e ? atoi(e) : 1;
  }
  const bool pair = g_ag_pair != 0 && M > 128;
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, x, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM, ab_dtype);
  if (rc) return rc;
  rc = make_tmap(&tb, w_ptrs[rank], (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, pair ? 128 : BN, ab_dtype);
  if (rc) return rc;
  cudaMemsetAsync(g_ready[dev], 0, nt * sizeof(uint32_t), stream);
  if (pair) {
    const int ptiles = ((M + P_BM - 1) / P_BM) * (N / P_BN);
    int pgrid = 2 * ptiles < sms ? 2 * ptiles : (sms & ~1);
    G.num_copiers = pgrid;
    int* perr = error_word(dev);
    if (ab_dtype == kBF16)
      rc = c_dtype == kF32
               ? launch_pair_gather<__nv_bfloat16, kStore32>(ta, tb, y, ldc, M, N, K, perr, pgrid, G, stream)
               : launch_pair_gather<__nv_bfloat16, kStore16>(ta, tb, y, ldc, M, N, K, perr, pgrid, G, stream);
    else
      rc = c_dtype == kF32
               ? launch_pair_gather<__half, kStore32>(ta, tb, y, ldc, M, N, K, perr, pgrid, G, stream)
               : launch_pair_gather<__half, kStore16>(ta, tb, y, ldc, M, N, K, perr, pgrid, G, stream);
    if (rc) return rc;
    FT_LAUNCHED(1);
    FT_CUDA_RETURN_IF_ERROR();
    return 0;
  }
  const int tiles = ((M + BM - 1) / BM) * nt;
  int grid = tiles + num_copiers < sms ? tiles + num_copiers : sms;
  int* err = error_word(dev);
#define FT_AG_LAUNCH(T, MODE)                                                                   \
  {                                                                                             \
    auto kern = gemm_kernel<T, false, false, MODE, true>;                                       \
    static bool configured = false;                                                             \
    if (!configured) {                                                                          \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);      \
      configured = true;                                                                        \
    }                                                                                           \
    kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, y, ldc, M, N, K, err, G);           \
  }
  if (ab_dtype == kBF16) {
    if (c_dtype == kF32) FT_AG_LAUNCH(__nv_bfloat16, kStore32) else FT_AG_LAUNCH(__nv_bfloat16, kStore16)
  } else {
    if (c_dtype == kF32) FT_AG_LAUNCH(__half, kStore32) else FT_AG_LAUNCH(__half, kStore16)
  }
#undef FT_AG_LAUNCH
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// Pull every remote shard of a flat buffer sharded in `shard_bytes` pieces
// (rank r owns bytes [r*shard_bytes, (r+1)*shard_bytes) of every rank's buffer)
// into the local buffer.  shard_bytes must be a multiple of 16.
int ft_peer_gather(int world, int rank, const void* const* buf_ptrs, uint32_t* const* flags,
                   uint32_t seq, int start_slot, int done_slot, int64_t shard_bytes, int num_copiers,
                   cudaStream_t stream) {
  if (world < 1 || world > peer::kMaxRanks || rank < 0 || rank >= world) return -1;
  if (shard_bytes % 16 || shard_bytes <= 0) return -2;
  if (world == 1) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -4;
  if (num_copiers < 1) num_copiers = 1;
  GatherArgs G;
  fill_gather(G, world, rank, buf_ptrs, flags, seq, start_slot, done_slot, num_copiers, dev);
  G.ready = g_ready[dev] + kReadyWords;
  G.shard_bytes = shard_bytes;
  G.block_bytes = (shard_bytes * world + kReadyWords - 1) / kReadyWords;
  if (G.block_bytes < PG_CHUNK) G.block_bytes = PG_CHUNK;
  if (g_gather_mode < 0) {
    const char* e = getenv("FLEXTRAIN_PEER_GATHER");
    g_gather_mode = (e && !strcmp(e, "bulk")) ? 0 : 1;
  }
  if (g_gather_mode == 1) {
    const int64_t chunks = ((shard_bytes / 16 + LS_THREADS - 1) / LS_THREADS) * (world - 1);
    const int64_t want = (chunks + LS_UNROLL - 1) / LS_UNROLL;
    const int grid = (int)(want < (int64_t)num_copiers ? want : num_copiers);
    peer_gather_ldst_kernel<<<grid, LS_THREADS, 0, stream>>>(G, error_word(dev));
  } else {
    peer_gather_kernel<<<num_copiers, 32, 0, stream>>>(G, error_word(dev));
  }
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

}  // extern "C"
