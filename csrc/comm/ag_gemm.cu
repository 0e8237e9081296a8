// Parameter all-gather over NVSwitch peer memory fused with the GEMM that
// consumes the gathered weight, and the stand-alone peer gather the engine uses
// for whole units.
//
// ft_ag_gemm: y[M,N] = x[M,K] * W[N,K]^T where W is a window of a flat, peer-mapped buffer
// that the ranks shard in contiguous pieces (a layer's parameters as the engine keeps them, or
// a matrix row-sharded by itself).  One persistent launch of the CTA-pair tcgen05 pipeline of
// kernels/gemm2_kernel.cuh on every SM, with one more warp per CTA that pulls its share of the
// window's remote chunks into the local buffer with non-multicast bulk copies (peer HBM ->
// shared memory -> local HBM) and publishes one counter per 256-row block.  The output tiles
// are walked from the rows this rank owns outwards, in the order the copies are issued, the
// TMA producers waiting (bounded) for a block's counter before loading it, so the transfer
// overlaps the math tile by tile and the weight crosses NVLink exactly once.
//
// ft_peer_gather / ft_peer_gather_range: the gather alone, for a flat sharded buffer or a byte range of it
// (loads and stores by every thread of one CTA per SM).
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

// The stand-alone gather with plain 16-byte peer loads and local stores issued by every thread
// (four loads in flight per thread), no shared memory: one CTA per SM keeps ~4.8 MB of
// requests in flight, more than the link's bandwidth-delay product, and the CTAs fit beside
// any resident kernel.  It covers a window [w_off_bytes, w_off_bytes + w_bytes) of the flat
// sharded buffer (the whole buffer, or what is left of a unit beside the matrix that the
// all-gather GEMM brings in itself); bytes this rank owns are skipped.  Every rank starts at
// a different place of the window so that the owners' links are loaded evenly.  Start / end
// barriers as in gather_role; CTAs never wait for each other.
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
    const int64_t nvec = G.w_bytes / 16;
    const int64_t chunks = (nvec + LS_THREADS - 1) / LS_THREADS;
    const int64_t rot = ((int64_t)R * chunks) / W;
    const int64_t own_lo = (int64_t)R * G.shard_bytes, own_hi = own_lo + G.shard_bytes;
    for (int64_t c0 = (int64_t)blockIdx.x * LS_UNROLL; c0 < chunks; c0 += (int64_t)gridDim.x * LS_UNROLL) {
      uint4 v[LS_UNROLL];
      int64_t iv[LS_UNROLL];
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u) {
        iv[u] = -1;
        if (c0 + u < chunks) {
          const int64_t i = ((c0 + u + rot) % chunks) * LS_THREADS + threadIdx.x;
          const int64_t flat = G.w_off_bytes + i * 16;
          if (i < nvec && (flat < own_lo || flat >= own_hi)) {
            int p = (int)(flat / G.shard_bytes);
            if (p >= W) p = W - 1;
            iv[u] = i;
            v[u] = __ldcg(reinterpret_cast<const uint4*>(G.w_peer[p]) + i);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u)
        if (iv[u] >= 0) reinterpret_cast<uint4*>(G.w_local)[iv[u]] = v[u];
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

}  // namespace

extern "C" {

void ft_ag_set_spin_budget(long long cycles) { g_spin_budget = cycles; }

// y[M,N] = x[M,K] * W^T with W[N,K] gathered from its owners inside the same launch.
// W is a window of a flat buffer that the ranks shard in contiguous pieces: buf_ptrs[r] is this
// process's mapping of rank r's whole flat buffer, rank r owns its bytes
// [r * shard_bytes, (r+1) * shard_bytes), and W starts w_off_bytes into it (16-bit dtype
// `ab_dtype`, row stride K).  The own part of the window must be in place in buf_ptrs[rank];
// afterwards the whole window is.  A matrix that is row-sharded by itself is the case
// w_off_bytes = 0, shard_bytes = (N / world) * K * 2.
// Requires M > 128 (the CTA-pair pipeline), K % 64 == 0 and shard_bytes, w_off_bytes multiples
// of 8192.  Returns 0, <0 for bad arguments (-7: shape outside the fused kernel, gather and
// multiply separately), >0 for a CUDA error.
int ft_ag_gemm(int world, int rank, const void* const* buf_ptrs, uint32_t* const* flags, uint32_t seq,
               int start_slot, int done_slot, int64_t w_off_bytes, int64_t shard_bytes, const void* x,
               int64_t lda, void* y, int64_t ldc, int c_dtype, int M, int N, int K, int ab_dtype,
               cudaStream_t stream) {
  if (world < 1 || world > peer::kMaxRanks || rank < 0 || rank >= world) return -1;
  if (K % 64 || M <= 0 || N <= 0) return -2;
  if (M <= 128) return -7;
  if (ab_dtype != kBF16 && ab_dtype != kF16) return -3;
  if (c_dtype != ab_dtype && c_dtype != kF32) return -3;
  if (shard_bytes <= 0 || shard_bytes % G2_CHUNK || w_off_bytes < 0 || w_off_bytes % G2_CHUNK) return -2;
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -4;
  const int nt = (N + P_BN - 1) / P_BN;
  if (nt > kReadyWords) return -5;
  const int sms = sm_count(dev);
  GatherArgs G{};
  fill_gather(G, world, rank, buf_ptrs, flags, seq, start_slot, done_slot, 0, dev);
  for (int r = 0; r < world; ++r)
    G.w_peer[r] = reinterpret_cast<const uint8_t*>(buf_ptrs[r]) + w_off_bytes;
  G.w_local = const_cast<uint8_t*>(reinterpret_cast<const uint8_t*>(buf_ptrs[rank]) + w_off_bytes);
  G.shard_bytes = shard_bytes;
  G.block_bytes = (int64_t)P_BN * K * 2;
  G.w_off_bytes = w_off_bytes;
  G.w_bytes = (int64_t)N * K * 2;
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, x, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM, ab_dtype);
  if (rc) return rc;
  rc = make_tmap(&tb, G.w_local, (uint64_t)K, (uint64_t)N, (uint64_t)K, BK, 128, ab_dtype);
  if (rc) return rc;
  cudaMemsetAsync(g_ready[dev], 0, nt * sizeof(uint32_t), stream);
  const int ptiles = ((M + P_BM - 1) / P_BM) * nt;
  const int pgrid = 2 * ptiles < sms ? 2 * ptiles : (sms & ~1);
  G.num_copiers = world > 1 ? pgrid : 0;
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

// Pull the bytes [range_lo, range_hi) of a flat buffer sharded in `shard_bytes` pieces (rank r
// owns bytes [r*shard_bytes, (r+1)*shard_bytes) of every rank's buffer) from their owners into
// the local buffer; what this rank owns is left alone.  All three are multiples of 16.
int ft_peer_gather_range(int world, int rank, const void* const* buf_ptrs, uint32_t* const* flags,
                         uint32_t seq, int start_slot, int done_slot, int64_t shard_bytes, int64_t range_lo,
                         int64_t range_hi, int num_copiers, cudaStream_t stream) {
  if (world < 1 || world > peer::kMaxRanks || rank < 0 || rank >= world) return -1;
  if (shard_bytes % 16 || shard_bytes <= 0 || range_lo % 16 || range_hi % 16) return -2;
  if (range_lo < 0 || range_hi > shard_bytes * world || range_hi < range_lo) return -2;
  if (world == 1) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -4;
  if (num_copiers < 1) num_copiers = 1;
  GatherArgs G{};
  fill_gather(G, world, rank, buf_ptrs, flags, seq, start_slot, done_slot, num_copiers, dev);
  for (int r = 0; r < world; ++r)
    G.w_peer[r] = reinterpret_cast<const uint8_t*>(buf_ptrs[r]) + range_lo;
  G.w_local = const_cast<uint8_t*>(reinterpret_cast<const uint8_t*>(buf_ptrs[rank]) + range_lo);
  G.shard_bytes = shard_bytes;
  G.w_off_bytes = range_lo;
  G.w_bytes = range_hi - range_lo;
  // at least one CTA even for an empty window: the barriers are part of the protocol
  const int64_t chunks = (G.w_bytes / 16 + LS_THREADS - 1) / LS_THREADS;
  int64_t want = (chunks + LS_UNROLL - 1) / LS_UNROLL;
  if (want < 1) want = 1;
  const int grid = (int)(want < (int64_t)num_copiers ? want : num_copiers);
  peer_gather_ldst_kernel<<<grid, LS_THREADS, 0, stream>>>(G, error_word(dev));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// Pull every remote shard of a flat buffer sharded in `shard_bytes` pieces into the local
// buffer.  shard_bytes must be a multiple of 16.
int ft_peer_gather(int world, int rank, const void* const* buf_ptrs, uint32_t* const* flags,
                   uint32_t seq, int start_slot, int done_slot, int64_t shard_bytes, int num_copiers,
                   cudaStream_t stream) {
  return ft_peer_gather_range(world, rank, buf_ptrs, flags, seq, start_slot, done_slot, shard_bytes, 0,
                              shard_bytes * world, num_copiers, stream);
}

}  // extern "C"
