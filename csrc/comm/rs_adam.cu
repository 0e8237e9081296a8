// Gradient reduce-scatter over NVSwitch peer memory fused with loss-scale
// unscale, the non-finite check, the HBM-resident share of the partitioned Adam
// update and the hand-off of the host-resident share.
//
// Every rank exposes its full unit gradient buffer to its peers.  The owner of
// shard r pulls slice r of all `world` buffers with plain peer loads (its own
// slice from local HBM), sums in fp32, multiplies by 1/(world*loss_scale) and,
// per element: [0, og) - applies Adam to the fp32 master / moments kept in HBM
// and writes the device-dtype parameter; [og, S) - writes the reduced gradient
// straight into pinned host memory for the AVX-512 Adam.  Optionally the reduced
// shard is also written back in place (two-phase mode used with dynamic loss
// scaling, where the update must wait for the whole shard's finite flag).
//
// Synchronisation: a start barrier (this rank's gradients are complete when its
// kernel starts; every CTA waits for all peers' start words) and an end barrier
// (the last CTA to finish tells all peers it no longer reads their buffers and
// waits for the same from them, so kernel completion means the local gradient
// buffer may be overwritten).  CTAs never wait for each other, only for other
// GPUs, so no co-residency is assumed.  All spins are bounded; on expiry an
// error word is set, the CTA skips its share of the work and still goes through the
// end barrier (counter and done words), so one late rank costs one wrong step on the
// fused path (the engine then switches to NCCL) instead of desynchronising every
// later call.
//
// Replaces, on the reference's path, the NCCL reduce-scatter of
// flextrain/memory/coordinator/optimizer.py:550-552, the D2H scatter :554-580 and
// (for the HBM share, which the reference cannot have) the CPU Adam.
#include "../kernels/common.cuh"
#include "peer.cuh"

namespace {

using namespace ft;
using namespace ft::peer;

constexpr int kMaxSeg = 8;

struct Segment {
  int64_t lo, hi;                 // shard coordinates, multiples of 8
  float beta2, one_m_beta1, one_m_beta2, eps, step_size, sqrt_bc2, l2_decay, decay_factor;
};

struct RsAdamParams {
  Peers peers;
  const void* grads[kMaxRanks];   // every rank's full gradient buffer
  int grad_dtype;
  int64_t shard;                  // S
  float scale;                    // 1 / (world * loss_scale)
  uint32_t seq;
  int start_slot, done_slot;      // rows of the flag page used by this call site
  unsigned int* block_counter;
  int* err;
  long long spin_budget;
  // outputs
  void* reduced_out;              // own shard slice of the local buffer, or nullptr
  int64_t og;                     // elements [0, og) are updated here
  int do_adam;
  float *master, *m, *v;
  void* param_a; int64_t a_hi;    // device-dtype parameters: [0, a_hi) -> param_a
  void* param_b;                  //                          [a_hi, og) -> param_b (indexed from a_hi)
  int param_dtype;
  void* host_grad;                // [og, S) -> host_grad (indexed from og), or nullptr
  int host_grad_dtype;
  int npush;                      // all-reduce form: updated parameters of [0, og) are also
  void* push[kMaxRanks];          // stored at [rank*S + i] of every rank's full parameter buffer
  int* finite_flag;               // or nullptr
  int* status;                    // or nullptr: receives 101 when this rank gave up at the start barrier
  int nseg;
  Segment seg[kMaxSeg];
};

// Raw 8-element loads of one chunk from every rank's buffer, issued back to back so that all
// `W` peer requests of a thread are in flight together (the reduction is latency-bound on the
// NVLink round trip: with one request per thread in flight a grid of one CTA per SM reaches a
// quarter of the link rate, with eight it saturates the link).
template <typename G>
struct Raw8 {
  uint4 lo;
  uint4 hi;   // second half of an fp32 chunk; unused for 16-bit gradients
};

template <typename G>
__device__ __forceinline__ Raw8<G> load_raw8(const void* base, int64_t idx) {
  Raw8<G> r;
  if constexpr (sizeof(G) == 4) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(base) + idx);
    r.lo = __ldcg(p);
    r.hi = __ldcg(p + 1);
  } else {
    r.lo = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const G*>(base) + idx));
  }
  return r;
}

template <typename G>
__device__ __forceinline__ void add_raw8(const Raw8<G>& r, float (&g)[8]) {
  if constexpr (sizeof(G) == 4) {
    g[0] += __uint_as_float(r.lo.x); g[1] += __uint_as_float(r.lo.y);
    g[2] += __uint_as_float(r.lo.z); g[3] += __uint_as_float(r.lo.w);
    g[4] += __uint_as_float(r.hi.x); g[5] += __uint_as_float(r.hi.y);
    g[6] += __uint_as_float(r.hi.z); g[7] += __uint_as_float(r.hi.w);
  } else {
    float t[8];
    unpack8<G>(r.lo, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] += t[j];
  }
}

__device__ __forceinline__ void store8(void* base, int dtype, int64_t idx, const float (&v)[8]) {
  if (dtype == kF32) {
    float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else if (dtype == kBF16) {
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = pack8<__nv_bfloat16>(v);
  } else {
    *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(base) + idx) = pack8<__half>(v);
  }
}

// Everything that happens to one reduced 8-element chunk: unscale, finite check, the optional
// in-place copy of the reduced gradient, Adam on the HBM share or the hand-off to the host.
__device__ __forceinline__ void finish_chunk(const RsAdamParams& P, int R, int64_t base, int64_t i, float (&g)[8],
                                             bool& bad) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    g[j] *= P.scale;
    bad |= !(fabsf(g[j]) < INFINITY);
  }
  if (P.reduced_out) store8(P.reduced_out, P.grad_dtype, i, g);
  if (i < P.og) {
    if (P.do_adam) {
      int s = 0;
      while (s + 1 < P.nseg && i >= P.seg[s].hi) ++s;
      const Segment& a = P.seg[s];
      float4* pm = reinterpret_cast<float4*>(P.master + i);
      float4* mm = reinterpret_cast<float4*>(P.m + i);
      float4* vm = reinterpret_cast<float4*>(P.v + i);
      float pv[8], mv[8], vv[8];
      *reinterpret_cast<float4*>(pv) = pm[0]; *reinterpret_cast<float4*>(pv + 4) = pm[1];
      *reinterpret_cast<float4*>(mv) = mm[0]; *reinterpret_cast<float4*>(mv + 4) = mm[1];
      *reinterpret_cast<float4*>(vv) = vm[0]; *reinterpret_cast<float4*>(vv + 4) = vm[1];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float gr = g[j] + a.l2_decay * pv[j];
        mv[j] = mv[j] + (gr - mv[j]) * a.one_m_beta1;
        vv[j] = a.beta2 * vv[j] + (a.one_m_beta2 * gr) * gr;
        float denom = sqrtf(vv[j]) / a.sqrt_bc2 + a.eps;
        pv[j] = pv[j] * a.decay_factor - a.step_size * (mv[j] / denom);
      }
      pm[0] = *reinterpret_cast<float4*>(pv); pm[1] = *reinterpret_cast<float4*>(pv + 4);
      mm[0] = *reinterpret_cast<float4*>(mv); mm[1] = *reinterpret_cast<float4*>(mv + 4);
      vm[0] = *reinterpret_cast<float4*>(vv); vm[1] = *reinterpret_cast<float4*>(vv + 4);
      if (i < P.a_hi) {
        if (P.param_a) store8(P.param_a, P.param_dtype, i, pv);
      } else if (P.param_b) {
        store8(P.param_b, P.param_dtype, i - P.a_hi, pv);
      }
      for (int k = 0; k < P.npush; ++k) store8(P.push[(R + k) % P.npush], P.param_dtype, base + i, pv);
    }
  } else if (P.host_grad) {
    store8(P.host_grad, P.host_grad_dtype, i - P.og, g);
  }
}

// CTAs of kThreads threads, at most 80 registers: two of them fit on an SM beside a resident
// GEMM CTA.  A thread works on two chunks at a time and issues the loads of two ranks for both
// before it adds anything, so four requests per thread are in flight whatever the number of
// ranks: ~4.8 MB per GPU at one 512-thread group per SM, above the link's bandwidth-delay
// product (the reduction is bound by the NVLink round trip, not by issue rate).
constexpr int kThreads = 256;

template <typename G>
__global__ void __maxnreg__(80) rs_adam_kernel(const __grid_constant__ RsAdamParams P) {
  __shared__ int s_ok;
  const int W = P.peers.world, R = P.peers.rank;
  uint32_t* mine = P.peers.flags[R];

  // ---- start barrier
  if (blockIdx.x == 0 && threadIdx.x < W && W > 1) {
    __threadfence_system();
    st_release_sys(P.peers.flags[threadIdx.x] + P.start_slot * kMaxRanks + R, P.seq);
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int p = 0; p < W && ok && W > 1; ++p)
      if (p != R && !wait_seq(mine + P.start_slot * kMaxRanks + p, P.seq, P.spin_budget)) ok = 0;
    if (!ok) {
      atomicCAS(P.err, 0, 101);
      // the caller's status word (pinned host or device memory): whoever consumes this call's
      // outputs on the host learns that nothing was written
      if (P.status) { *reinterpret_cast<volatile int*>(P.status) = 101; __threadfence_system(); }
    }
    s_ok = ok;
  }
  __syncthreads();
  // A CTA whose start wait ran out skips the work but still takes part in the end barrier
  // below: leaving here would keep the CTA counter short and the peers without this rank's
  // done word, and every later call on this slot would then wait out its budget as well.
  const bool run = s_ok != 0;

  // ---- reduce + update
  const int64_t base = (int64_t)R * P.shard;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 8;
  bool bad = false;
  for (int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8; run && i0 < P.shard; i0 += 2 * stride) {
    const int64_t i1 = i0 + stride;
    const bool two = i1 < P.shard;
    float g0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float g1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // two ranks per batch: four raw vectors (two chunks x two ranks) are loaded before any is added
    constexpr int PB = 2;
#pragma unroll
    for (int k0 = 0; k0 < kMaxRanks; k0 += PB) {
      Raw8<G> r0[PB], r1[PB];
#pragma unroll
      for (int k = 0; k < PB; ++k) {         // local copy first, peers spread over the links
        if (k0 + k < W) {
          const void* src = P.grads[(R + k0 + k) % W];
          r0[k] = load_raw8<G>(src, base + i0);
          if (two) r1[k] = load_raw8<G>(src, base + i1);
        }
      }
#pragma unroll
      for (int k = 0; k < PB; ++k) {         // fixed summation order: the result does not depend on timing
        if (k0 + k < W) {
          add_raw8<G>(r0[k], g0);
          if (two) add_raw8<G>(r1[k], g1);
        }
      }
    }
    finish_chunk(P, R, base, i0, g0, bad);
    if (two) finish_chunk(P, R, base, i1, g1, bad);
  }
  if (bad && P.finite_flag) atomicOr(P.finite_flag, 1);

  // ---- end barrier (last CTA only)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int done = atomicAdd(P.block_counter, 1u);
    if (done == gridDim.x - 1) {
      __threadfence_system();     // every CTA's peer stores precede the done words below
      *P.block_counter = 0;
      if (W > 1) {
        for (int p = 0; p < W; ++p)
          if (p != R) st_release_sys(P.peers.flags[p] + P.done_slot * kMaxRanks + R, P.seq);
        // a rank that gave up at the start has read nothing: it owes the peers its done word
        // (sent above) but has no reason to wait for theirs
        for (int p = 0; p < W && run; ++p)
          if (p != R && !wait_seq(mine + P.done_slot * kMaxRanks + p, P.seq, P.spin_budget)) atomicCAS(P.err, 0, 102);
      }
    }
  }
}

long long g_spin_budget = 0;   // 0: default
// One "CTAs finished" counter per call site (indexed by the call's start slot): the unit
// reduce-scatter on the optimizer stream and the non-layerwise all-reduce on the compute
// stream can be in flight at the same time and must not count each other's CTAs.
constexpr int kCounters = 64;
unsigned int* g_counter[16] = {nullptr};
int* g_err[16] = {nullptr};

int ensure_state(int dev) {
  if (!g_counter[dev]) {
    if (cudaMalloc(&g_counter[dev], kCounters * sizeof(unsigned int)) != cudaSuccess) return -1;
    cudaMemset(g_counter[dev], 0, kCounters * sizeof(unsigned int));
    if (cudaMalloc(&g_err[dev], sizeof(int)) != cudaSuccess) return -1;
    cudaMemset(g_err[dev], 0, sizeof(int));
  }
  return 0;
}

}  // namespace

extern "C" {

struct FtAdamSegment {
  int64_t lo, hi;
  float lr, beta1, beta2, eps, weight_decay;
  int adamw, bias_correction;
  int64_t step;
};

static int rs_adam_impl(int world, int rank, const void* const* grads, uint32_t* const* flags,
                        int grad_dtype, int64_t shard, float scale, uint32_t seq, int start_slot,
                        int done_slot, void* reduced_out, int64_t og, int do_adam, float* master, float* m,
                        float* v, void* param_a, int64_t a_hi, void* param_b, int param_dtype,
                        void* host_grad, int host_grad_dtype, int* finite_flag, int* status, int nseg,
                        const FtAdamSegment* segs, int max_blocks, void* const* pushes,
                        cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -1;
  if (shard % 8 || og % 8 || a_hi % 8 || nseg > kMaxSeg) return -2;
  if (shard <= 0) return 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -3;
  RsAdamParams P;
  memset(&P, 0, sizeof(P));
  P.peers.world = world;
  P.peers.rank = rank;
  for (int r = 0; r < world; ++r) {
    P.peers.flags[r] = flags ? flags[r] : nullptr;
    P.grads[r] = grads[r];
  }
  P.grad_dtype = grad_dtype;
  P.shard = shard;
  P.scale = scale;
  P.seq = seq;
  P.start_slot = start_slot;
  P.done_slot = done_slot;
  P.block_counter = g_counter[dev] + (start_slot & (kCounters - 1));
  P.err = g_err[dev];
  P.spin_budget = g_spin_budget > 0 ? g_spin_budget : kSpinCycles;
  P.reduced_out = reduced_out;
  P.og = og;
  P.do_adam = do_adam;
  P.master = master; P.m = m; P.v = v;
  P.param_a = param_a; P.a_hi = a_hi; P.param_b = param_b; P.param_dtype = param_dtype;
  P.host_grad = host_grad; P.host_grad_dtype = host_grad_dtype;
  P.finite_flag = finite_flag;
  P.status = status;
  P.npush = pushes ? world : 0;
  for (int r = 0; r < P.npush; ++r) P.push[r] = pushes[r];
  P.nseg = nseg;
  for (int s = 0; s < nseg; ++s) {
    const FtAdamSegment& in = segs[s];
    if (in.lo % 8 || in.hi % 8) return -2;
    Segment& o = P.seg[s];
    o.lo = in.lo; o.hi = in.hi;
    const int64_t step = in.step < 1 ? 1 : in.step;
    double bc1 = 1.0, bc2 = 1.0;
    if (in.bias_correction) {
      bc1 = 1.0 - pow((double)in.beta1, (double)step);
      bc2 = 1.0 - pow((double)in.beta2, (double)step);
    }
    o.beta2 = in.beta2;
    o.one_m_beta1 = 1.0f - in.beta1;
    o.one_m_beta2 = 1.0f - in.beta2;
    o.eps = in.eps;
    o.step_size = (float)((double)in.lr / bc1);
    o.sqrt_bc2 = (float)sqrt(bc2);
    o.l2_decay = in.adamw ? 0.f : in.weight_decay;
    o.decay_factor = in.adamw ? (float)(1.0 - (double)in.lr * (double)in.weight_decay) : 1.f;
  }
  // `max_blocks` counts 512-thread groups (one per SM by default): two CTAs of kThreads each
  const int64_t work = (shard / 8 + 2 * kThreads - 1) / (2 * kThreads);
  const int64_t cap = (int64_t)max_blocks * (512 / kThreads);
  int grid = (int)(work < cap ? work : cap);
  if (grid < 1) grid = 1;
  if (grad_dtype == kF32) rs_adam_kernel<float><<<grid, kThreads, 0, stream>>>(P);
  else if (grad_dtype == kBF16) rs_adam_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(P);
  else rs_adam_kernel<__half><<<grid, kThreads, 0, stream>>>(P);
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// See the file comment.  `grads[r]` / `flags[r]` are this process's mappings of
// rank r's gradient buffer and flag page.  Alignment: shard, og, a_hi and every
// segment bound must be multiples of 8 elements; returns -2 otherwise.
int ft_rs_adam(int world, int rank, const void* const* grads, uint32_t* const* flags, int grad_dtype,
               int64_t shard, float scale, uint32_t seq, int start_slot, int done_slot,
               void* reduced_out, int64_t og, int do_adam, float* master, float* m, float* v,
               void* param_a, int64_t a_hi, void* param_b, int param_dtype, void* host_grad,
               int host_grad_dtype, int* finite_flag, int* status, int nseg, const FtAdamSegment* segs,
               int max_blocks, cudaStream_t stream) {
  return rs_adam_impl(world, rank, grads, flags, grad_dtype, shard, scale, seq, start_slot, done_slot,
                      reduced_out, og, do_adam, master, m, v, param_a, a_hi, param_b, param_dtype,
                      host_grad, host_grad_dtype, finite_flag, status, nseg, segs, max_blocks, nullptr,
                      stream);
}

// All-reduce form for parameters that every rank keeps whole (embedding, final
// norm, head): the same kernel with og = shard, whose owner of slice r reduces
// it, applies Adam to its slice of the fp32 state (which is therefore sharded,
// not replicated) and stores the updated device-dtype parameters into slice r of
// EVERY rank's parameter buffer `params[p]` over NVLink.  When the kernel has
// finished on a rank, all slices of its parameter buffer are up to date (the end
// barrier follows the peers' stores) and its gradient buffer may be zeroed.
// With `do_adam` = 0 only the reduced, unscaled slice is written to
// `reduced_out` (two-phase use under dynamic loss scaling).  Replaces the NCCL
// all-reduce + replicated optimizer step of flextrain/optimizer.py:273-300.
int ft_ar_adam(int world, int rank, const void* const* grads, uint32_t* const* flags, int grad_dtype,
               int64_t shard, float scale, uint32_t seq, int start_slot, int done_slot,
               void* reduced_out, int do_adam, float* master, float* m, float* v, void* const* params,
               int param_dtype, int* finite_flag, int nseg, const FtAdamSegment* segs, int max_blocks,
               cudaStream_t stream) {
  if (do_adam && !params) return -1;
  return rs_adam_impl(world, rank, grads, flags, grad_dtype, shard, scale, seq, start_slot, done_slot,
                      reduced_out, shard, do_adam, master, m, v, nullptr, 0, nullptr, param_dtype,
                      nullptr, -1, finite_flag, nullptr, nseg, segs, max_blocks, do_adam ? params : nullptr,
                      stream);
}

// Clock-cycle budget of every cross-GPU wait (0 restores the default of ~10 s).
// Tests shorten it to make a wait run out on purpose.
void ft_comm_set_spin_budget(long long cycles) { g_spin_budget = cycles; }
long long ft_comm_spin_budget() { return g_spin_budget > 0 ? g_spin_budget : kSpinCycles; }

// Reads and clears the error word of the fused collective kernels (synchronises).
int ft_comm_error() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (ensure_state(dev)) return -1;
  int host = 0;
  if (cudaMemcpy(&host, g_err[dev], sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (host) cudaMemset(g_err[dev], 0, sizeof(int));
  return host;
}

}  // extern "C"
