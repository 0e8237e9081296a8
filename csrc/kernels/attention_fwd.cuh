// Causal grouped-query flash attention, forward, on tcgen05 tensor cores.
//
// One CTA per (batch, query head, 128-row query block).  K/V blocks of 128 rows
// stream through a 2-stage TMA ring (128B swizzle, [64-column chunk][row][64]).
//   warp 0    TMA producer (Q once, then K_j / V_j)
//   warp 1    MMA issuer: S_j = Q K_j^T into one of two TMEM buffers (so S_{j+1}
//             is computed while the softmax of block j runs), then
//             O_j = P_j V_j into a third TMEM region
//   warps 2-5 softmax: one thread per query row reads its S row from TMEM,
//             keeps the running max / sum, writes P_j (bf16) into shared memory
//             in the swizzled A-operand layout, then folds O_j into the fp32
//             output row it keeps in registers (O = O * alpha + O_j)
// Outputs: O [B,S,Hq,D] (16-bit) and the per-row log-sum-exp (fp32, natural log
// of sum exp(scale * s)) that the backward pass needs.  All waits are bounded.
#pragma once
#include "common.cuh"
#include "tcgen05.cuh"

namespace ft {
namespace attn {

using namespace ft::sm100;

constexpr int BQ = 128, BKV = 128, KV_STAGES = 2;
constexpr int ATTN_THREADS = 192;

template <int D>
struct FwdSmem {
  static constexpr int TILE = BQ * D * 2;            // bytes of one [128, D] 16-bit tile
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int BYTES = TILE + 2 * KV_STAGES * TILE + P_BYTES + 1024 + 256;
};

struct FwdBars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, o_full;
  uint32_t tmem_base;
  uint32_t abort;
};

struct FwdParams {
  void* o;                 // [B, S, Hq, D] contiguous
  float* lse;              // [B, Hq, S]
  int B, S, Hq, Hkv;
  float scale_log2;        // softmax scale * log2(e)
  float scale_ln;          // softmax scale
  int q_col0, k_col0, v_col0;   // column of head 0 inside the respective tensor map rows
  int* err;
};

// byte offset of 16-byte unit `u` (0..7) of row `r` inside a 128B-swizzled [rows][64] chunk
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t u) {
  return (r >> 3) * 1024 + (r & 7) * 128 + ((u ^ (r & 7)) << 4);
}

template <typename T, int D>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams P) {
  constexpr int TILE = FwdSmem<D>::TILE;
  constexpr int CHUNKS = D / 64;                     // 64-column chunks per tile
  constexpr int CHUNK_BYTES = BQ * 128;              // [128 rows][64 x 2 B]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;
  uint8_t* sV = sK + KV_STAGES * TILE;
  uint8_t* sP = sV + KV_STAGES * TILE;
  FwdBars* bars = reinterpret_cast<FwdBars*>(sP + FwdSmem<D>::P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (P.S + BQ - 1) / BQ;
  // heaviest (last) query blocks first
  const int qb = num_qb - 1 - (int)(blockIdx.x % num_qb);
  const int head = (int)((blockIdx.x / num_qb) % P.Hq);
  const int batch = (int)(blockIdx.x / (num_qb * P.Hq));
  const int kv_head = head / (P.Hq / P.Hkv);
  const int num_kv = qb + 1;                         // causal: blocks 0..qb
  const int q_row0 = batch * P.S + qb * BQ;          // row in the [B*S, width] maps

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&bars->s_full[s], 1); mbar_init(&bars->s_empty[s], 128); }
    mbar_init(&bars->p_full, 128);
    mbar_init(&bars->o_full, 1);
    bars->abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;
  const uint32_t tmem_o = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, TILE);
      for (int c = 0; c < CHUNKS; ++c)
        tma_load_2d(sQ + c * CHUNK_BYTES, &tmap_q, &bars->q_full, P.q_col0 + head * D + c * 64, q_row0);
      for (int j = 0; j < num_kv && !*abort_flag; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int kv_row0 = batch * P.S + j * BKV;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 301); break; }
        mbar_expect_tx(&bars->k_full[s], TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sK + s * TILE + c * CHUNK_BYTES, &tmap_k, &bars->k_full[s],
                      P.k_col0 + kv_head * D + c * 64, kv_row0);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 302); break; }
        mbar_expect_tx(&bars->v_full[s], TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sV + s * TILE + c * CHUNK_BYTES, &tmap_v, &bars->v_full[s],
                      P.v_col0 + kv_head * D + c * 64, kv_row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(AB, 0, 0, BQ, BKV);      // Q, K both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(AB, 0, 1, BQ, D);        // P K-major, V MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        if (!mbar_wait(&bars->k_full[s], (j / KV_STAGES) & 1)) { atomicCAS(P.err, 0, 303); return false; }
        if (!mbar_wait(&bars->s_empty[b], ((j >> 1) & 1) ^ 1)) { atomicCAS(P.err, 0, 304); return false; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tmem + b * BKV, make_smem_desc(q_addr + off, 16, 1024),
                   make_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&bars->k_empty[s]);
        umma_commit(&bars->s_full[b]);
        return true;
      };
      bool ok = mbar_wait(&bars->q_full, 0);
      if (!ok) atomicCAS(P.err, 0, 300);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < num_kv && ok && !*abort_flag; ++j) {
        if (j + 1 < num_kv) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j % KV_STAGES;
        if (!mbar_wait(&bars->v_full[s], (j / KV_STAGES) & 1)) { atomicCAS(P.err, 0, 305); ok = false; break; }
        if (!mbar_wait(&bars->p_full, j & 1)) { atomicCAS(P.err, 0, 306); ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * TILE);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A = P: chunk kk/4, 32 bytes per 16-column step; B = V (MN-major): 16 kv rows = 2048 B
          const uint32_t a_off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tmem_o, make_smem_desc(p_addr + a_off, 16, 1024),
                   make_smem_desc(v_addr + kk * 2048, CHUNK_BYTES, 1024), idesc_o, kk != 0);
        }
        umma_commit(&bars->v_empty[s]);
        umma_commit(&bars->o_full);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ softmax
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;               // row inside the query block
    const int q_pos = qb * BQ + r;                   // position in the sequence
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < num_kv; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&bars->s_full[b], (j >> 1) & 1)) { atomicCAS(P.err, 0, 307); ok = false; break; }
      tc_fence_after();
      // pass 1: row max
      float m_blk = -INFINITY;
      const bool diag = (j == qb);
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_addr + b * BKV + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);
          if (diag && (j * BKV + c * 32 + i) > q_pos) s = -INFINITY;
          m_blk = fmaxf(m_blk, s);
        }
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float alpha = exp2f((m_run - m_new) * P.scale_log2);
      // P of the previous block must have been consumed before it is overwritten
      if (j > 0) {
        if (!mbar_wait(&bars->o_full, (j - 1) & 1)) { atomicCAS(P.err, 0, 308); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] += __uint_as_float(v[i]);
        }
      }
      // pass 2: p = exp2((s - m_new) * scale), row sum, write P
      float l_blk = 0.f;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_addr + b * BKV + c * 32, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);
          if (diag && (j * BKV + c * 32 + i) > q_pos) s = -INFINITY;
          p[i] = exp2f((s - m_new) * P.scale_log2);
          l_blk += p[i];
        }
        uint8_t* chunk = sP + (c / 2) * CHUNK_BYTES;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float t[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) t[i] = p[u * 8 + i];
          *reinterpret_cast<uint4*>(chunk + swz(r, (c % 2) * 4 + u)) = pack8<T>(t);
        }
      }
      // rescale what has been accumulated so far (it was built with the old max)
#pragma unroll
      for (int i = 0; i < D; ++i) o_acc[i] *= alpha;
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      tc_fence_before();
      mbar_arrive(&bars->s_empty[b]);
      fence_proxy_async();
      mbar_arrive(&bars->p_full);
    }
    if (ok) {
      if (!mbar_wait(&bars->o_full, (num_kv - 1) & 1)) { atomicCAS(P.err, 0, 309); ok = false; }
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l_run;
      const bool valid = q_pos < P.S;
      T* orow = reinterpret_cast<T*>(P.o) + ((int64_t)(batch * P.S + q_pos) * P.Hq + head) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = (o_acc[c * 32 + u * 8 + i] + __uint_as_float(v[u * 8 + i])) * inv_l;
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = pack8<T>(t);
          }
        }
      }
      if (valid)
        P.lse[((int64_t)batch * P.Hq + head) * P.S + q_pos] = m_run * P.scale_ln + logf(l_run);
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace attn
}  // namespace ft
