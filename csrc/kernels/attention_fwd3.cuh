// Causal grouped-query flash attention, forward, third generation.
//
// Same structure as attention_fwd2.cuh (one CTA per pair of 128-row query tiles,
// P and O in tensor memory, lazy rescale, packed fp32 math) with K/V consumed in
// 64-row sub-blocks and TWO score buffers per query tile: the tensor core fills
// buffer (i+1)%2 while the softmax warps work on buffer i%2, so a tile's softmax
// steps run back to back instead of waiting for their own Q K^T each time.
//   tensor memory: tile t scores at t*128 + (i%2)*64, O_t at 256 + t*128
//   shared memory: 2 Q tiles, 4-stage rings of 64-row K and V sub-blocks
//   MMA order:  PV0(i) QK0(i+2) PV1(i) QK1(i+2)
// Measured slower than the second generation (640 vs 930 TFLOP/s at sequence 4096, head
// dim 128): the fixed per-step latencies (barrier hand-offs, tensor-memory load and
// store waits) are paid twice as often and outweigh the better overlap, so it is not
// the default.  All waits are bounded.
#pragma once
#include "attention_fwd2.cuh"

namespace ft {
namespace attn {

constexpr int SUB = 64;            // K/V rows per step
constexpr int F3_STAGES = 4;

template <int D>
struct Fwd3Smem {
  static constexpr int TILE = BQ * D * 2;            // one Q tile
  static constexpr int KV_TILE = SUB * D * 2;        // one K or V sub-block
  static constexpr int BYTES = 2 * TILE + 2 * F3_STAGES * KV_TILE + 1024 + 256;
};

struct Fwd3Bars {
  uint64_t q_full;
  uint64_t k_full[F3_STAGES], k_empty[F3_STAGES];
  uint64_t v_full[F3_STAGES], v_empty[F3_STAGES];
  uint64_t s_full[2][2], p_full[2][2], o_full[2][2]; // [tile][step parity]
  uint32_t tmem_base;
  uint32_t abort;
};

template <typename T, int D>
__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams P) {
  constexpr int TILE = Fwd3Smem<D>::TILE;
  constexpr int KV_TILE = Fwd3Smem<D>::KV_TILE;
  constexpr int CHUNKS = D / 64;
  constexpr int CHUNK_BYTES = BQ * 128;              // one 64-column chunk of a Q tile
  constexpr int KV_CHUNK = SUB * 128;                // one 64-column chunk of a K/V sub-block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                                // two tiles
  uint8_t* sK = sQ + 2 * TILE;
  uint8_t* sV = sK + F3_STAGES * KV_TILE;
  Fwd3Bars* bars = reinterpret_cast<Fwd3Bars*>(sV + F3_STAGES * KV_TILE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (P.S + BQ - 1) / BQ;
  const int num_pairs = (num_qb + 1) / 2;
  const int pi = num_pairs - 1 - (int)(blockIdx.x % num_pairs);      // heaviest pairs first
  const int head = (int)((blockIdx.x / num_pairs) % P.Hq);
  const int batch = (int)(blockIdx.x / (num_pairs * P.Hq));
  const int kv_head = head / (P.Hq / P.Hkv);
  const int qb0 = 2 * pi, qb1 = 2 * pi + 1;
  const int n0 = 2 * (qb0 + 1);                      // 64-row K/V steps tile 0 needs (causal)
  const int n1 = qb1 < num_qb ? 2 * (qb1 + 1) : 0;   // tile 1 may not exist
  const int nmax = n0 > n1 ? n0 : n1;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < F3_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bars->s_full[t][b], 1);
        mbar_init(&bars->p_full[t][b], 128);
        mbar_init(&bars->o_full[t][b], 1);
      }
    }
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

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, (n1 > 0 ? 2 : 1) * TILE);
      for (int t = 0; t < (n1 > 0 ? 2 : 1); ++t)
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sQ + t * TILE + c * CHUNK_BYTES, &tmap_q, &bars->q_full,
                      P.q_col0 + head * D + c * 64, batch * P.S + (qb0 + t) * BQ);
      for (int i = 0; i < nmax && !*abort_flag; ++i) {
        const int s = i % F3_STAGES;
        const uint32_t ph = (i / F3_STAGES) & 1;
        const int kv_row0 = batch * P.S + i * SUB;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 331); break; }
        mbar_expect_tx(&bars->k_full[s], KV_TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sK + s * KV_TILE + c * KV_CHUNK, &tmap_k, &bars->k_full[s],
                      P.k_col0 + kv_head * D + c * 64, kv_row0);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 332); break; }
        mbar_expect_tx(&bars->v_full[s], KV_TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sV + s * KV_TILE + c * KV_CHUNK, &tmap_v, &bars->v_full[s],
                      P.v_col0 + kv_head * D + c * 64, kv_row0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA
    if (lane == 0) {
      constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(AB, 0, 0, BQ, SUB);      // Q, K both K-major
      constexpr uint32_t idesc_o = make_idesc_f16(AB, 0, 1, BQ, D);        // P (tmem) K-major, V MN-major
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = true;
      auto qk = [&](int t, int i) {
        const int s = i % F3_STAGES, b = i & 1;
        if (!mbar_wait(&bars->k_full[s], (i / F3_STAGES) & 1)) { atomicCAS(P.err, 0, 333); ok = false; return; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * KV_TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + t * 128 + b * SUB,
                   make_smem_desc(q_addr + t * TILE + (kk / 4) * CHUNK_BYTES + (kk % 4) * 32, 16, 1024),
                   make_smem_desc(k_addr + (kk / 4) * KV_CHUNK + (kk % 4) * 32, 16, 1024), idesc_s, kk != 0);
        if (t == 1 || i >= n1) umma_commit(&bars->k_empty[s]);       // last reader of K_i
        umma_commit(&bars->s_full[t][b]);
      };
      auto pv = [&](int t, int i) {
        const int s = i % F3_STAGES, b = i & 1;
        if (!mbar_wait(&bars->v_full[s], (i / F3_STAGES) & 1)) { atomicCAS(P.err, 0, 334); ok = false; return; }
        if (!mbar_wait(&bars->p_full[t][b], (i >> 1) & 1)) { atomicCAS(P.err, 0, 335); ok = false; return; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * KV_TILE);
#pragma unroll
        for (int kk = 0; kk < SUB / 16; ++kk)
          umma_f16_ts(tmem + 256 + t * 128, tmem + t * 128 + b * SUB + kk * 8,
                      make_smem_desc(v_addr + kk * 2048, KV_CHUNK, 1024), idesc_o, (i | kk) != 0);
        if (t == 1 || i >= n1) umma_commit(&bars->v_empty[s]);       // last reader of V_i
        // two completion barriers per tile, alternating by step: a softmax warp may be two
        // steps ahead of the P V products, which a single parity bit could not tell apart
        umma_commit(&bars->o_full[t][b]);
      };
      if (!mbar_wait(&bars->q_full, 0)) { atomicCAS(P.err, 0, 330); ok = false; }
      for (int i = 0; i < 2 && ok; ++i) {
        if (i < n0) qk(0, i);
        if (ok && i < n1) qk(1, i);
      }
      for (int i = 0; i < nmax && ok && !*abort_flag; ++i) {
        if (i < n0) pv(0, i);
        if (ok && i + 2 < n0) qk(0, i + 2);
        if (ok && i < n1) pv(1, i);
        if (ok && i + 2 < n1) qk(1, i + 2);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ------------------------------------------------------------ softmax
    const int t = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qb = t ? qb1 : qb0;
    const int n_t = t ? n1 : n0;
    const int q_pos = qb * BQ + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tm_s = tmem + t * 128 + lane_addr;
    const uint32_t tm_o = tmem + 256 + t * 128 + lane_addr;
    const uint64_t scale2 = pm::pack2(P.scale_log2, P.scale_log2);
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int i = 0; i < n_t; ++i) {
      const int b = i & 1;
      if (!mbar_wait(&bars->s_full[t][b], (i >> 1) & 1)) { atomicCAS(P.err, 0, 336); ok = false; break; }
      tc_fence_after();
      const bool diag = (i >= 2 * qb);               // the two sub-blocks of the diagonal block
      const int kv0 = i * SUB;
      const uint32_t tm_sb = tm_s + b * SUB;
      uint32_t v[SUB / 32][32];
#pragma unroll
      for (int c = 0; c < SUB / 32; ++c) tmem_ld_32x32(tm_sb + c * 32, v[c]);
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int c = 0; c < SUB / 32; ++c)
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (kv0 + c * 32 + k > q_pos) v[c][k] = 0xff800000u;     // -inf
      }
      float mx[4];                                   // independent chains
#pragma unroll
      for (int h = 0; h < 4; ++h) mx[h] = -INFINITY;
#pragma unroll
      for (int c = 0; c < SUB / 32; ++c)
#pragma unroll
        for (int k = 0; k < 32; k += 2)
          mx[(c * 2 + (k >> 4)) & 3] = pm::max3(mx[(c * 2 + (k >> 4)) & 3], __uint_as_float(v[c][k]),
                                                __uint_as_float(v[c][k + 1]));
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // rescale O only when some row of the warp outgrew its maximum by more than 2^8
      const bool grow = (m_blk - m_used) * P.scale_log2 > kRescaleLog2;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, m_blk);
        if (i > 0) {
          if (!mbar_wait(&bars->o_full[t][(i - 1) & 1], ((i - 1) >> 1) & 1)) { atomicCAS(P.err, 0, 337); ok = false; break; }
          tc_fence_after();
          const float alpha = pm::ex2((m_used - m_new) * P.scale_log2);
          const uint64_t alpha2 = pm::pack2(alpha, alpha);
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t w[32];
            tmem_ld_32x32(tm_o + c * 32, w);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 32; k += 2) {
              float x, y;
              pm::unpack2(pm::mul2(pm::pack2(__uint_as_float(w[k]), __uint_as_float(w[k + 1])), alpha2), x, y);
              w[k] = __float_as_uint(x);
              w[k + 1] = __float_as_uint(y);
            }
            tmem_st_32x32(tm_o + c * 32, w);
          }
          l_run *= alpha;
        }
        m_used = m_new;
      }
      // p = 2^((s - m) * scale), row sum, P written over the first half of this score buffer
      const float neg_m = -m_used * P.scale_log2;
      const uint64_t neg_m2 = pm::pack2(neg_m, neg_m);
      uint64_t ls[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) ls[h] = pm::pack2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < SUB / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float x, y;
          pm::unpack2(pm::fma2(pm::pack2(__uint_as_float(v[c][2 * k]), __uint_as_float(v[c][2 * k + 1])), scale2,
                               neg_m2), x, y);
          x = pm::ex2(x);
          y = pm::ex2(y);
          ls[k & 3] = pm::add2(ls[k & 3], pm::pack2(x, y));
          pk[k] = pm::cvt2<T>(x, y);
        }
        tmem_st_32x16(tm_sb + c * 16, pk);
      }
      const uint64_t l2 = pm::add2(pm::add2(ls[0], ls[1]), pm::add2(ls[2], ls[3]));
      float la, lb;
      pm::unpack2(l2, la, lb);
      l_run += la + lb;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[t][b]);
    }
    if (ok && n_t > 0) {
      if (!mbar_wait(&bars->o_full[t][(n_t - 1) & 1], ((n_t - 1) >> 1) & 1)) { atomicCAS(P.err, 0, 338); ok = false; }
    }
    if (ok && n_t > 0) {
      tc_fence_after();
      const float inv_l = 1.f / l_run;
      const bool valid = q_pos < P.S;
      T* orow = reinterpret_cast<T*>(P.o) + ((int64_t)(batch * P.S + q_pos) * P.Hq + head) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tm_o + c * 32, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pm::cvt2<T>(__uint_as_float(v[u * 8 + 0]) * inv_l, __uint_as_float(v[u * 8 + 1]) * inv_l);
            w.y = pm::cvt2<T>(__uint_as_float(v[u * 8 + 2]) * inv_l, __uint_as_float(v[u * 8 + 3]) * inv_l);
            w.z = pm::cvt2<T>(__uint_as_float(v[u * 8 + 4]) * inv_l, __uint_as_float(v[u * 8 + 5]) * inv_l);
            w.w = pm::cvt2<T>(__uint_as_float(v[u * 8 + 6]) * inv_l, __uint_as_float(v[u * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + u * 8) = w;
          }
        }
      }
      if (valid)
        P.lse[((int64_t)batch * P.Hq + head) * P.S + q_pos] = m_used * P.scale_ln + logf(l_run);
    } else if (!ok) {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace attn
}  // namespace ft
