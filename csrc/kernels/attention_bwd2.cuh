// Causal grouped-query flash attention, backward, second generation.
//
// Same decomposition and math as attention_bwd.cuh (one CTA per (batch, kv head,
// kv block); K_n, V_n resident; walk over the query heads of the group and the query
// blocks m >= n; dK / dV accumulated in tensor memory, dQ reduce-added into an fp32
// buffer by TMA).  What changes is the dependency chain between consecutive query
// blocks, which in the first generation left the tensor pipe idle for most of a block:
//
//   * Q is double-buffered and dO is given back right after the dV product, so the
//     loads of block i+1 are issued one block (Q) or half a block (dO) ahead instead of
//     after the last product of block i;
//   * dQ is accumulated on the dP columns of tensor memory (free once dS sits in
//     registers) instead of the S columns, and the S columns are released as soon as the
//     softmax warps have loaded them, so S of block i+1 is issued directly behind dQ of
//     block i and is ready when the softmax warps come back from draining dQ.
//
// Issue order on the tensor pipe per block i: dP_i, dV_i, dK_i, dQ_i, S_{i+1}.
// Shared memory at D = 128: K, V, Q x2, dO, P, dS tiles of 32 KB = 224 KB.
// All waits are bounded and report through the error word (codes 42x).
#pragma once
#include "attention_bwd.cuh"

namespace ft {
namespace attn {

template <int D>
struct Bwd2Smem {
  static constexpr int TILE = BQ * D * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int BYTES = 5 * TILE + 2 * P_BYTES + 1024 + 256;
};

struct Bwd2Bars {
  uint64_t kv_full, q_full[2], q_empty[2], do_full, do_empty;
  uint64_t s_full, s_free, dp_full, dp_free, p_full, ds_full, dq_full, dqs_full, stage_free, acc_full;
  uint32_t tmem_base;
  uint32_t abort;
};

template <typename T, int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                 const __grid_constant__ CUtensorMap tmap_dq, const __grid_constant__ BwdParams P) {
  constexpr int TILE = Bwd2Smem<D>::TILE;
  constexpr int CHUNKS = D / 64;
  constexpr int CHUNK_BYTES = BQ * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;                 // two stages of TILE bytes
  uint8_t* sdO = sQ + 2 * TILE;
  uint8_t* sP = sdO + TILE;
  uint8_t* sdS = sP + Bwd2Smem<D>::P_BYTES;
  Bwd2Bars* bars = reinterpret_cast<Bwd2Bars*>(sdS + Bwd2Smem<D>::P_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_blk = (P.S + BQ - 1) / BQ;
  const int nb = (int)(blockIdx.x % num_blk);        // kv block; low blocks (most work) first
  const int kv_head = (int)((blockIdx.x / num_blk) % P.Hkv);
  const int batch = (int)(blockIdx.x / (num_blk * P.Hkv));
  const int group = P.Hq / P.Hkv;
  const int q_blocks = num_blk - nb;                 // m = nb .. num_blk-1
  const int iters = group * q_blocks;
  const int kv_row0 = batch * P.S + nb * BKV;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&bars->q_full[s], 1); mbar_init(&bars->q_empty[s], 1); }
    mbar_init(&bars->do_full, 1);
    mbar_init(&bars->do_empty, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_free, 256);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->dp_free, 256);
    mbar_init(&bars->p_full, 256);
    mbar_init(&bars->ds_full, 256);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dqs_full, 256);
    mbar_init(&bars->stage_free, 1);
    mbar_init(&bars->acc_full, 1);
    bars->abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
    prefetch_tmap(&tmap_dq);
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;
  const uint32_t tm_s = tmem, tm_dp = tmem + 128, tm_dv = tmem + 256, tm_dk = tmem + 384;
  const uint32_t tm_dq = tm_dp;                      // dP is in registers by the time dQ is issued

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&bars->kv_full, 2 * TILE);
      for (int c = 0; c < CHUNKS; ++c) {
        tma_load_2d(sK + c * CHUNK_BYTES, &tmap_k, &bars->kv_full, kv_head * D + c * 64, kv_row0);
        tma_load_2d(sV + c * CHUNK_BYTES, &tmap_v, &bars->kv_full, kv_head * D + c * 64, kv_row0);
      }
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int head = kv_head * group + it / q_blocks;
        const int m = nb + it % q_blocks;
        const int q_row0 = batch * P.S + m * BQ;
        const int st = it & 1;
        // Q_it goes into the stage that dK of block it-2 has finished reading
        if (!mbar_wait(&bars->q_empty[st], ((it >> 1) & 1) ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 421); break; }
        mbar_expect_tx(&bars->q_full[st], TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sQ + st * TILE + c * CHUNK_BYTES, &tmap_q, &bars->q_full[st], head * D + c * 64, q_row0);
        // dO_it once dV of block it-1 has finished reading the buffer
        if (!mbar_wait(&bars->do_empty, (it & 1) ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 422); break; }
        mbar_expect_tx(&bars->do_full, TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sdO + c * CHUNK_BYTES, &tmap_do, &bars->do_full, head * D + c * 64, q_row0);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t id_s = make_idesc_f16(AB, 0, 0, BQ, BKV);     // K-major x K-major
      constexpr uint32_t id_t = make_idesc_f16(AB, 1, 1, BKV, D);      // MN-major x MN-major
      constexpr uint32_t id_q = make_idesc_f16(AB, 0, 1, BQ, D);       // K-major x MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ0 = smem_u32(sQ), aDO = smem_u32(sdO),
                     aP = smem_u32(sP), aDS = smem_u32(sdS);
      auto issue_s = [&](uint32_t aQ) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_s, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), id_s, kk != 0);
        }
        umma_commit(&bars->s_full);
      };
      bool ok = mbar_wait(&bars->kv_full, 0);
      if (!ok) atomicCAS(P.err, 0, 423);
      if (ok && iters > 0) {
        if (!mbar_wait(&bars->q_full[0], 0)) { atomicCAS(P.err, 0, 424); ok = false; }
        else { tc_fence_after(); issue_s(aQ0); }
      }
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        const uint32_t ph = it & 1;
        const int st = it & 1;
        const uint32_t aQ = aQ0 + st * TILE;
        // dP_it: dO_it loaded, dP columns drained of dQ_{it-1}
        if (!mbar_wait(&bars->do_full, ph)) { atomicCAS(P.err, 0, 425); ok = false; break; }
        if (it > 0 && !mbar_wait(&bars->dp_free, ph ^ 1)) { atomicCAS(P.err, 0, 426); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_dp, make_smem_desc(aDO + off, 16, 1024), make_smem_desc(aV + off, 16, 1024), id_s,
                   kk != 0);
        }
        umma_commit(&bars->dp_full);
        // dV += P^T dO
        if (!mbar_wait(&bars->p_full, ph)) { atomicCAS(P.err, 0, 427); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {       // reduction over the 128 query rows
          const uint32_t row_off = kk * 2048;
          umma_f16(tm_dv, make_smem_desc(aP + row_off, CHUNK_BYTES, 1024),
                   make_smem_desc(aDO + row_off, CHUNK_BYTES, 1024), id_t, (it | kk) != 0);
        }
        umma_commit(&bars->do_empty);                // dO_it has no reader left
        // dK += dS^T Q, dQ = dS K
        if (!mbar_wait(&bars->ds_full, ph)) { atomicCAS(P.err, 0, 428); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint32_t row_off = kk * 2048;
          umma_f16(tm_dk, make_smem_desc(aDS + row_off, CHUNK_BYTES, 1024),
                   make_smem_desc(aQ + row_off, CHUNK_BYTES, 1024), id_t, (it | kk) != 0);
        }
        umma_commit(&bars->q_empty[st]);             // Q_it has no reader left
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {      // reduction over the 128 kv rows
          const uint32_t a_off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_dq, make_smem_desc(aDS + a_off, 16, 1024),
                   make_smem_desc(aK + kk * 2048, CHUNK_BYTES, 1024), id_q, kk != 0);
        }
        umma_commit(&bars->dq_full);
        // S_{it+1} directly behind: its columns were released when P_it was extracted
        if (it + 1 < iters) {
          const int nst = (it + 1) & 1;
          if (!mbar_wait(&bars->q_full[nst], ((it + 1) >> 1) & 1)) { atomicCAS(P.err, 0, 429); ok = false; break; }
          if (!mbar_wait(&bars->s_free, ph)) { atomicCAS(P.err, 0, 430); ok = false; break; }
          tc_fence_after();
          issue_s(aQ0 + nst * TILE);
        }
      }
      if (ok) umma_commit(&bars->acc_full);
      else *abort_flag = 1;
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ dQ store warp
    if (lane == 0) {
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int head = kv_head * group + it / q_blocks;
        const int m = nb + it % q_blocks;
        if (!mbar_wait(&bars->dqs_full, it & 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 431); break; }
#pragma unroll
        for (int c = 0; c < D / 32; ++c)
          tma_reduce_add_2d(&tmap_dq, sP + c * (BQ * 128), head * D + c * 32, batch * P.S + m * BQ);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(&bars->stage_free);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    // --------------------------------------------------------- softmax warps
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;                // which half of the columns this warp owns
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float log2e = 1.4426950408889634f;
    const uint64_t scale2 = pm::pack2(P.scale_log2, P.scale_log2);
    constexpr int NC = BKV / 64;                     // 32-column chunks per warp
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const uint32_t ph = it & 1;
      const int head = kv_head * group + it / q_blocks;
      const int m = nb + it % q_blocks;
      const int q_pos = m * BQ + r;
      const bool valid = q_pos < P.S;
      const int64_t stat = ((int64_t)batch * P.Hq + head) * P.S + q_pos;
      // rows past the end of the sequence: lse = +inf makes every P (and dS) of the row zero
      const float neg_lse2 = valid ? -P.lse[stat] * log2e : -INFINITY;
      const float neg_delta = valid ? -P.delta[stat] : 0.f;
      const uint64_t neg_lse22 = pm::pack2(neg_lse2, neg_lse2);
      const uint64_t neg_delta2 = pm::pack2(neg_delta, neg_delta);
      const bool diag = (m == nb);
      float p[NC][32];
      // ---- S into registers, columns given back at once
      if (!mbar_wait(&bars->s_full, ph)) { atomicCAS(P.err, 0, 432); ok = false; break; }
      tc_fence_after();
      uint32_t sv[NC][32];
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) tmem_ld_32x32(tm_s + lane_addr + (half * NC + cc) * 32, sv[cc]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars->s_free);
      // the P / dS tiles double as the dQ staging area: the previous reduce must have read it
      if (it > 0 && !mbar_wait(&bars->stage_free, (it - 1) & 1)) { atomicCAS(P.err, 0, 433); ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < NC; ++cc) {
        const int c = half * NC + cc;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a, b;
          pm::unpack2(pm::fma2(pm::pack2(__uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1])), scale2,
                               neg_lse22), a, b);
          p[cc][i] = pm::ex2(a);
          p[cc][i + 1] = pm::ex2(b);
        }
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (nb * BKV + c * 32 + i > q_pos) p[cc][i] = 0.f;
        }
        uint8_t* pc = sP + (c / 2) * CHUNK_BYTES;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 w;
          w.x = pm::cvt2<T>(p[cc][u * 8 + 0], p[cc][u * 8 + 1]);
          w.y = pm::cvt2<T>(p[cc][u * 8 + 2], p[cc][u * 8 + 3]);
          w.z = pm::cvt2<T>(p[cc][u * 8 + 4], p[cc][u * 8 + 5]);
          w.w = pm::cvt2<T>(p[cc][u * 8 + 6], p[cc][u * 8 + 7]);
          *reinterpret_cast<uint4*>(pc + swz(r, (c % 2) * 4 + u)) = w;
        }
      }
      fence_proxy_async();
      mbar_arrive(&bars->p_full);
      // ---- dS once dP is complete
      if (!mbar_wait(&bars->dp_full, ph)) { atomicCAS(P.err, 0, 434); ok = false; break; }
      tc_fence_after();
      {
        uint32_t dv[NC][32];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) tmem_ld_32x32(tm_dp + lane_addr + (half * NC + cc) * 32, dv[cc]);
        tmem_ld_wait();
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
          const int c = half * NC + cc;
          uint8_t* dc = sdS + (c / 2) * CHUNK_BYTES;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w[4];
#pragma unroll
            for (int h2 = 0; h2 < 4; ++h2) {
              const int i = u * 8 + h2 * 2;
              float a, b;
              pm::unpack2(pm::mul2(pm::add2(pm::pack2(__uint_as_float(dv[cc][i]), __uint_as_float(dv[cc][i + 1])),
                                            neg_delta2), pm::pack2(p[cc][i], p[cc][i + 1])), a, b);
              w[h2] = pm::cvt2<T>(a, b);
            }
            *reinterpret_cast<uint4*>(dc + swz(r, (c % 2) * 4 + u)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      // orders this thread's reads of the dP columns before the dQ product that overwrites them
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&bars->ds_full);
      if (!mbar_wait(&bars->dq_full, ph)) { atomicCAS(P.err, 0, 435); ok = false; break; }
      tc_fence_after();
      // dQ tile -> fp32 staging (32-column slabs of [128 rows][128 B], 128B-swizzled); rows
      // past the end of the sequence hold exact zeros (their P and dS are zero)
      {
        uint32_t v[D / 64][32];
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) tmem_ld_32x32(tm_dq + lane_addr + (half * (D / 64) + cc) * 32, v[cc]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars->dp_free);                 // the dP columns may be overwritten
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          uint8_t* slab = sP + (half * (D / 64) + cc) * (BQ * 128);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(slab + swz(r, u)) =
                make_uint4(v[cc][u * 4], v[cc][u * 4 + 1], v[cc][u * 4 + 2], v[cc][u * 4 + 3]);
        }
      }
      fence_proxy_async();
      mbar_arrive(&bars->dqs_full);
    }
    if (ok && !mbar_wait(&bars->acc_full, 0)) { atomicCAS(P.err, 0, 436); ok = false; }
    if (ok) {
      tc_fence_after();
      const int kv_pos = nb * BKV + r;
      if (kv_pos < P.S) {
        T* dk_row = reinterpret_cast<T*>(P.dk) + (int64_t)(batch * P.S + kv_pos) * P.dk_stride + kv_head * D;
        T* dv_row = reinterpret_cast<T*>(P.dv) + (int64_t)(batch * P.S + kv_pos) * P.dv_stride + kv_head * D;
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t a[32], b[32];
          tmem_ld_32x32(tm_dk + lane_addr + c * 32, a);
          tmem_ld_32x32(tm_dv + lane_addr + c * 32, b);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float t[8], w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              t[i] = __uint_as_float(a[u * 8 + i]) * P.scale;          // dS carried no softmax scale
              w[i] = __uint_as_float(b[u * 8 + i]);
            }
            *reinterpret_cast<uint4*>(dk_row + c * 32 + u * 8) = pack8<T>(t);
            *reinterpret_cast<uint4*>(dv_row + c * 32 + u * 8) = pack8<T>(w);
          }
        }
      } else {
        // rows past the end of the sequence still have to drain their TMEM loads uniformly
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t a[32];
          tmem_ld_32x32(tm_dk + lane_addr + c * 32, a);
          tmem_ld_wait();
        }
      }
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
