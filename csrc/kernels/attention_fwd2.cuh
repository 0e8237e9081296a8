// Causal grouped-query flash attention, forward, second generation.
//
// One CTA per (batch, query head, PAIR of 128-row query blocks).  Both query tiles
// share every K/V block that streams through a 2-stage TMA ring, and while the
// softmax of one tile runs the tensor core works on the other tile:
//   warp 0      TMA producer (Q tiles once, then K_j / V_j)
//   warp 1      MMA issuer, in the order  PV0(j) QK0(j+1) PV1(j) QK1(j+1)
//   warps 2-5   softmax of tile 0;  warps 6-9  softmax of tile 1 (one row per thread)
// Tensor memory (512 columns): S0 | S1 | O0 | O1.  The probabilities P_j are
// written back into the first 64 columns of their S buffer as packed 16-bit pairs
// and the P V product takes its A operand straight from tensor memory, so P never
// touches shared memory.  O accumulates in tensor memory across the K/V blocks;
// it is rescaled only when some row's maximum grew by more than 2^8 (the stale
// maximum is used consistently for P, the row sum and the final log-sum-exp, so
// the result is exact).  The softmax arithmetic uses the two-wide fp32
// instructions and the bare ex2 approximation (packed_math.cuh).
// Outputs: O [B,S,Hq,D] (16-bit) and lse [B,Hq,S] (fp32, natural log of the row sums).  All waits
// are bounded.
#pragma once
#include "attention_common.cuh"
#include "packed_math.cuh"

namespace ft {
namespace attn {

constexpr int F2_THREADS = 320;
constexpr float kRescaleLog2 = 8.f;

template <int D>
struct Fwd2Smem {
  static constexpr int TILE = BQ * D * 2;
  static constexpr int BYTES = 2 * TILE + 2 * KV_STAGES * TILE + 1024 + 256;
};

struct Fwd2Bars {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  uint32_t abort;
};

// POLY: which of every eight pairs of probabilities take the polynomial 2^x of packed_math.cuh
// (bit j = pair j) instead of the special-function unit.  None by default: with one thread per
// score row the extra instructions cost more than the unit's 16 results per clock (13B shape:
// 1.362 ms with none, 1.387 / 1.412 / 1.427 ms with one / two / three pairs of eight).
template <typename T, int D, unsigned POLY = 0x00u, bool TRACE = false>
__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ FwdParams P) {
  constexpr int TILE = Fwd2Smem<D>::TILE;
  constexpr int CHUNKS = D / 64;
  constexpr int CHUNK_BYTES = BQ * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                                // two tiles
  uint8_t* sK = sQ + 2 * TILE;
  uint8_t* sV = sK + KV_STAGES * TILE;
  Fwd2Bars* bars = reinterpret_cast<Fwd2Bars*>(sV + KV_STAGES * TILE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_qb = (P.S + BQ - 1) / BQ;
  const int num_pairs = (num_qb + 1) / 2;
  const int pi = num_pairs - 1 - (int)(blockIdx.x % num_pairs);      // heaviest pairs first
  const int head = (int)((blockIdx.x / num_pairs) % P.Hq);
  const int batch = (int)(blockIdx.x / (num_pairs * P.Hq));
  const int kv_head = head / (P.Hq / P.Hkv);
  const int qb0 = 2 * pi, qb1 = 2 * pi + 1;
  const int n0 = qb0 + 1;                            // K/V blocks tile 0 needs (causal)
  const int n1 = qb1 < num_qb ? qb1 + 1 : 0;         // tile 1 may not exist
  const int nmax = n0 > n1 ? n0 : n1;
  // role: 0 product warp, 1 first softmax warp of tile 0, 2 first softmax warp of tile 1
  auto stamp = [&](int role, int site, int j) {
    if constexpr (TRACE) {
      if ((int)blockIdx.x == P.trace_cta && j >= P.trace_it0 && j < P.trace_it0 + 8)
        P.trace[(role * 8 + site) * 8 + (j - P.trace_it0)] = clock64();
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1); mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1); mbar_init(&bars->v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_full[t], 128);
      mbar_init(&bars->o_full[t], 1);
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
      for (int j = 0; j < nmax && !*abort_flag; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int kv_row0 = batch * P.S + j * BKV;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 321); break; }
        mbar_expect_tx(&bars->k_full[s], TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sK + s * TILE + c * CHUNK_BYTES, &tmap_k, &bars->k_full[s],
                      P.k_col0 + kv_head * D + c * 64, kv_row0);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 322); break; }
        mbar_expect_tx(&bars->v_full[s], TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sV + s * TILE + c * CHUNK_BYTES, &tmap_v, &bars->v_full[s],
                      P.v_col0 + kv_head * D + c * 64, kv_row0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA
    // The whole warp runs this loop and one elected lane issues: with warp-uniform control flow
    // around them the waits, fences and commits between two products cost the issuing thread
    // less, and what they cost is time the tensor pipe stands still (its queue covers about two
    // 128-wide instructions; csrc/kernels/mma_probe.cu, issue styles 1 and 2).  K_j and V_j are
    // waited for once per block, not once per tile.
    constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr uint32_t idesc_s = make_idesc_f16(AB, 0, 0, BQ, BKV);      // Q, K both K-major
    constexpr uint32_t idesc_o = make_idesc_f16(AB, 0, 1, BQ, D);        // P (tmem) K-major, V MN-major
    constexpr uint32_t dhi = smem_desc_hi(1024);
    const uint32_t q_lo[2] = {smem_desc_lo(smem_u32(sQ), 16), smem_desc_lo(smem_u32(sQ + TILE), 16)};
    uint32_t k_lo[KV_STAGES], v_lo[KV_STAGES];
#pragma unroll
    for (int s = 0; s < KV_STAGES; ++s) {
      k_lo[s] = smem_desc_lo(smem_u32(sK + s * TILE), 16);
      v_lo[s] = smem_desc_lo(smem_u32(sV + s * TILE), CHUNK_BYTES);
    }
    bool ok = true;
    auto fail = [&](int code) { if (lane == 0) atomicCAS(P.err, 0, code); ok = false; };
    // the lanes poll on their own, so a wait that runs out is made the whole warp's verdict
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
    };
    // S_t = Q_t K_j^T
    auto qk_issue = [&](int t, int j) {
      const int s = j % KV_STAGES;
      const uint32_t ql = q_lo[t], kl = k_lo[s];
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = ((kk / 4) * CHUNK_BYTES + (kk % 4) * 32) >> 4;
        umma_f16(tmem + t * 128, smem_desc_join(ql + off, dhi), smem_desc_join(kl + off, dhi), idesc_s, kk != 0);
      }
      if (t == 1 || j >= n1) umma_commit(&bars->k_empty[s]);       // last reader of K_j
      umma_commit(&bars->s_full[t]);
    };
    // O_t += P_t V_j
    auto pv_issue = [&](int t, int j) {
      const int s = j % KV_STAGES;
      const uint32_t vl = v_lo[s];
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk)
        umma_f16_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, smem_desc_join(vl + kk * 128, dhi), idesc_o,
                    (j | kk) != 0);
      if (t == 1 || j >= n1) umma_commit(&bars->v_empty[s]);       // last reader of V_j
      umma_commit(&bars->o_full[t]);
    };
    // One hand-over per tile and block: everything PV_t(j) and QK_t(j+1) wait for is waited for
    // first (K_{j+1} landed long ago, its stage was released a block earlier), then the sixteen
    // instructions go out back to back with their commits behind them.
    // first_v / first_k: this tile is the first to read V_j / K_{j+1} and waits for it to land
    auto tile_step = [&](int t, int j, int n_t, bool first_v, bool first_k) {
      const bool has_pv = j < n_t, has_qk = j + 1 < n_t;
      if (has_pv) {
        if (first_v && !wait_all(&bars->v_full[j % KV_STAGES], (j / KV_STAGES) & 1)) { fail(324); return; }
        if (!wait_all(&bars->p_full[t], j & 1)) { fail(325); return; }
      }
      if (has_qk && first_k &&
          !wait_all(&bars->k_full[(j + 1) % KV_STAGES], ((j + 1) / KV_STAGES) & 1)) { fail(323); return; }
      if (!has_pv && !has_qk) return;
      tc_fence_after();
      if (elect_one()) {
        stamp(0, 1 + 3 * t, j);
        if (has_pv) pv_issue(t, j);
        stamp(0, 2 + 3 * t, j);
        if (has_qk) qk_issue(t, j + 1);
        stamp(0, 3 + 3 * t, j);
      }
      __syncwarp();
    };
    if (!wait_all(&bars->q_full, 0)) fail(320);
    if (ok && !wait_all(&bars->k_full[0], 0)) fail(323);
    if (ok) {
      tc_fence_after();
      if (elect_one()) {
        qk_issue(0, 0);
        if (n1 > 0) qk_issue(1, 0);
      }
      __syncwarp();
    }
    for (int j = 0; j < nmax && ok && !*abort_flag; ++j) {
      if (lane == 0) stamp(0, 0, j);
      tile_step(0, j, n0, true, true);
      if (ok) tile_step(1, j, n1, j >= n0, j + 1 >= n0);     // tile 1 is first only where tile 0 has no product
    }
    if (!ok) *abort_flag = 1;
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
    const int trole = (lane == 0 && quarter == 2) ? 1 + t : -1;     // warps 2 and 6
    auto sstamp = [&](int site, int j) { if (TRACE && trole >= 0) stamp(trole, site, j); };
    for (int j = 0; j < n_t; ++j) {
      sstamp(0, j);
      if (!mbar_wait(&bars->s_full[t], j & 1)) { atomicCAS(P.err, 0, 326); ok = false; break; }
      sstamp(1, j);
      tc_fence_after();
      const bool diag = (j == qb);
      const int kv0 = j * BKV;
      // the whole S row goes to registers once: four loads in flight, one wait
      uint32_t v[BKV / 32][32];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld_32x32(tm_s + c * 32, v[c]);
      tmem_ld_wait();
      sstamp(2, j);
      if (diag) {
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + c * 32 + i > q_pos) v[c][i] = 0xff800000u;     // -inf
      }
      float mx[BKV / 32];                            // independent chains, one per chunk
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        mx[c] = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx[c] = pm::max3(mx[c], __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
      }
      const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // rescale O only when some row of the warp outgrew its maximum by more than 2^8
      const bool grow = (m_blk - m_used) * P.scale_log2 > kRescaleLog2;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, m_blk);
        if (j > 0) {
          if (!mbar_wait(&bars->o_full[t], (j - 1) & 1)) { atomicCAS(P.err, 0, 327); ok = false; break; }
          tc_fence_after();
          const float alpha = pm::ex2((m_used - m_new) * P.scale_log2);
          const uint64_t alpha2 = pm::pack2(alpha, alpha);
          // Sixteen columns at a time: this rare path must not cost the common one registers (with
          // 32-column pieces the kernel spilled 230-250 bytes per thread and the 13B shape took
          // 1.403 ms instead of 1.342).
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {
            uint32_t w[16];
            tmem_ld_32x16(tm_o + c * 16, w);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              float a, b;
              pm::unpack2(pm::mul2(pm::pack2(__uint_as_float(w[i]), __uint_as_float(w[i + 1])), alpha2), a, b);
              w[i] = __float_as_uint(a);
              w[i + 1] = __float_as_uint(b);
            }
            tmem_st_32x16(tm_o + c * 16, w);
          }
          l_run *= alpha;
        }
        m_used = m_new;
      }
      sstamp(3, j);
      // p = 2^((s - m) * scale), row sum, P written over the first half of S
      const float neg_m = -m_used * P.scale_log2;
      const uint64_t neg_m2 = pm::pack2(neg_m, neg_m);
      uint64_t ls[BKV / 32];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        ls[c] = pm::pack2(0.f, 0.f);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a, b;
          pm::unpack2(pm::fma2(pm::pack2(__uint_as_float(v[c][2 * i]), __uint_as_float(v[c][2 * i + 1])), scale2,
                               neg_m2), a, b);
          if ((POLY >> (i & 7)) & 1u) {
            pm::ex2_poly2(a, b, a, b);
          } else {
            a = pm::ex2(a);
            b = pm::ex2(b);
          }
          ls[c] = pm::add2(ls[c], pm::pack2(a, b));
          pk[i] = pm::cvt2<T>(a, b);
        }
        tmem_st_32x16(tm_s + c * 16, pk);
      }
      const uint64_t l2 = pm::add2(pm::add2(ls[0], ls[1]), pm::add2(ls[2], ls[3]));
      float la, lb;
      pm::unpack2(l2, la, lb);
      l_run += la + lb;
      sstamp(4, j);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->p_full[t]);
      sstamp(5, j);
    }
    if (ok && n_t > 0) {
      if (!mbar_wait(&bars->o_full[t], (n_t - 1) & 1)) { atomicCAS(P.err, 0, 328); ok = false; }
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
