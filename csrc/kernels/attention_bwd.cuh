// Causal grouped-query flash attention, backward, on tcgen05 tensor cores.
//
// One CTA per (batch, kv head, 128-row kv block n).  K_n and V_n stay in shared
// memory; the CTA walks every query head of the group and every query block
// m >= n, and per (head, m):
//   TMA      Q_m, dO_m                      ([64-col chunk][row][64], 128B swizzle)
//   MMA      S  = Q K^T,  dP = dO V^T       -> TMEM (separate completion signals)
//   warps    P  = exp(scale*S - lse) as soon as S is there (dP is still running),
//            then dS = P * (dP - delta); both written as 16-bit tiles [q][kv] into
//            shared memory.  The softmax scale is not applied to dS: dK is scaled
//            once when it is written and dQ by the conversion pass.
//   MMA      dV += P^T dO as soon as P is written (dS is still being computed),
//            dK += dS^T Q (both accumulated in TMEM over the whole walk),
//            dQ_m = dS K                    -> TMEM -> fp32 slabs in shared memory (half of them in
//            memory of their own, half in the dS tile, idle by then) -> one TMA reduce-add per
//            32-column slab into dq_acc, issued by a dedicated warp; nothing of the next block
//            waits for it except the next dS, which needs its tile back
// dO is released for the next load as soon as dV is complete and Q as soon as dK is.
// The same shared-memory bytes serve as K-major operand (reduction over the 64
// contiguous columns) and as MN-major operand (reduction over the rows), so no
// tile is ever transposed.  dK / dV are written once at the end; dq_acc is
// converted to the 16-bit dq by a separate pass.  All waits are bounded.
#pragma once
#include "attention_common.cuh"
#include "packed_math.cuh"

namespace ft {
namespace attn {

// 2 control warps + 4 * SPLIT compute warps + the dQ store warp.  The 128 columns of S / dP (and
// the D columns of dQ / dK / dV) are cut into SPLIT parts; warps 2 + 4 * part .. 5 + 4 * part own
// part `part` (each warp still reads only its own TMEM lane quarter, warp % 4), so every score
// row is shared by SPLIT threads.  The warp after them issues the dQ reduce-adds.
constexpr int bwd_threads(int split) { return 32 * (2 + 4 * split + 1); }

template <int D>
struct BwdSmem {
  static constexpr int TILE = BQ * D * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  // dQ leaves through fp32 slabs of [128 rows][32 columns] (16 KB each).  At head size 128 the
  // first two have shared memory of their own and the last two reuse the dS tile, which is idle
  // between the dQ product and the next dS; at head size 64 both slabs have their own.
  static constexpr int SLAB = BQ * 128;
  static constexpr int OWN_SLABS = 2;
  static constexpr int BYTES = 4 * TILE + 2 * P_BYTES + OWN_SLABS * SLAB + 1024 + 256;
};

struct BwdBars {
  uint64_t kv_full, q_full, do_full, q_empty, do_empty, s_full, dp_full, p_full, ds_full, dq_full, s_free,
      acc_full;
  uint64_t dqs_full, own_free, shared_free;
  uint32_t tmem_base;
  uint32_t abort;
};

struct BwdParams {
  const float* lse;        // [B, Hq, S]
  const float* delta;      // [B, Hq, S]  rowsum(dO * O)
  float* dq_acc;           // [B, S, Hq, D] fp32, zeroed by the caller
  void* dk; int64_t dk_stride;   // [B, S, Hkv, D] with token stride
  void* dv; int64_t dv_stride;
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int* err;
  // timeline capture (TRACE instantiation only): clock64() of CTA trace_cta at the hand-over points
  // of iterations trace_it0 .. trace_it0 + 7, as trace[(role * 16 + site) * 8 + iteration]
  long long* trace;
  int trace_cta, trace_it0;
};

// fp32 tile in shared memory (128B-swizzled [rows][32] slab) added into global memory
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* smem_src, int32_t x,
                                                  int32_t y) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(smem_src)), "r"(x), "r"(y)
      : "memory");
}

// POLY: which of every eight pairs of P values take the polynomial 2^x (bit j = pair j); the
// rest use the special-function unit, so both pipes work on one score row.
template <typename T, int D, int SPLIT, bool TRACE = false, unsigned POLY = 0xAAu>
__global__ void __launch_bounds__(bwd_threads(SPLIT), 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_dq, const __grid_constant__ BwdParams P) {
  constexpr int TILE = BwdSmem<D>::TILE;
  constexpr int CHUNKS = D / 64;
  constexpr int CHUNK_BYTES = BQ * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sP = sdO + TILE;
  uint8_t* sdS = sP + BwdSmem<D>::P_BYTES;
  uint8_t* sStage = sdS + BwdSmem<D>::P_BYTES;
  BwdBars* bars = reinterpret_cast<BwdBars*>(sStage + BwdSmem<D>::OWN_SLABS * BwdSmem<D>::SLAB);
  constexpr int OWN_SLABS = BwdSmem<D>::OWN_SLABS;
  // fp32 slab c of the dQ tile
  auto slab_ptr = [&](int c) -> uint8_t* {
    return c < OWN_SLABS ? sStage + c * BwdSmem<D>::SLAB : sdS + (c - OWN_SLABS) * BwdSmem<D>::SLAB;
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_blk = (P.S + BQ - 1) / BQ;
  const int nb = (int)(blockIdx.x % num_blk);        // kv block; low blocks (most work) first
  const int kv_head = (int)((blockIdx.x / num_blk) % P.Hkv);
  const int batch = (int)(blockIdx.x / (num_blk * P.Hkv));
  const int group = P.Hq / P.Hkv;
  const int q_blocks = num_blk - nb;                 // m = nb .. num_blk-1
  const int iters = group * q_blocks;
  const int kv_row0 = batch * P.S + nb * BKV;
  // role: 0 loads, 1 products, 2 first softmax warp, 3 last softmax warp, 4 dQ reduce warp
  auto stamp = [&](int role, int site, int it) {
    if constexpr (TRACE) {
      if ((int)blockIdx.x == P.trace_cta && it >= P.trace_it0 && it < P.trace_it0 + 8)
        P.trace[(role * 16 + site) * 8 + (it - P.trace_it0)] = clock64();
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->do_full, 1);
    mbar_init(&bars->q_empty, 1);
    mbar_init(&bars->do_empty, 1);
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->p_full, 128 * SPLIT);
    mbar_init(&bars->ds_full, 128 * SPLIT);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->s_free, 128 * SPLIT);
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->dqs_full, 128 * SPLIT);
    mbar_init(&bars->own_free, 1);
    mbar_init(&bars->shared_free, 1);
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
  const uint32_t tm_dq = tmem;                       // reuses the S columns once P is extracted

  if (warp == 0) {
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
        // dO is released first (after the dV product), Q after the dK product
        if (!mbar_wait(&bars->do_empty, (it & 1) ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 401); break; }
        stamp(0, 0, it);
        mbar_expect_tx(&bars->do_full, TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sdO + c * CHUNK_BYTES, &tmap_do, &bars->do_full, head * D + c * 64, q_row0);
        if (!mbar_wait(&bars->q_empty, (it & 1) ^ 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 413); break; }
        stamp(0, 1, it);
        mbar_expect_tx(&bars->q_full, TILE);
        for (int c = 0; c < CHUNKS; ++c)
          tma_load_2d(sQ + c * CHUNK_BYTES, &tmap_q, &bars->q_full, head * D + c * 64, q_row0);
      }
    }
  } else if (warp == 1) {
    // The whole warp runs this loop and an elected lane issues (warp-uniform control flow around
    // the tensor instructions costs the issuer less, and what it spends between two products is
    // time the pipe stands still; csrc/kernels/mma_probe.cu).
    constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
    constexpr uint32_t id_s = make_idesc_f16(AB, 0, 0, BQ, BKV);     // K-major x K-major
    constexpr uint32_t id_t = make_idesc_f16(AB, 1, 1, BKV, D);      // MN-major x MN-major
    constexpr uint32_t id_q = make_idesc_f16(AB, 0, 1, BQ, D);       // K-major x MN-major
    // descriptor halves of the six tiles, prepared once: an instruction then costs two integer adds
    constexpr uint32_t dhi = smem_desc_hi(1024);
    const uint32_t q_k = smem_desc_lo(smem_u32(sQ), 16), k_k = smem_desc_lo(smem_u32(sK), 16),
                   do_k = smem_desc_lo(smem_u32(sdO), 16), v_k = smem_desc_lo(smem_u32(sV), 16),
                   ds_k = smem_desc_lo(smem_u32(sdS), 16);
    const uint32_t p_m = smem_desc_lo(smem_u32(sP), CHUNK_BYTES), do_m = smem_desc_lo(smem_u32(sdO), CHUNK_BYTES),
                   ds_m = smem_desc_lo(smem_u32(sdS), CHUNK_BYTES), q_m = smem_desc_lo(smem_u32(sQ), CHUNK_BYTES),
                   k_m = smem_desc_lo(smem_u32(sK), CHUNK_BYTES);
    auto desc = [&](uint32_t lo, uint32_t off_bytes) { return smem_desc_join(lo + (off_bytes >> 4), dhi); };
    // the lanes poll on their own, so a wait that runs out is made the whole warp's verdict
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity)) != 0;
    };
    bool ok = true;
    auto fail = [&](int code) { if (lane == 0) atomicCAS(P.err, 0, code); ok = false; };
    auto mstamp = [&](int site, int it) { if (TRACE && lane == 0) stamp(1, site, it); };
    if (!wait_all(&bars->kv_full, 0)) fail(402);
    for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
      const uint32_t ph = it & 1;
      mstamp(0, it);
      if (!wait_all(&bars->q_full, ph)) { fail(403); break; }
      mstamp(1, it);
      if (!wait_all(&bars->s_free, ph ^ 1)) { fail(404); break; }
      // dO landed before Q did (it is released first); waiting for it here keeps the sixteen
      // instructions of S and dP back to back
      if (!wait_all(&bars->do_full, ph)) { fail(414); break; }
      mstamp(2, it);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_s, desc(q_k, off), desc(k_k, off), id_s, kk != 0);
        }
        umma_commit(&bars->s_full);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_dp, desc(do_k, off), desc(v_k, off), id_s, kk != 0);
        }
        umma_commit(&bars->dp_full);
      }
      __syncwarp();
      mstamp(3, it);
      if (!wait_all(&bars->p_full, ph)) { fail(405); break; }
      mstamp(4, it);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {       // reduction over the 128 query rows
          const uint32_t row_off = kk * 2048;
          umma_f16(tm_dv, desc(p_m, row_off), desc(do_m, row_off), id_t, (it | kk) != 0);
        }
        umma_commit(&bars->do_empty);
      }
      __syncwarp();
      mstamp(5, it);
      if (!wait_all(&bars->ds_full, ph)) { fail(409); break; }
      mstamp(6, it);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          const uint32_t row_off = kk * 2048;
          umma_f16(tm_dk, desc(ds_m, row_off), desc(q_m, row_off), id_t, (it | kk) != 0);
        }
        umma_commit(&bars->q_empty);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {      // reduction over the 128 kv rows
          const uint32_t a_off = (kk / 4) * CHUNK_BYTES + (kk % 4) * 32;
          umma_f16(tm_dq, desc(ds_k, a_off), desc(k_m, kk * 2048), id_q, kk != 0);
        }
        umma_commit(&bars->dq_full);
      }
      __syncwarp();
      mstamp(7, it);
    }
    if (ok) {
      if (elect_one()) umma_commit(&bars->acc_full);
      __syncwarp();
    } else {
      *abort_flag = 1;
    }
  } else if (warp == 2 + 4 * SPLIT) {
    // ------------------------------------------------------------ dQ store warp
    if (lane == 0) {
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int head = kv_head * group + it / q_blocks;
        const int m = nb + it % q_blocks;
        if (!mbar_wait(&bars->dqs_full, it & 1)) { *abort_flag = 1; atomicCAS(P.err, 0, 411); break; }
        stamp(4, 0, it);
        // the slabs inside the dS tile first: the next dS waits for them to be read
#pragma unroll
        for (int c = OWN_SLABS; c < D / 32; ++c)
          tma_reduce_add_2d(&tmap_dq, slab_ptr(c), head * D + c * 32, batch * P.S + m * BQ);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
#pragma unroll
        for (int c = 0; c < OWN_SLABS && c < D / 32; ++c)
          tma_reduce_add_2d(&tmap_dq, slab_ptr(c), head * D + c * 32, batch * P.S + m * BQ);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        stamp(4, 1, it);
        mbar_arrive(&bars->shared_free);
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        stamp(4, 2, it);
        mbar_arrive(&bars->own_free);
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else {
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;                // which part of the columns this warp owns
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float log2e = 1.4426950408889634f;
    const uint64_t scale2 = pm::pack2(P.scale_log2, P.scale_log2);
    constexpr int NC = BKV / (32 * SPLIT);           // 32-column chunks of S / dP per warp
    static_assert(NC >= 1, "at most four parts of 32 columns");
    // 32-column chunks of dQ / dK / dV per warp; with fewer chunks than parts the last parts have none
    constexpr int DC = (D / 32 >= SPLIT) ? (D / 32) / SPLIT : 1;
    const bool owns_d = part * DC < D / 32;
    bool ok = true;
    // the first and the last softmax warp record the timeline
    const int trole = (lane == 0 && warp == 2) ? 2 : ((lane == 0 && warp == 1 + 4 * SPLIT) ? 3 : -1);
    auto sstamp = [&](int site, int it) { if (TRACE && trole >= 0) stamp(trole, site, it); };
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
      sstamp(0, it);
      // ---- P as soon as S is complete
      if (!mbar_wait(&bars->s_full, ph)) { atomicCAS(P.err, 0, 406); ok = false; break; }
      sstamp(1, it);
      tc_fence_after();
      {
        uint32_t sv[NC][32];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) tmem_ld_32x32(tm_s + lane_addr + (part * NC + cc) * 32, sv[cc]);
        tmem_ld_wait();
        sstamp(3, it);
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
          const int c = part * NC + cc;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float a, b;
            pm::unpack2(pm::fma2(pm::pack2(__uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1])), scale2,
                                 neg_lse22), a, b);
            if ((POLY >> ((i >> 1) & 7)) & 1u) {
              pm::ex2_poly2(a, b, p[cc][i], p[cc][i + 1]);
            } else {
              p[cc][i] = pm::ex2(a);
              p[cc][i + 1] = pm::ex2(b);
            }
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
      }
      sstamp(4, it);
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&bars->p_full);
      sstamp(5, it);
      // ---- dS once dP is complete
      if (!mbar_wait(&bars->dp_full, ph)) { atomicCAS(P.err, 0, 410); ok = false; break; }
      sstamp(6, it);
      // part of the previous dQ tile left through the dS tile: its reduce-add must have read it
      if (it > 0 && !mbar_wait(&bars->shared_free, (it - 1) & 1)) { atomicCAS(P.err, 0, 412); ok = false; break; }
      sstamp(2, it);
      tc_fence_after();
      {
        uint32_t dv[NC][32];
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) tmem_ld_32x32(tm_dp + lane_addr + (part * NC + cc) * 32, dv[cc]);
        tmem_ld_wait();
        sstamp(7, it);
#pragma unroll
        for (int cc = 0; cc < NC; ++cc) {
          const int c = part * NC + cc;
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
      sstamp(8, it);
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(&bars->ds_full);
      sstamp(9, it);
      if (!mbar_wait(&bars->dq_full, ph)) { atomicCAS(P.err, 0, 407); ok = false; break; }
      sstamp(10, it);
      tc_fence_after();
      // dQ tile -> fp32 staging (32-column slabs of [128 rows][128 B], 128B-swizzled); rows
      // past the end of the sequence hold exact zeros (their P and dS are zero)
      if (owns_d) {                                  // uniform per warp
        uint32_t v[DC][32];
#pragma unroll
        for (int cc = 0; cc < DC; ++cc) tmem_ld_32x32(tm_dq + lane_addr + (part * DC + cc) * 32, v[cc]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars->s_free);                  // the S columns may be overwritten
        sstamp(11, it);
        if (it > 0 && !mbar_wait(&bars->own_free, (it - 1) & 1)) { atomicCAS(P.err, 0, 415); ok = false; break; }
#pragma unroll
        for (int cc = 0; cc < DC; ++cc) {
          uint8_t* slab = slab_ptr(part * DC + cc);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            *reinterpret_cast<uint4*>(slab + swz(r, u)) =
                make_uint4(v[cc][u * 4], v[cc][u * 4 + 1], v[cc][u * 4 + 2], v[cc][u * 4 + 3]);
        }
      } else {
        tc_fence_before();
        mbar_arrive(&bars->s_free);
      }
      fence_proxy_async();
      mbar_arrive(&bars->dqs_full);
      sstamp(12, it);
    }
    if (ok && !mbar_wait(&bars->acc_full, 0)) { atomicCAS(P.err, 0, 408); ok = false; }
    if (ok) {
      tc_fence_after();
      const int kv_pos = nb * BKV + r;
      // every lane of a warp issues the same tensor-memory loads (they are warp-wide
      // instructions); only the stores depend on whether the lane's row exists
      const bool row_ok = kv_pos < P.S;
      const int64_t row = (int64_t)(batch * P.S + (row_ok ? kv_pos : 0));
      T* dk_row = reinterpret_cast<T*>(P.dk) + row * P.dk_stride + kv_head * D;
      T* dv_row = reinterpret_cast<T*>(P.dv) + row * P.dv_stride + kv_head * D;
#pragma unroll 1
      for (int c = part * DC; owns_d && c < (part + 1) * DC; ++c) {
        uint32_t a[32], b[32];
        tmem_ld_32x32(tm_dk + lane_addr + c * 32, a);
        tmem_ld_32x32(tm_dv + lane_addr + c * 32, b);
        tmem_ld_wait();
        if (row_ok) {
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
      }
    } else {
      *abort_flag = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// delta[b,h,s] = sum_d dO * O.  D / 8 lanes per (head, token) row (16 bytes of each tensor per
// lane), so a warp covers 32 * 8 / D rows at once, and every thread does that for two rows with
// all four loads in flight.  Rows are numbered in the order of delta ([b, h, s]), so neighbouring
// lanes write neighbouring floats; the reads are whole 2 * D-byte pieces either way.  D in {64, 128}.
constexpr int kDeltaRowsPerBlock(int D) { return 2 * 8 * (256 / D); }   // 2 passes x 8 warps x rows per warp

template <typename T>
__global__ void __launch_bounds__(256) attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                         int64_t do_stride, float* __restrict__ delta,
                                                         int B, int S, int Hq, int D) {
  const int lpr = D / 8, rpw = 32 / lpr;             // lanes per row, rows per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % lpr;
  const int64_t rows = (int64_t)B * S * Hq;
  const int64_t row0 = (int64_t)blockIdx.x * (2 * 8 * rpw) + warp * rpw + lane / lpr;
  float acc[2];
  uint4 a[2], b[2];
  bool ok[2];
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int64_t row = row0 + (int64_t)p * 8 * rpw;
    ok[p] = row < rows;
    const int64_t r = ok[p] ? row : 0;
    const int64_t bh = r / S;
    const int64_t tok = (bh / Hq) * S + r % S;
    const int h = (int)(bh % Hq);
    a[p] = *reinterpret_cast<const uint4*>(o + (tok * Hq + h) * D + sub * 8);
    b[p] = *reinterpret_cast<const uint4*>(d_o + tok * do_stride + (int64_t)h * D + sub * 8);
  }
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    float x[8], y[8];
    unpack8<T>(a[p], x);
    unpack8<T>(b[p], y);
    acc[p] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[p] += x[k] * y[k];
    for (int off = lpr / 2; off > 0; off >>= 1) acc[p] += __shfl_xor_sync(0xffffffffu, acc[p], off);
    const int64_t row = row0 + (int64_t)p * 8 * rpw;
    if (ok[p] && sub == 0) delta[row] = acc[p];
  }
}

// dq (16-bit, token stride) <- scale * dq_acc (fp32, contiguous [tokens, W])
template <typename T>
__global__ void __launch_bounds__(256) attn_dq_cast_kernel(const float* __restrict__ acc, T* __restrict__ dq,
                                                           int64_t dq_stride, int64_t tokens, int W,
                                                           float scale) {
  const int vec = W / 8;
  const int64_t total = tokens * vec;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vec;
    const int c = (int)(idx % vec) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + t * W + c);
    const float4 b = *reinterpret_cast<const float4*>(acc + t * W + c + 4);
    float v[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                  b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    *reinterpret_cast<uint4*>(dq + t * dq_stride + c) = pack8<T>(v);
  }
}

}  // namespace attn
}  // namespace ft
