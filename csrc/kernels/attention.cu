// Host launchers of the causal flash-attention kernels (attention_fwd*.cuh,
// attention_bwd*.cuh).  q / k / v may be views into one packed QKV tensor: each is
// described by its own base pointer and token stride, rows of H*D columns.
// Replaces the scaled-dot-product attention library call a PyTorch model makes.
#include <cstdlib>

#include "attention_bwd.cuh"
#include "attention_fwd2.cuh"
#include "gemm_host.h"

namespace {

using namespace ft;
using namespace ft::attn;

// dynamic shared memory a CTA may ask for on sm_100 (227 KB)
constexpr int kMaxDynamicSmem = 232448;
static_assert(Fwd2Smem<128>::BYTES <= kMaxDynamicSmem && BwdSmem<128>::BYTES <= kMaxDynamicSmem,
              "an attention kernel outgrew the shared memory of an SM");

// Forward: one CTA per pair of query blocks.
template <typename T, int D, bool TRACE>
int launch_fwd2_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& P,
                  cudaStream_t s) {
  auto kern = attn_fwd2_kernel<T, D, 0x00u, TRACE>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Smem<D>::BYTES);
    configured = true;
  }
  const int num_pairs = ((P.S + BQ - 1) / BQ + 1) / 2;
  kern<<<P.B * P.Hq * num_pairs, F2_THREADS, Fwd2Smem<D>::BYTES, s>>>(tq, tk, tv, P);
  return 0;
}

// The timeline instantiations exist for bf16 at head size 128 only (the benchmark shapes).
template <typename T, int D>
int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& P,
                cudaStream_t s) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value && D == 128) {
    if (P.trace != nullptr) return launch_fwd2_t<T, D, true>(tq, tk, tv, P, s);
  }
  return launch_fwd2_t<T, D, false>(tq, tk, tv, P, s);
}

// Backward: four threads per score row (2.6 % faster than two at the 13B shape, 96 registers
// instead of 158); every other pair of probabilities takes the polynomial 2^x (4.524 ms against
// 4.752 ms with none and 4.635 ms with five of eight at the 13B shape).
constexpr int kBwdSplit = 4;

template <typename T, int D, bool TRACE>
int launch_bwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                 const CUtensorMap& tdq, const BwdParams& P, cudaStream_t s) {
  auto kern = attn_bwd_kernel<T, D, kBwdSplit, TRACE>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<D>::BYTES);
    configured = true;
  }
  const int num_blk = (P.S + BQ - 1) / BQ;
  kern<<<P.B * P.Hkv * num_blk, bwd_threads(kBwdSplit), BwdSmem<D>::BYTES, s>>>(tq, tk, tv, tdo, tdq, P);
  return 0;
}

template <typename T, int D>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               const CUtensorMap& tdq, const BwdParams& P, cudaStream_t s) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value && D == 128) {
    if (P.trace != nullptr) return launch_bwd_t<T, D, true>(tq, tk, tv, tdo, tdq, P, s);
  }
  return launch_bwd_t<T, D, false>(tq, tk, tv, tdo, tdq, P, s);
}

template <typename T>
void launch_pre_post(bool post, const void* o, const void* d_o, int64_t do_stride, float* delta,
                     const float* dq_acc, void* dq, int64_t dq_stride, int B, int S, int Hq, int D,
                     float scale, cudaStream_t s) {
  if (!post) {
    const int64_t rows = (int64_t)B * S * Hq;
    const int per_block = kDeltaRowsPerBlock(D);
    attn_delta_kernel<T><<<(unsigned)((rows + per_block - 1) / per_block), 256, 0, s>>>(
        (const T*)o, (const T*)d_o, do_stride, delta, B, S, Hq, D);
  } else {
    const int64_t tokens = (int64_t)B * S;
    attn_dq_cast_kernel<T><<<grid_for(tokens * (Hq * D / 8), 256), 256, 0, s>>>(dq_acc, (T*)dq, dq_stride,
                                                                                tokens, Hq * D, scale);
  }
}

}  // namespace

extern "C" {

// o[B,S,Hq,D], lse[B,Hq,S] <- causal attention of q[B,S,Hq,D], k/v[B,S,Hkv,D].
// *_stride: elements between consecutive tokens of that tensor.  D in {64, 128}.
// ft_attn_fwd_traced additionally records the timeline of one CTA: `trace` is nullptr or a device
// buffer of 3 * 8 * 8 clock values (see FwdParams).
int ft_attn_fwd_traced(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                       int64_t v_stride, void* o, float* lse, int B, int S, int Hq, int Hkv, int D,
                       float scale, int dtype, cudaStream_t stream, long long* trace, int trace_cta,
                       int trace_it0) {
  if (D != 64 && D != 128) return -1;
  if (dtype != kBF16 && dtype != kF16) return -2;
  if (Hq % Hkv) return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  CUtensorMap tq, tk, tv;
  int rc = gemm::make_tmap(&tq, q, (uint64_t)Hq * D, (uint64_t)B * S, (uint64_t)q_stride, 64, BQ, dtype);
  if (rc) return rc;
  rc = gemm::make_tmap(&tk, k, (uint64_t)Hkv * D, (uint64_t)B * S, (uint64_t)k_stride, 64, BKV, dtype);
  if (rc) return rc;
  rc = gemm::make_tmap(&tv, v, (uint64_t)Hkv * D, (uint64_t)B * S, (uint64_t)v_stride, 64, BKV, dtype);
  if (rc) return rc;
  FwdParams P;
  P.o = o; P.lse = lse; P.B = B; P.S = S; P.Hq = Hq; P.Hkv = Hkv;
  P.scale_log2 = scale * 1.4426950408889634f;
  P.scale_ln = scale;
  P.q_col0 = P.k_col0 = P.v_col0 = 0;
  P.err = gemm::error_word(dev);
  P.trace = trace; P.trace_cta = trace_cta; P.trace_it0 = trace_it0;
  if (dtype == kBF16) {
    if (D == 128) launch_fwd2<__nv_bfloat16, 128>(tq, tk, tv, P, stream);
    else launch_fwd2<__nv_bfloat16, 64>(tq, tk, tv, P, stream);
  } else {
    if (D == 128) launch_fwd2<__half, 128>(tq, tk, tv, P, stream);
    else launch_fwd2<__half, 64>(tq, tk, tv, P, stream);
  }
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_attn_fwd(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                int64_t v_stride, void* o, float* lse, int B, int S, int Hq, int Hkv, int D, float scale,
                int dtype, cudaStream_t stream) {
  return ft_attn_fwd_traced(q, q_stride, k, k_stride, v, v_stride, o, lse, B, S, Hq, Hkv, D, scale, dtype,
                            stream, nullptr, 0, 0);
}

// Gradients of ft_attn_fwd (ft_attn_bwd), optionally with a timeline of one CTA: `trace` is
// nullptr or a device buffer of 5 * 16 * 8 clock values (see BwdParams).  d_o is [B,S,Hq,D] with token stride do_stride; o and
// lse are the forward's outputs.  Scratch provided by the caller: delta
// [B*Hq*S] floats and dq_acc [B*S*Hq*D] floats (zeroed here).  dq / dk / dv are
// written with their own token strides, so they may be views of one packed tensor.
int ft_attn_bwd_traced(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                       int64_t v_stride, const void* o, const void* d_o, int64_t do_stride, const float* lse,
                       float* delta, float* dq_acc, void* dq, int64_t dq_stride, void* dk, int64_t dk_stride,
                       void* dv, int64_t dv_stride, int B, int S, int Hq, int Hkv, int D, float scale,
                       int dtype, cudaStream_t stream, long long* trace, int trace_cta, int trace_it0) {
  if (D != 64 && D != 128) return -1;
  if (dtype != kBF16 && dtype != kF16) return -2;
  if (Hq % Hkv) return -3;
  int dev = 0;
  cudaGetDevice(&dev);
  CUtensorMap tq, tk, tv, tdo;
  int rc = gemm::make_tmap(&tq, q, (uint64_t)Hq * D, (uint64_t)B * S, (uint64_t)q_stride, 64, BQ, dtype);
  if (rc) return rc;
  rc = gemm::make_tmap(&tk, k, (uint64_t)Hkv * D, (uint64_t)B * S, (uint64_t)k_stride, 64, BKV, dtype);
  if (rc) return rc;
  rc = gemm::make_tmap(&tv, v, (uint64_t)Hkv * D, (uint64_t)B * S, (uint64_t)v_stride, 64, BKV, dtype);
  if (rc) return rc;
  rc = gemm::make_tmap(&tdo, d_o, (uint64_t)Hq * D, (uint64_t)B * S, (uint64_t)do_stride, 64, BQ, dtype);
  if (rc) return rc;
  // dq_acc viewed as [B*S, Hq*D] fp32; the kernel adds 128-row x 32-column slabs into it
  CUtensorMap tdq;
  rc = gemm::make_tmap(&tdq, dq_acc, (uint64_t)Hq * D, (uint64_t)B * S, (uint64_t)Hq * D, 32, BQ, kF32);
  if (rc) return rc;
  cudaMemsetAsync(dq_acc, 0, (size_t)B * S * Hq * D * sizeof(float), stream);
  BwdParams P;
  P.lse = lse; P.delta = delta; P.dq_acc = dq_acc;
  P.dk = dk; P.dk_stride = dk_stride; P.dv = dv; P.dv_stride = dv_stride;
  P.B = B; P.S = S; P.Hq = Hq; P.Hkv = Hkv;
  P.scale = scale; P.scale_log2 = scale * 1.4426950408889634f;
  P.err = gemm::error_word(dev);
  P.trace = trace; P.trace_cta = trace_cta; P.trace_it0 = trace_it0;
  if (dtype == kBF16) {
    launch_pre_post<__nv_bfloat16>(false, o, d_o, do_stride, delta, nullptr, nullptr, 0, B, S, Hq, D, scale, stream);
    if (D == 128) launch_bwd<__nv_bfloat16, 128>(tq, tk, tv, tdo, tdq, P, stream);
    else launch_bwd<__nv_bfloat16, 64>(tq, tk, tv, tdo, tdq, P, stream);
    launch_pre_post<__nv_bfloat16>(true, nullptr, nullptr, 0, nullptr, dq_acc, dq, dq_stride, B, S, Hq, D, scale, stream);
  } else {
    launch_pre_post<__half>(false, o, d_o, do_stride, delta, nullptr, nullptr, 0, B, S, Hq, D, scale, stream);
    if (D == 128) launch_bwd<__half, 128>(tq, tk, tv, tdo, tdq, P, stream);
    else launch_bwd<__half, 64>(tq, tk, tv, tdo, tdq, P, stream);
    launch_pre_post<__half>(true, nullptr, nullptr, 0, nullptr, dq_acc, dq, dq_stride, B, S, Hq, D, scale, stream);
  }
  FT_LAUNCHED(3);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_attn_bwd(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                int64_t v_stride, const void* o, const void* d_o, int64_t do_stride, const float* lse,
                float* delta, float* dq_acc, void* dq, int64_t dq_stride, void* dk, int64_t dk_stride,
                void* dv, int64_t dv_stride, int B, int S, int Hq, int Hkv, int D, float scale, int dtype,
                cudaStream_t stream) {
  return ft_attn_bwd_traced(q, q_stride, k, k_stride, v, v_stride, o, d_o, do_stride, lse, delta, dq_acc, dq,
                            dq_stride, dk, dk_stride, dv, dv_stride, B, S, Hq, Hkv, D, scale, dtype, stream,
                            nullptr, 0, 0);
}

}  // extern "C"
