// Host-side Adam / AdamW for the DRAM-resident share of the partitioned
// optimizer state.
//
// One pass over (master fp32, grad, m, v) that also: multiplies the gradient by
// `grad_scale` (loss-scale unscale and 1/world folded together), optionally
// detects non-finite gradients, and writes a device-dtype copy (bf16 / fp16 /
// fp32) of the updated parameter straight into the pinned buffer the next
// host->device copy reads.  AVX-512 path selected at run time, portable scalar
// path otherwise; OpenMP over fixed-size blocks so results do not depend on the
// thread count.
//
// Capability parity: flextrain/ops/csrc/includes/cpu_adam.h:30-217,
// flextrain/ops/csrc/adam/cpu_adam_impl.cpp:20-302, flextrain/ops/csrc/includes/simd.h.
// Unlike that kernel the half-precision copy honours bf16 (the reference
// always emits fp16 bit patterns, simd.h:33-37).
#include <immintrin.h>
#include "omp_compat.h"

#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>

namespace {

enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2, kNone = -1 };

struct AdamConfig {
  float lr, beta1, beta2, eps, weight_decay;
  int adamw;
};

std::mutex g_registry_mu;
std::map<int, AdamConfig> g_registry;

struct StepConsts {
  float beta1, beta2, one_m_beta1, one_m_beta2;
  float eps, step_size, sqrt_bc2;
  float l2_decay;      // added to the gradient (classic Adam)
  float decay_factor;  // 1 - lr * wd, AdamW (1 when classic)
  float grad_scale;
};

inline StepConsts make_consts(int64_t step, float lr, float b1, float b2, float eps, float wd,
                              int adamw, int bias_correction, float grad_scale) {
  StepConsts c;
  c.beta1 = b1;
  c.beta2 = b2;
  c.one_m_beta1 = 1.0f - b1;
  c.one_m_beta2 = 1.0f - b2;
  c.eps = eps;
  double bc1 = 1.0, bc2 = 1.0;
  if (bias_correction) {
    bc1 = 1.0 - std::pow((double)b1, (double)step);
    bc2 = 1.0 - std::pow((double)b2, (double)step);
  }
  c.step_size = (float)((double)lr / bc1);
  c.sqrt_bc2 = (float)std::sqrt(bc2);
  c.l2_decay = adamw ? 0.0f : wd;
  c.decay_factor = adamw ? (float)(1.0 - (double)lr * (double)wd) : 1.0f;
  c.grad_scale = grad_scale;
  return c;
}

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

inline float f16_to_f32(uint16_t h) { return _cvtsh_ss(h); }
inline uint16_t f32_to_f16(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT); }

inline float load_grad(const void* g, int dtype, int64_t i) {
  switch (dtype) {
    case kBF16: return bf16_to_f32(((const uint16_t*)g)[i]);
    case kF16: return f16_to_f32(((const uint16_t*)g)[i]);
    default: return ((const float*)g)[i];
  }
}

inline void store_copy(void* out, int dtype, int64_t i, float p) {
  switch (dtype) {
    case kBF16: ((uint16_t*)out)[i] = f32_to_bf16(p); break;
    case kF16: ((uint16_t*)out)[i] = f32_to_f16(p); break;
    case kF32: ((float*)out)[i] = p; break;
    default: break;
  }
}

// ------------------------------------------------------------------ scalar
__attribute__((target("f16c"))) bool adam_block_scalar(
    const StepConsts& c, float* p, const void* g, int gdt, float* m, float* v, void* out, int odt,
    int64_t lo, int64_t hi) {
  bool bad = false;
  for (int64_t i = lo; i < hi; ++i) {
    float grad = load_grad(g, gdt, i) * c.grad_scale;
    bad |= !std::isfinite(grad);
    float param = p[i];
    grad += c.l2_decay * param;
    float mi = m[i] + (grad - m[i]) * c.one_m_beta1;
    float vi = c.beta2 * v[i] + (c.one_m_beta2 * grad) * grad;
    float denom = std::sqrt(vi) / c.sqrt_bc2 + c.eps;
    param *= c.decay_factor;
    param -= c.step_size * (mi / denom);
    m[i] = mi;
    v[i] = vi;
    p[i] = param;
    store_copy(out, odt, i, param);
  }
  return bad;
}

// ----------------------------------------------------------------- AVX-512
#define FT_AVX512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512dq,f16c")))

FT_AVX512 inline __m512 load_grad16(const void* g, int dtype, int64_t i) {
  if (dtype == kF32) return _mm512_loadu_ps((const float*)g + i);
  __m256i h = _mm256_loadu_si256((const __m256i*)((const uint16_t*)g + i));
  if (dtype == kBF16)
    return _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(h), 16));
  return _mm512_cvtph_ps(h);
}

FT_AVX512 inline __m256i f32x16_to_bf16(__m512 x) {
  __m512i u = _mm512_castps_si512(x);
  __m512i lsb = _mm512_and_si512(_mm512_srli_epi32(u, 16), _mm512_set1_epi32(1));
  __m512i rounded = _mm512_add_epi32(u, _mm512_add_epi32(lsb, _mm512_set1_epi32(0x7fff)));
  __mmask16 nan = _mm512_cmp_ps_mask(x, x, _CMP_UNORD_Q);
  __m512i quiet = _mm512_or_si512(u, _mm512_set1_epi32(0x00400000));
  rounded = _mm512_mask_mov_epi32(rounded, nan, quiet);
  return _mm512_cvtepi32_epi16(_mm512_srli_epi32(rounded, 16));
}

FT_AVX512 inline void store_copy16(void* out, int dtype, int64_t i, __m512 p) {
  if (dtype == kBF16) {
    _mm256_storeu_si256((__m256i*)((uint16_t*)out + i), f32x16_to_bf16(p));
  } else if (dtype == kF16) {
    _mm256_storeu_si256((__m256i*)((uint16_t*)out + i),
                        _mm512_cvtps_ph(p, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
  } else if (dtype == kF32) {
    _mm512_storeu_ps((float*)out + i, p);
  }
}

FT_AVX512 bool adam_block_avx512(const StepConsts& c, float* p, const void* g, int gdt, float* m,
                                 float* v, void* out, int odt, int64_t lo, int64_t hi) {
  const __m512 b2 = _mm512_set1_ps(c.beta2);
  const __m512 ob1 = _mm512_set1_ps(c.one_m_beta1), ob2 = _mm512_set1_ps(c.one_m_beta2);
  const __m512 eps = _mm512_set1_ps(c.eps), step = _mm512_set1_ps(c.step_size);
  const __m512 sbc2 = _mm512_set1_ps(c.sqrt_bc2), l2 = _mm512_set1_ps(c.l2_decay);
  const __m512 dec = _mm512_set1_ps(c.decay_factor), gs = _mm512_set1_ps(c.grad_scale);
  const __m512 inf = _mm512_set1_ps(INFINITY);
  const __m512 absmask = _mm512_castsi512_ps(_mm512_set1_epi32(0x7fffffff));
  __mmask16 bad = 0;
  int64_t i = lo;
  for (; i + 16 <= hi; i += 16) {
    __m512 grad = _mm512_mul_ps(load_grad16(g, gdt, i), gs);
    // non-finite <=> !(|g| < inf)   (NaN compares false)
    bad |= (__mmask16)~_mm512_cmp_ps_mask(_mm512_and_ps(grad, absmask), inf, _CMP_LT_OQ);
    __m512 param = _mm512_loadu_ps(p + i);
    grad = _mm512_add_ps(grad, _mm512_mul_ps(l2, param));
    __m512 m_old = _mm512_loadu_ps(m + i);
    __m512 mi = _mm512_add_ps(m_old, _mm512_mul_ps(_mm512_sub_ps(grad, m_old), ob1));
    __m512 vi = _mm512_add_ps(_mm512_mul_ps(b2, _mm512_loadu_ps(v + i)),
                              _mm512_mul_ps(_mm512_mul_ps(ob2, grad), grad));
    __m512 denom = _mm512_add_ps(_mm512_div_ps(_mm512_sqrt_ps(vi), sbc2), eps);
    param = _mm512_mul_ps(param, dec);
    param = _mm512_sub_ps(param, _mm512_mul_ps(step, _mm512_div_ps(mi, denom)));
    _mm512_storeu_ps(m + i, mi);
    _mm512_storeu_ps(v + i, vi);
    _mm512_storeu_ps(p + i, param);
    store_copy16(out, odt, i, param);
  }
  bool tail_bad = false;
  if (i < hi) tail_bad = adam_block_scalar(c, p, g, gdt, m, v, out, odt, i, hi);
  return bad != 0 || tail_bad;
}

bool cpu_has_avx512() {
  static const bool ok = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
                         __builtin_cpu_supports("avx512vl") && __builtin_cpu_supports("avx512dq");
  return ok;
}

constexpr int64_t kBlock = 1 << 16;  // elements per OpenMP work item

}  // namespace

extern "C" {

// 1: AVX-512 kernels are in use, 0: portable path.
int ft_adam_simd_level() { return cpu_has_avx512() ? 512 : 0; }

// Registry kept for API parity with create_adam/destroy_adam of the reference
// binding (flextrain/ops/csrc/adam/cpu_adam.cpp:8-16).  Hyper-parameters are
// passed again on every update call, so the registry only stores defaults.
int ft_adam_create(int id, float lr, float beta1, float beta2, float eps, float weight_decay,
                   int adamw) {
  std::lock_guard<std::mutex> lk(g_registry_mu);
  g_registry[id] = AdamConfig{lr, beta1, beta2, eps, weight_decay, adamw};
  return 0;
}

int ft_adam_destroy(int id) {
  std::lock_guard<std::mutex> lk(g_registry_mu);
  return g_registry.erase(id) ? 0 : -1;
}

// Returns 0 on success, 1 if a non-finite (scaled) gradient was seen, <0 on bad
// arguments.  `force_scalar` selects the portable path (tests compare the two).
int ft_adam_update(int64_t step, float lr, float beta1, float beta2, float eps, float weight_decay,
                   int adamw, int bias_correction, float grad_scale, float* param, const void* grad,
                   int grad_dtype, float* exp_avg, float* exp_avg_sq, int64_t n, void* out_copy,
                   int copy_dtype, int threads, int force_scalar) {
  if (n < 0 || !param || !grad || !exp_avg || !exp_avg_sq) return -1;
  if (grad_dtype < kF32 || grad_dtype > kF16) return -2;
  if (!out_copy) copy_dtype = kNone;
  if (step < 1) step = 1;
  const StepConsts c =
      make_consts(step, lr, beta1, beta2, eps, weight_decay, adamw, bias_correction, grad_scale);
  const bool simd = cpu_has_avx512() && !force_scalar;
  const int64_t blocks = (n + kBlock - 1) / kBlock;
  int bad = 0;
  if (threads <= 0) threads = omp_get_max_threads();
  if (blocks < threads) threads = (int)(blocks > 0 ? blocks : 1);
#pragma omp parallel for num_threads(threads) schedule(static) reduction(| : bad)
  for (int64_t b = 0; b < blocks; ++b) {
    int64_t lo = b * kBlock, hi = lo + kBlock < n ? lo + kBlock : n;
    bool r = simd ? adam_block_avx512(c, param, grad, grad_dtype, exp_avg, exp_avg_sq, out_copy,
                                      copy_dtype, lo, hi)
                  : adam_block_scalar(c, param, grad, grad_dtype, exp_avg, exp_avg_sq, out_copy,
                                      copy_dtype, lo, hi);
    bad |= r ? 1 : 0;
  }
  return bad;
}

// 1 if any element of `grad` times `grad_scale` is inf/nan, else 0.
int ft_has_nonfinite(const void* grad, int grad_dtype, int64_t n, int threads) {
  const int64_t blocks = (n + kBlock - 1) / kBlock;
  int bad = 0;
  if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static) reduction(| : bad)
  for (int64_t b = 0; b < blocks; ++b) {
    int64_t lo = b * kBlock, hi = lo + kBlock < n ? lo + kBlock : n;
    float acc = 0.f;
    for (int64_t i = lo; i < hi; ++i) acc += load_grad(grad, grad_dtype, i) * 0.0f;
    bad |= std::isfinite(acc) ? 0 : 1;  // x*0 is NaN exactly when x is inf or NaN
  }
  return bad;
}

// dst[i] = (dtype) src[i], fp32 source.  Used to seed device-dtype parameter
// copies from master weights.
int ft_cast_from_f32(const float* src, void* dst, int dst_dtype, int64_t n, int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
  const int64_t blocks = (n + kBlock - 1) / kBlock;
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    int64_t lo = b * kBlock, hi = lo + kBlock < n ? lo + kBlock : n;
    for (int64_t i = lo; i < hi; ++i) store_copy(dst, dst_dtype, i, src[i]);
  }
  return 0;
}

// dst[i] = (float) src[i] for bf16 / fp16 / fp32 sources.
int ft_cast_to_f32(const void* src, int src_dtype, float* dst, int64_t n, int threads) {
  if (threads <= 0) threads = omp_get_max_threads();
  const int64_t blocks = (n + kBlock - 1) / kBlock;
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    int64_t lo = b * kBlock, hi = lo + kBlock < n ? lo + kBlock : n;
    for (int64_t i = lo; i < hi; ++i) dst[i] = load_grad(src, src_dtype, i);
  }
  return 0;
}

}  // extern "C"
