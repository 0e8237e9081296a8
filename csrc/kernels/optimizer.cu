// Device-side optimizer kernels for the HBM-resident share of the partitioned
// state, plus the streaming helpers the engine issues around them.
//
//   ft_adam_cuda        fused Adam / AdamW over fp32 (master, m, v): gradient in
//                       fp32 / bf16 / fp16 multiplied by grad_scale (loss-scale
//                       unscale), update predicated on a device-resident skip
//                       flag, device-dtype parameter copy written in the same pass.
//   ft_check_finite     raises an int32 flag when a buffer holds inf / NaN.
//   ft_accumulate_zero  acc += src; src = 0   (gradient accumulation over
//                       micro-batches into a wider buffer, one pass).
//   ft_cast_copy        dtype-converting flat copy.
//   ft_pinned_alloc     exact-size page-locked host allocation.
//
// The reference keeps all optimizer state on the host
// (flextrain/memory/coordinator/optimizer.py:133-136); these kernels are what
// lets the optimizer live next to the parameters on a 180 GB part.  All are
// HBM-bandwidth bound: 128-bit accesses, grid-stride loops, 148 x 16 blocks max.
#include <atomic>

#include "common.cuh"

namespace {

using namespace ft;

struct AdamArgs {
  float beta2, one_m_beta1, one_m_beta2, eps, step_size, sqrt_bc2, l2_decay, decay_factor, grad_scale;
};

__device__ __forceinline__ float adam_one(const AdamArgs& a, float& p, float g, float& m, float& v) {
  g *= a.grad_scale;
  g += a.l2_decay * p;
  m = m + (g - m) * a.one_m_beta1;
  v = a.beta2 * v + (a.one_m_beta2 * g) * g;
  float denom = sqrtf(v) / a.sqrt_bc2 + a.eps;
  p = p * a.decay_factor - a.step_size * (m / denom);
  return p;
}

template <typename G, typename O, bool kHasOut>
__global__ void __launch_bounds__(256) adam_vec4_kernel(AdamArgs a, float* __restrict__ p,
                                                        const G* __restrict__ g, float* __restrict__ m,
                                                        float* __restrict__ v, O* __restrict__ out,
                                                        int64_t n4, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gv[4];
    if constexpr (sizeof(G) == 4) {
      float4 t = reinterpret_cast<const float4*>(g)[i];
      gv[0] = t.x; gv[1] = t.y; gv[2] = t.z; gv[3] = t.w;
    } else {
      uint2 raw = reinterpret_cast<const uint2*>(g)[i];
      const G* h = reinterpret_cast<const G*>(&raw);
#pragma unroll
      for (int k = 0; k < 4; ++k) gv[k] = to_float(h[k]);
    }
    adam_one(a, pv.x, gv[0], mv.x, vv.x);
    adam_one(a, pv.y, gv[1], mv.y, vv.y);
    adam_one(a, pv.z, gv[2], mv.z, vv.z);
    adam_one(a, pv.w, gv[3], mv.w, vv.w);
    reinterpret_cast<float4*>(p)[i] = pv;
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    if constexpr (kHasOut) {
      if constexpr (sizeof(O) == 4) {
        reinterpret_cast<float4*>(out)[i] = pv;
      } else {
        uint2 raw;
        O* h = reinterpret_cast<O*>(&raw);
        h[0] = from_float<O>(pv.x); h[1] = from_float<O>(pv.y);
        h[2] = from_float<O>(pv.z); h[3] = from_float<O>(pv.w);
        reinterpret_cast<uint2*>(out)[i] = raw;
      }
    }
  }
}

// unaligned heads / tails and odd sizes
__global__ void adam_scalar_kernel(AdamArgs a, float* p, const void* g, int gdt, float* m, float* v,
                                   void* out, int odt, int64_t lo, int64_t n, const int* skip) {
  if (skip != nullptr && *skip != 0) return;
  for (int64_t i = lo + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    float pv = p[i], mv = m[i], vv = v[i];
    adam_one(a, pv, load_as_float(g, gdt, i), mv, vv);
    p[i] = pv; m[i] = mv; v[i] = vv;
    if (out) store_from_float(out, odt, i, pv);
  }
}

template <typename G, typename O>
void launch_adam_vec(const AdamArgs& a, float* p, const void* g, float* m, float* v, void* out,
                     int64_t n4, const int* skip, cudaStream_t s) {
  int grid = grid_for(n4, 256);
  if (out)
    adam_vec4_kernel<G, O, true><<<grid, 256, 0, s>>>(a, p, (const G*)g, m, v, (O*)out, n4, skip);
  else
    adam_vec4_kernel<G, O, false><<<grid, 256, 0, s>>>(a, p, (const G*)g, m, v, (O*)nullptr, n4, skip);
}

template <typename G>
void dispatch_out(int odt, const AdamArgs& a, float* p, const void* g, float* m, float* v, void* out,
                  int64_t n4, const int* skip, cudaStream_t s) {
  if (!out || odt == kF32) launch_adam_vec<G, float>(a, p, g, m, v, out, n4, skip, s);
  else if (odt == kBF16) launch_adam_vec<G, __nv_bfloat16>(a, p, g, m, v, out, n4, skip, s);
  else launch_adam_vec<G, __half>(a, p, g, m, v, out, n4, skip, s);
}

template <typename T>
__global__ void __launch_bounds__(256) check_finite_kernel(const T* __restrict__ x, int64_t n,
                                                           int* __restrict__ flag) {
  // x * 0 is NaN exactly when x is inf or NaN; summing keeps the NaN.
  float acc = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    acc += to_float(x[i]) * 0.f;
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0 && !(acc == 0.f)) atomicOr(flag, 1);
}

template <typename A, typename S>
__global__ void __launch_bounds__(256) accumulate_zero_kernel(A* __restrict__ acc, S* __restrict__ src,
                                                              int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    acc[i] = from_float<A>(to_float(acc[i]) + to_float(src[i]));
    src[i] = from_float<S>(0.f);
  }
}

// fp32 += 16-bit, 8 elements per thread
template <typename S>
__global__ void __launch_bounds__(256) accumulate_zero_vec8_kernel(float* __restrict__ acc,
                                                                   S* __restrict__ src, int64_t n8) {
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8;
       i += (int64_t)gridDim.x * blockDim.x) {
    uint4 raw = reinterpret_cast<uint4*>(src)[i];
    float s[8];
    unpack8<S>(raw, s);
    float4 a0 = reinterpret_cast<float4*>(acc)[2 * i], a1 = reinterpret_cast<float4*>(acc)[2 * i + 1];
    a0.x += s[0]; a0.y += s[1]; a0.z += s[2]; a0.w += s[3];
    a1.x += s[4]; a1.y += s[5]; a1.z += s[6]; a1.w += s[7];
    reinterpret_cast<float4*>(acc)[2 * i] = a0;
    reinterpret_cast<float4*>(acc)[2 * i + 1] = a1;
    reinterpret_cast<uint4*>(src)[i] = zero;
  }
}

template <typename D, typename S>
__global__ void __launch_bounds__(256) cast_copy_kernel(D* __restrict__ dst, const S* __restrict__ src,
                                                        int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_float<D>(to_float(src[i]));
}

template <typename D>
void cast_dispatch_src(D* dst, const void* src, int sdt, int64_t n, cudaStream_t s) {
  int grid = grid_for(n, 256);
  if (sdt == kF32) cast_copy_kernel<D, float><<<grid, 256, 0, s>>>(dst, (const float*)src, n);
  else if (sdt == kBF16) cast_copy_kernel<D, __nv_bfloat16><<<grid, 256, 0, s>>>(dst, (const __nv_bfloat16*)src, n);
  else cast_copy_kernel<D, __half><<<grid, 256, 0, s>>>(dst, (const __half*)src, n);
}

}  // namespace

static std::atomic<long long> g_launches{0};

extern "C" {

long long ft_launch_count() { return g_launches.load(); }
void ft_note_launches(int n) { g_launches.fetch_add(n); }

int ft_adam_cuda(float* p, const void* g, int gdt, float* m, float* v, void* out, int odt, int64_t n,
                 int64_t step, float lr, float beta1, float beta2, float eps, float wd, int adamw,
                 int bias_correction, float grad_scale, const int* skip_flag, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (step < 1) step = 1;
  double bc1 = 1.0, bc2 = 1.0;
  if (bias_correction) {
    bc1 = 1.0 - pow((double)beta1, (double)step);
    bc2 = 1.0 - pow((double)beta2, (double)step);
  }
  AdamArgs a;
  a.beta2 = beta2;
  a.one_m_beta1 = 1.0f - beta1;
  a.one_m_beta2 = 1.0f - beta2;
  a.eps = eps;
  a.step_size = (float)((double)lr / bc1);
  a.sqrt_bc2 = (float)sqrt(bc2);
  a.l2_decay = adamw ? 0.f : wd;
  a.decay_factor = adamw ? (float)(1.0 - (double)lr * (double)wd) : 1.f;
  a.grad_scale = grad_scale;
  if (!out) odt = kNone;
  const int gs = dtype_size(gdt), os = out ? dtype_size(odt) : 4;
  const bool aligned = ((uintptr_t)p % 16 == 0) && ((uintptr_t)m % 16 == 0) && ((uintptr_t)v % 16 == 0) &&
                       ((uintptr_t)g % (4 * gs) == 0) && (!out || (uintptr_t)out % (4 * os) == 0);
  int64_t n4 = aligned ? n / 4 : 0;
  if (n4 > 0) {
    if (gdt == kF32) dispatch_out<float>(odt, a, p, g, m, v, out, n4, skip_flag, stream);
    else if (gdt == kBF16) dispatch_out<__nv_bfloat16>(odt, a, p, g, m, v, out, n4, skip_flag, stream);
    else dispatch_out<__half>(odt, a, p, g, m, v, out, n4, skip_flag, stream);
  }
  if (n4 * 4 < n) {
    int64_t rest = n - n4 * 4;
    adam_scalar_kernel<<<grid_for(rest, 256), 256, 0, stream>>>(a, p, g, gdt, m, v, out, odt, n4 * 4, n,
                                                                skip_flag);
    FT_LAUNCHED(1);
  }
  if (n4 > 0) FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_check_finite(const void* x, int dt, int64_t n, int* flag, cudaStream_t stream) {
  if (n <= 0) return 0;
  int grid = grid_for(n, 256 * 8);
  if (dt == kF32) check_finite_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, n, flag);
  else if (dt == kBF16) check_finite_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, n, flag);
  else check_finite_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)x, n, flag);
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_accumulate_zero(void* acc, int adt, void* src, int sdt, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const bool vec = adt == kF32 && sdt != kF32 && n % 8 == 0 && (uintptr_t)acc % 16 == 0 &&
                   (uintptr_t)src % 16 == 0;
  if (vec) {
    int grid = grid_for(n / 8, 256);
    if (sdt == kBF16) accumulate_zero_vec8_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((float*)acc, (__nv_bfloat16*)src, n / 8);
    else accumulate_zero_vec8_kernel<__half><<<grid, 256, 0, stream>>>((float*)acc, (__half*)src, n / 8);
  } else {
    int grid = grid_for(n, 256);
    if (adt == kF32 && sdt == kF32) accumulate_zero_kernel<float, float><<<grid, 256, 0, stream>>>((float*)acc, (float*)src, n);
    else if (adt == kF32 && sdt == kBF16) accumulate_zero_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>((float*)acc, (__nv_bfloat16*)src, n);
    else if (adt == kF32 && sdt == kF16) accumulate_zero_kernel<float, __half><<<grid, 256, 0, stream>>>((float*)acc, (__half*)src, n);
    else if (adt == kBF16 && sdt == kBF16) accumulate_zero_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)acc, (__nv_bfloat16*)src, n);
    else if (adt == kF16 && sdt == kF16) accumulate_zero_kernel<__half, __half><<<grid, 256, 0, stream>>>((__half*)acc, (__half*)src, n);
    else return -1;
  }
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_cast_copy(void* dst, int ddt, const void* src, int sdt, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (ddt == kF32) cast_dispatch_src<float>((float*)dst, src, sdt, n, stream);
  else if (ddt == kBF16) cast_dispatch_src<__nv_bfloat16>((__nv_bfloat16*)dst, src, sdt, n, stream);
  else cast_dispatch_src<__half>((__half*)dst, src, sdt, n, stream);
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// Exact-size page-locked host memory (PyTorch's pinned allocator rounds to a
// power of two).  Capability parity: flextrain/ops/csrc/aio/py_lib/deepspeed_pin_tensor.cpp:23-61.
void* ft_pinned_alloc(size_t nbytes) {
  void* p = nullptr;
  if (cudaHostAlloc(&p, nbytes, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

int ft_pinned_free(void* p) { return (int)cudaFreeHost(p); }

}  // extern "C"
