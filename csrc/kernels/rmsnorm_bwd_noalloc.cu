// RMSNorm backward that allocates nothing: the per-CTA partial sums of the
// weight gradient live in a file-scope device array instead of a caller-provided
// scratch buffer.  See no_alloc.h for who needs this and for the contract.
#include "common.cuh"
#include "no_alloc.h"

namespace {

using namespace ft;

constexpr int kParts = FT_RMSNORM_NOALLOC_PARTS;
constexpr int kMaxH = FT_RMSNORM_NOALLOC_MAX_H;

// Partial weight gradients, [kParts][H] floats, one copy per device.
static __device__ __align__(256) float g_dw_scratch[(size_t)kParts * kMaxH];

// In host code `g_dw_scratch` is only a handle for the symbol, not an address a
// kernel can use; the real device address is fetched once per device.
float* g_scratch_addr[64] = {nullptr};

template <typename T>
__global__ void __launch_bounds__(256) bwd_partial_kernel(const T* __restrict__ x,
                                                          const T* __restrict__ w,
                                                          const T* __restrict__ dy,
                                                          const float* __restrict__ inv_rms,
                                                          T* __restrict__ dx, float* __restrict__ part,
                                                          int64_t rows, int H) {
  __shared__ float red[32];
  const int nvec = H / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  constexpr int kMaxVec = kMaxH / (8 * 256);
  float acc[kMaxVec][8];
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[j][k] = 0.f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
    uint4* dr = reinterpret_cast<uint4*>(dx + row * H);
    const float inv = inv_rms[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < nvec) {
        float xv[8], gv[8], wv[8];
        unpack8<T>(xr[i], xv);
        unpack8<T>(gr[i], gv);
        unpack8<T>(wr[i], wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot += gv[k] * wv[k] * xv[k];
          acc[j][k] += gv[k] * xv[k] * inv;
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = dot * inv * inv / (float)H;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < nvec) {
        float xv[8], gv[8], wv[8], o[8];
        unpack8<T>(xr[i], xv);
        unpack8<T>(gr[i], gv);
        unpack8<T>(wr[i], wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = inv * (gv[k] * wv[k] - xv[k] * coef);
        dr[i] = pack8<T>(o);
      }
    }
  }
  // every element of this CTA's scratch row that the reduction reads is written here
  float* out = part + (int64_t)blockIdx.x * H;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) out[i * 8 + k] = acc[j][k];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) bwd_reduce_kernel(const float* __restrict__ part,
                                                         T* __restrict__ dw, int parts, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += part[(int64_t)p * H + c];
  dw[c] = from_float<T>(s);
}

template <typename T>
void launch(const void* x, const void* w, const void* dy, const float* inv_rms, void* dx, void* dw,
            float* scratch, int64_t rows, int H, int parts, cudaStream_t s) {
  bwd_partial_kernel<T><<<parts, 256, 0, s>>>((const T*)x, (const T*)w, (const T*)dy, inv_rms, (T*)dx,
                                              scratch, rows, H);
  bwd_reduce_kernel<T><<<(H + 255) / 256, 256, 0, s>>>(scratch, (T*)dw, parts, H);
}

}  // namespace

extern "C" int ft_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy,
                                      const float* inv_rms, void* dx, void* dw, int64_t rows, int H,
                                      int dt, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  if (H > kMaxH) return -3;            // larger than the built-in scratch was sized for
  if (dt != kBF16 && dt != kF16) return -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -4;
  if (g_scratch_addr[dev] == nullptr) {
    // once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_dw_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = p;
  }
  int parts = kParts;
  if (parts > rows) parts = (int)rows;
  if (dt == kBF16)
    launch<__nv_bfloat16>(x, w, dy, inv_rms, dx, dw, g_scratch_addr[dev], rows, H, parts, stream);
  else
    launch<__half>(x, w, dy, inv_rms, dx, dw, g_scratch_addr[dev], rows, H, parts, stream);
  FT_LAUNCHED(2);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}
