// Shared device helpers for the sm_100a kernels: dtype codes that match the
// Python side, packed bf16/fp16 conversion and 128-bit vector access.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ft {

enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2, kNone = -1 };

__host__ __device__ inline int dtype_size(int dt) { return dt == kF32 ? 4 : 2; }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float load_as_float(const void* p, int dt, int64_t i) {
  if (dt == kF32) return ((const float*)p)[i];
  if (dt == kBF16) return __bfloat162float(((const __nv_bfloat16*)p)[i]);
  return __half2float(((const __half*)p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int dt, int64_t i, float v) {
  if (dt == kF32) ((float*)p)[i] = v;
  else if (dt == kBF16) ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
  else if (dt == kF16) ((__half*)p)[i] = __float2half_rn(v);
}

// 8 x 16-bit values <-> 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_float(h[i]);
}

template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&in)[8]) {
  uint4 raw;
  T* h = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = from_float<T>(in[i]);
  return raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

inline int grid_for(int64_t work_items, int block, int max_blocks = 148 * 16) {
  int64_t b = (work_items + block - 1) / block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return (int)b;
}

}  // namespace ft

// Number of kernels this library has launched in the process (all devices).
extern "C" long long ft_launch_count();
extern "C" void ft_note_launches(int n);
#define FT_LAUNCHED(n) ft_note_launches(n)

#define FT_CUDA_RETURN_IF_ERROR()                \
  do {                                           \
    cudaError_t e__ = cudaGetLastError();        \
    if (e__ != cudaSuccess) return (int)e__;     \
  } while (0)
