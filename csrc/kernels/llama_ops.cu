// Bandwidth-bound model ops of the Llama block, bf16/fp16/fp32 I/O with fp32
// math: RMSNorm (fwd, bwd), rotary embedding (fwd = bwd with the sign of sin
// flipped; strided input or output so it reads / writes slices of the fused QKV
// tensor directly), SwiGLU (fwd, bwd) and the softmax cross-entropy row kernels
// used by the chunked head (row log-sum-exp + loss; in-place dlogits).
//
// The reference has no model code: these replace the ATen kernels a user model
// would call.  One 128-bit access per thread per step; rows are processed by
// one CTA each so every reduction stays on chip.
#include "common.cuh"

namespace {

using namespace ft;

// ----------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w ; inv_rms saved per row.  H % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const T* __restrict__ x,
                                                          const T* __restrict__ w, T* __restrict__ y,
                                                          float* __restrict__ inv_rms, int H, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
  const int nvec = H / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8<T>(xr[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0) inv_rms[row] = inv;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[8], g[8], o[8];
    unpack8<T>(xr[i], v);
    unpack8<T>(wr[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = v[k] * inv * g[k];
    yr[i] = pack8<T>(o);
  }
}

// dx = inv * (g*w - x * inv^2 * mean(g*w*x)); partial dw per CTA (rows strided by grid).
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const T* __restrict__ x,
                                                          const T* __restrict__ w,
                                                          const T* __restrict__ dy,
                                                          const float* __restrict__ inv_rms,
                                                          T* __restrict__ dx, float* __restrict__ dw_part,
                                                          int64_t rows, int H) {
  __shared__ float red[32];
  const int nvec = H / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  constexpr int kMaxVec = 8;   // per-thread column groups kept in registers: H <= 8 * 8 * 256
  float dw_acc[kMaxVec][8];
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) dw_acc[j][k] = 0.f;

  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
    uint4* dr = reinterpret_cast<uint4*>(dx + row * H);
    const float inv = inv_rms[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      int i = threadIdx.x + j * blockDim.x;
      if (i < nvec) {
        float xv[8], gv[8], wv[8];
        unpack8<T>(xr[i], xv);
        unpack8<T>(gr[i], gv);
        unpack8<T>(wr[i], wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot += gv[k] * wv[k] * xv[k];
          dw_acc[j][k] += gv[k] * xv[k] * inv;
        }
      }
    }
    dot = block_sum(dot, red);
    const float coef = dot * inv * inv / (float)H;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      int i = threadIdx.x + j * blockDim.x;
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
  float* out = dw_part + (int64_t)blockIdx.x * H;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) out[i * 8 + k] = dw_acc[j][k];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_dw_reduce_kernel(const float* __restrict__ part,
                                                                T* __restrict__ dw, int parts, int H) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += part[(int64_t)p * H + c];
  dw[c] = from_float<T>(s);
}

// -------------------------------------------------------------------- RoPE
// x viewed as [tokens, heads, D] with token strides in elements; rotate-half
// pairs (i, i + D/2); position = token % seq_len.  sin_sign = -1 gives the
// transpose rotation (backward).  One thread per (token, 8 columns of the first half): it
// loads its 8 cosines and sines once and walks the heads, four at a time, so the tables are
// read once per token instead of once per head and eight 16-byte loads are in flight per thread.
template <typename T>
__device__ __forceinline__ void rope_rotate8(const uint4& xa, const uint4& xb, const float (&c)[8],
                                             const float (&s)[8], uint4& ya, uint4& yb) {
  float a[8], b[8], oa[8], ob[8];
  unpack8<T>(xa, a);
  unpack8<T>(xb, b);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    oa[k] = a[k] * c[k] - b[k] * s[k];
    ob[k] = b[k] * c[k] + a[k] * s[k];
  }
  ya = pack8<T>(oa);
  yb = pack8<T>(ob);
}

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, int64_t x_tok_stride,
                                                   T* __restrict__ y, int64_t y_tok_stride,
                                                   const float* __restrict__ cos_t,
                                                   const float* __restrict__ sin_t, int64_t tokens,
                                                   int heads, int D, int seq_len, float sin_sign) {
  const int half = D / 2, vec = half / 8;
  const int64_t total = tokens * vec;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec);
    const int64_t tok = idx / vec;
    const int pos = (int)(tok % seq_len);
    float c[8], s[8];
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (int64_t)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (int64_t)pos * half + v * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
#pragma unroll
    for (int k = 0; k < 8; ++k) s[k] *= sin_sign;
    const T* xp = x + tok * x_tok_stride + v * 8;
    T* yp = y + tok * y_tok_stride + v * 8;
    int h = 0;
    for (; h + 4 <= heads; h += 4) {
      uint4 xa[4], xb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {                  // all loads before any store: x may be y
        xa[u] = *reinterpret_cast<const uint4*>(xp + (int64_t)(h + u) * D);
        xb[u] = *reinterpret_cast<const uint4*>(xp + (int64_t)(h + u) * D + half);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 ya, yb;
        rope_rotate8<T>(xa[u], xb[u], c, s, ya, yb);
        *reinterpret_cast<uint4*>(yp + (int64_t)(h + u) * D) = ya;
        *reinterpret_cast<uint4*>(yp + (int64_t)(h + u) * D + half) = yb;
      }
    }
    for (; h < heads; ++h) {
      const uint4 xa = *reinterpret_cast<const uint4*>(xp + (int64_t)h * D);
      const uint4 xb = *reinterpret_cast<const uint4*>(xp + (int64_t)h * D + half);
      uint4 ya, yb;
      rope_rotate8<T>(xa, xb, c, s, ya, yb);
      *reinterpret_cast<uint4*>(yp + (int64_t)h * D) = ya;
      *reinterpret_cast<uint4*>(yp + (int64_t)h * D + half) = yb;
    }
  }
}

// ------------------------------------------------------------------ SwiGLU
// in: [rows, 2F] = [gate | up]; out: [rows, F].
template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out,
                                                         int64_t rows, int F) {
  const int vec = F / 8;
  const int64_t total = rows * vec;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vec;
    const int c = (int)(idx % vec) * 8;
    float g[8], u[8], o[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(gu + r * 2 * F + c), g);
    unpack8<T>(*reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = __fdividef(g[k], 1.f + __expf(-g[k])) * u[k];
    *reinterpret_cast<uint4*>(out + r * F + c) = pack8<T>(o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ gu,
                                                         const T* __restrict__ dout,
                                                         T* __restrict__ dgu, int64_t rows, int F) {
  const int vec = F / 8;
  const int64_t total = rows * vec;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vec;
    const int c = (int)(idx % vec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(gu + r * 2 * F + c), g);
    unpack8<T>(*reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c), u);
    unpack8<T>(*reinterpret_cast<const uint4*>(dout + r * F + c), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float sig = __fdividef(1.f, 1.f + __expf(-g[k]));   // approximate reciprocal: the result is rounded to 16 bits
      float silu = g[k] * sig;
      dg[k] = d[k] * u[k] * sig * (1.f + g[k] * (1.f - sig));
      du[k] = d[k] * silu;
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + c) = pack8<T>(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + F + c) = pack8<T>(du);
  }
}

// ----------------------------------------------------- softmax cross-entropy
// One CTA per row of logits [rows, V] (row stride ld).  Forward: lse[row] and the
// row's loss (0 for ignored labels) accumulated into *loss_sum.  Backward (in
// place): logits <- (softmax - onehot) * (*grad_scale_ptr) * inv_count, rows with
// an ignored label become 0.
template <typename T>
__device__ __forceinline__ void row_max_sum(const T* row, int V, float* red, float& mx, float& sum) {
  const int nvec = V / 8;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8<T>(reinterpret_cast<const uint4*>(row)[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) m = fmaxf(m, v[k]);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, to_float(row[i]));
  m = block_max(m, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8<T>(reinterpret_cast<const uint4*>(row)[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += __expf(v[k] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) s += __expf(to_float(row[i]) - m);
  s = block_sum(s, red);
  mx = m;
  sum = s;
}

template <typename T>
__global__ void __launch_bounds__(512) xent_fwd_kernel(const T* __restrict__ logits, int64_t ld,
                                                       const int64_t* __restrict__ labels, int V,
                                                       int64_t ignore_index, float* __restrict__ lse,
                                                       float* __restrict__ loss_sum) {
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  const T* row = logits + r * ld;
  float mx, sum;
  row_max_sum<T>(row, V, red, mx, sum);
  if (threadIdx.x == 0) {
    float l = mx + logf(sum);
    lse[r] = l;
    int64_t lab = labels[r];
    if (lab != ignore_index && lab >= 0 && lab < V) atomicAdd(loss_sum, l - to_float(row[lab]));
  }
}

template <typename T>
__global__ void __launch_bounds__(512) xent_bwd_kernel(T* __restrict__ logits, int64_t ld,
                                                       const int64_t* __restrict__ labels, int V,
                                                       int64_t ignore_index,
                                                       const float* __restrict__ lse,
                                                       const float* __restrict__ grad_out,
                                                       float inv_count) {
  const int64_t r = blockIdx.x;
  T* row = logits + r * ld;
  const int64_t lab = labels[r];
  const bool valid = lab != ignore_index && lab >= 0 && lab < V;
  const float scale = valid ? (*grad_out) * inv_count : 0.f;
  const float l = lse[r];
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float v[8], o[8];
    unpack8<T>(reinterpret_cast<uint4*>(row)[i], v);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(v[k] - l);
      o[k] = (p - ((int64_t)(i * 8 + k) == lab ? 1.f : 0.f)) * scale;
    }
    reinterpret_cast<uint4*>(row)[i] = pack8<T>(o);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float p = __expf(to_float(row[i]) - l);
    row[i] = from_float<T>((p - ((int64_t)i == lab ? 1.f : 0.f)) * scale);
  }
}

__global__ void count_valid_kernel(const int64_t* __restrict__ labels, int64_t n, int64_t ignore_index,
                                   int V, int* __restrict__ count) {
  int local = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t lab = labels[i];
    local += (lab != ignore_index && lab >= 0 && lab < V) ? 1 : 0;
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0 && local) atomicAdd(count, local);
}

#define FT_DISPATCH_16(dt, T, ...)                            \
  if (dt == kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if (dt == kF16) { using T = __half; __VA_ARGS__; }     \
  else return -1;

}  // namespace

extern "C" {

int ft_rmsnorm_fwd(const void* x, const void* w, void* y, float* inv_rms, int64_t rows, int H,
                   float eps, int dt, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8) return -2;
  FT_DISPATCH_16(dt, T, (rmsnorm_fwd_kernel<T><<<(unsigned)rows, 256, 0, s>>>(
                            (const T*)x, (const T*)w, (T*)y, inv_rms, H, eps)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// dw_part: scratch of parts * H floats; parts returned by ft_rmsnorm_bwd_parts().
int ft_rmsnorm_bwd_parts() { return 148 * 2; }

int ft_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* inv_rms, void* dx,
                   void* dw, float* dw_part, int64_t rows, int H, int dt, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8 || H > 8 * 8 * 256) return -2;
  int parts = ft_rmsnorm_bwd_parts();
  if (parts > rows) parts = (int)rows;
  FT_DISPATCH_16(dt, T, {
    rmsnorm_bwd_kernel<T><<<parts, 256, 0, s>>>((const T*)x, (const T*)w, (const T*)dy, inv_rms, (T*)dx,
                                                 dw_part, rows, H);
    rmsnorm_dw_reduce_kernel<T><<<(H + 255) / 256, 256, 0, s>>>(dw_part, (T*)dw, parts, H);
  });
  FT_LAUNCHED(1);
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_rope(const void* x, int64_t x_tok_stride, void* y, int64_t y_tok_stride, const float* cos_t,
            const float* sin_t, int64_t tokens, int heads, int D, int seq_len, float sin_sign, int dt,
            cudaStream_t s) {
  if (tokens <= 0) return 0;
  if (D % 16 || x_tok_stride % 8 || y_tok_stride % 8) return -2;
  int64_t total = tokens * (D / 16);
  FT_DISPATCH_16(dt, T, (rope_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(
                            (const T*)x, x_tok_stride, (T*)y, y_tok_stride, cos_t, sin_t, tokens, heads,
                            D, seq_len, sin_sign)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_swiglu_fwd(const void* gu, void* out, int64_t rows, int F, int dt, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  FT_DISPATCH_16(dt, T, (swiglu_fwd_kernel<T><<<grid_for(rows * (F / 8), 256), 256, 0, s>>>(
                            (const T*)gu, (T*)out, rows, F)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_swiglu_bwd(const void* gu, const void* dout, void* dgu, int64_t rows, int F, int dt,
                  cudaStream_t s) {
  if (rows <= 0) return 0;
  if (F % 8) return -2;
  FT_DISPATCH_16(dt, T, (swiglu_bwd_kernel<T><<<grid_for(rows * (F / 8), 256), 256, 0, s>>>(
                            (const T*)gu, (const T*)dout, (T*)dgu, rows, F)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_xent_fwd(const void* logits, int64_t ld, const int64_t* labels, int64_t rows, int V,
                int64_t ignore_index, float* lse, float* loss_sum, int dt, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (ld % 8) return -2;
  FT_DISPATCH_16(dt, T, (xent_fwd_kernel<T><<<(unsigned)rows, 512, 0, s>>>(
                            (const T*)logits, ld, labels, V, ignore_index, lse, loss_sum)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_xent_bwd(void* logits, int64_t ld, const int64_t* labels, int64_t rows, int V,
                int64_t ignore_index, const float* lse, const float* grad_out, float inv_count, int dt,
                cudaStream_t s) {
  if (rows <= 0) return 0;
  if (ld % 8) return -2;
  FT_DISPATCH_16(dt, T, (xent_bwd_kernel<T><<<(unsigned)rows, 512, 0, s>>>(
                            (T*)logits, ld, labels, V, ignore_index, lse, grad_out, inv_count)));
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_count_valid(const int64_t* labels, int64_t n, int64_t ignore_index, int V, int* count,
                   cudaStream_t s) {
  if (n <= 0) return 0;
  count_valid_kernel<<<grid_for(n, 256, 148), 256, 0, s>>>(labels, n, ignore_index, V, count);
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

}  // extern "C"
