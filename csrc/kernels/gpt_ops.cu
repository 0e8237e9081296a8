// Bandwidth-bound ops of a GPT-style block (LayerNorm, biased projections, tanh
// GELU), bf16 / fp16 I/O with fp32 math, plus a register-resident RMSNorm built
// from the same row kernel.
//
//   ft_norm_fwd / ft_norm_bwd      LayerNorm (mean + rstd saved) or RMSNorm (rstd
//                                  saved).  A row is read ONCE: each thread keeps
//                                  its four 128-bit pieces in registers across the
//                                  reductions, so all loads of a row are in flight
//                                  together and nothing is re-read from L2.
//   ft_bias_act_fwd / _bwd         y = act(x + bias), act in {identity, tanh GELU};
//                                  the backward writes dx and the per-CTA column
//                                  sums of dx (the bias gradient) in one pass.
//   ft_parts_reduce                sums the per-CTA partial rows into the parameter
//                                  gradient.
//
// The reference has no model code (its users bring Megatron-style GPT blocks whose
// fused bias-GELU and LayerNorm come from Megatron / Apex); these are the
// counterparts of those fused kernels.  Every pointer that is accessed through
// 128-bit vectors is checked for 16-byte alignment on the host; a launch that would
// be misaligned is refused with -2 instead of faulting.
#include "common.cuh"

namespace {

using namespace ft;

constexpr int kNV = 4;             // 128-bit pieces of a row per thread

__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch /* 64 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) { scratch[warp] = a; scratch[32 + warp] = b; }
  __syncthreads();
  float ra = lane < nwarps ? scratch[lane] : 0.f;
  float rb = lane < nwarps ? scratch[32 + lane] : 0.f;
  a = warp_sum(ra);
  b = warp_sum(rb);
}

// One CTA per row.  H % 8 == 0 and H <= 8 * kNV * THREADS.
template <typename T, bool LN, int THREADS>
__global__ void __launch_bounds__(THREADS) norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ b, T* __restrict__ y,
                                                           float* __restrict__ mean_out,
                                                           float* __restrict__ rstd_out, int H, float eps,
                                                           const T* __restrict__ res, T* __restrict__ sum_out) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = H / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  uint4 raw[kNV];
#pragma unroll
  for (int j = 0; j < kNV; ++j) {
    const int i = threadIdx.x + j * THREADS;
    raw[j] = i < nvec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
  }
  if (res != nullptr) {
    // fused residual add: the row that is normalised (and written to sum_out) is x + res,
    // rounded to T first so that the statistics are those of the stored sum
    const uint4* rr = reinterpret_cast<const uint4*>(res + row * H);
    uint4* sr = reinterpret_cast<uint4*>(sum_out + row * H);
    uint4 rraw[kNV];
#pragma unroll
    for (int j = 0; j < kNV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      rraw[j] = i < nvec ? rr[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < kNV; ++j) {
      const int i = threadIdx.x + j * THREADS;
      float a[8], c[8];
      unpack8<T>(raw[j], a);
      unpack8<T>(rraw[j], c);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] += c[k];
      raw[j] = pack8<T>(a);
      if (i < nvec) sr[i] = raw[j];
    }
  }
  float mean = 0.f;
  if constexpr (LN) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kNV; ++j) {
      float v[8];
      unpack8<T>(raw[j], v);                 // pieces past the row hold zeros
#pragma unroll
      for (int k = 0; k < 8; ++k) s += v[k];
    }
    mean = block_sum(s, red) / (float)H;
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNV; ++j) {
    if (threadIdx.x + j * THREADS < nvec) {
      float v[8];
      unpack8<T>(raw[j], v);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += (v[k] - mean) * (v[k] - mean);
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0) {
    if (LN) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int j = 0; j < kNV; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i < nvec) {
      float v[8], g[8], o[8];
      unpack8<T>(raw[j], v);
      unpack8<T>(wr[i], g);
      if constexpr (LN) {
        float bb[8];
        unpack8<T>(br[i], bb);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (v[k] - mean) * rstd * g[k] + bb[k];
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = v[k] * rstd * g[k];
      }
      yr[i] = pack8<T>(o);
    }
  }
}

// Sums N values over the CTA with one pair of barriers; `scratch` holds N * 32 floats.
template <int N>
__device__ __forceinline__ void block_sum_n(float (&v)[N], float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int n = 0; n < N; ++n) v[n] = warp_sum(v[n]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int n = 0; n < N; ++n) scratch[n * 32 + warp] = v[n];
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < N; ++n) v[n] = warp_sum(lane < nwarps ? scratch[n * 32 + lane] : 0.f);
}

// Backward.  One CTA per SM; a CTA takes R rows per step and each thread NV 128-bit
// column pieces of them (NV * blockDim.x * 8 >= H), so a step has 2 * R * NV 128-bit
// loads per thread in flight at once (the bandwidth of this kernel is set by how many
// bytes an SM keeps in flight, and the weight-gradient accumulators, which scale with
// the pieces but not with R, are what limits the register budget).  The 2 * R row sums
// of a step share one CTA-wide reduction.  Every CTA leaves one partial row of dw (and db).
//   xh = (x - mean) * rstd, gw = dy * w
//   dx = rstd * (gw - mean(gw) - xh * mean(gw * xh))       (mean(gw) term: LayerNorm only)
template <typename T, bool LN, int NV, int R, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ dy,
                                                           const float* __restrict__ mean_in,
                                                           const float* __restrict__ rstd_in,
                                                           T* __restrict__ dx, float* __restrict__ dw_part,
                                                           float* __restrict__ db_part, int64_t rows, int H,
                                                           const T* __restrict__ dres) {
  __shared__ float red[2 * R * 32];
  const int nvec = H / 8;
  const int nthr = blockDim.x;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 wraw[NV];
  float dw_acc[NV][8];
  float db_acc[LN ? NV : 1][8];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * nthr;
    wraw[j] = i < nvec ? wr[i] : zero;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      dw_acc[j][k] = 0.f;
      if constexpr (LN) db_acc[j][k] = 0.f;
    }
  }
  const float inv_h = 1.f / (float)H;
  const int64_t groups = (rows + R - 1) / R;
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
    uint4 xraw[R][NV], graw[R][NV];
    float mean[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = g * R + r;
      const bool ok = row < rows;
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
      const uint4* gr = reinterpret_cast<const uint4*>(dy + row * H);
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int i = threadIdx.x + j * nthr;
        const bool p = ok && i < nvec;
        xraw[r][j] = p ? xr[i] : zero;
        graw[r][j] = p ? gr[i] : zero;
      }
      // a row past the end reads as zeros with rstd 0: it adds nothing anywhere
      mean[r] = (LN && ok) ? mean_in[row] : 0.f;
      rstd[r] = ok ? rstd_in[row] : 0.f;
    }
    float s[2 * R];
#pragma unroll
    for (int n = 0; n < 2 * R; ++n) s[n] = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        float xv[8], gv[8], wv[8];
        unpack8<T>(xraw[r][j], xv);
        unpack8<T>(graw[r][j], gv);
        unpack8<T>(wraw[j], wv);                     // zeros past the row's end
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (xv[k] - mean[r]) * rstd[r];
          const float gw = gv[k] * wv[k];
          s[2 * r] += gw;
          s[2 * r + 1] += gw * xh;
          dw_acc[j][k] += gv[k] * xh;
          if constexpr (LN) db_acc[j][k] += gv[k];
        }
      }
    }
    block_sum_n<2 * R>(s, red);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = g * R + r;
      if (row < rows) {
        uint4* dr = reinterpret_cast<uint4*>(dx + row * H);
        const float c1 = LN ? s[2 * r] * inv_h : 0.f;
        const float c2 = s[2 * r + 1] * inv_h;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
          const int i = threadIdx.x + j * nthr;
          if (i < nvec) {
            float xv[8], gv[8], wv[8], o[8];
            unpack8<T>(xraw[r][j], xv);
            unpack8<T>(graw[r][j], gv);
            unpack8<T>(wraw[j], wv);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float xh = (xv[k] - mean[r]) * rstd[r];
              o[k] = rstd[r] * (gv[k] * wv[k] - c1 - xh * c2);
            }
            if (dres != nullptr) {
              // the gradient that reaches the normalised tensor along the residual branch
              float e[8];
              unpack8<T>(reinterpret_cast<const uint4*>(dres + row * H)[i], e);
#pragma unroll
              for (int k = 0; k < 8; ++k) o[k] += e[k];
            }
            dr[i] = pack8<T>(o);
          }
        }
      }
    }
  }
  float4* ow = reinterpret_cast<float4*>(dw_part + (int64_t)blockIdx.x * H);
  float4* ob = LN ? reinterpret_cast<float4*>(db_part + (int64_t)blockIdx.x * H) : nullptr;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int i = threadIdx.x + j * nthr;
    if (i < nvec) {
      ow[2 * i] = make_float4(dw_acc[j][0], dw_acc[j][1], dw_acc[j][2], dw_acc[j][3]);
      ow[2 * i + 1] = make_float4(dw_acc[j][4], dw_acc[j][5], dw_acc[j][6], dw_acc[j][7]);
      if constexpr (LN) {
        ob[2 * i] = make_float4(db_acc[j][0], db_acc[j][1], db_acc[j][2], db_acc[j][3]);
        ob[2 * i + 1] = make_float4(db_acc[j][4], db_acc[j][5], db_acc[j][6], db_acc[j][7]);
      }
    }
  }
}

// out[c] (+)= sum_p part[p][c]
template <typename T>
__global__ void __launch_bounds__(256) parts_reduce_kernel(const float* __restrict__ part, T* __restrict__ out,
                                                           int parts, int N, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = accumulate ? to_float(out[c]) : 0.f;
  for (int p = 0; p < parts; ++p) s += part[(int64_t)p * N + c];
  out[c] = from_float<T>(s);
}

// ------------------------------------------------------------ bias + activation
__device__ __forceinline__ float tanh_fast(float z) {
  // 1 - 2 / (1 + e^{2z}); exact limits at +-inf
  return 1.f - __fdividef(2.f, 1.f + __expf(2.f * z));
}

constexpr float kGeluK = 0.7978845608028654f;    // sqrt(2 / pi)
constexpr float kGeluC = 0.044715f;

__device__ __forceinline__ float gelu_tanh(float u) {
  return 0.5f * u * (1.f + tanh_fast(kGeluK * (u + kGeluC * u * u * u)));
}

__device__ __forceinline__ float gelu_tanh_grad(float u) {
  const float t = tanh_fast(kGeluK * (u + kGeluC * u * u * u));
  return 0.5f * (1.f + t) + 0.5f * u * (1.f - t * t) * kGeluK * (1.f + 3.f * kGeluC * u * u);
}

// x, y: [rows, N] with row stride N; y may alias x.  ACT 0: identity, 1: tanh GELU.
template <typename T, int ACT>
__global__ void __launch_bounds__(256) bias_act_fwd_kernel(const T* x, const T* __restrict__ bias, T* y,
                                                           int64_t rows, int N) {
  const int vec = N / 8;
  const int64_t total = rows * vec;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % vec);
    float v[8], bb[8], o[8];
    unpack8<T>(reinterpret_cast<const uint4*>(x)[idx], v);
    unpack8<T>(reinterpret_cast<const uint4*>(bias)[c], bb);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float u = v[k] + bb[k];
      o[k] = ACT == 1 ? gelu_tanh(u) : u;
    }
    reinterpret_cast<uint4*>(y)[idx] = pack8<T>(o);
  }
}

// CTA = 32 column groups (8 columns each) x 8 row lanes; grid (ceil(N / 256), parts).
// dx = dy * act'(x + bias) (not written when dx == nullptr, i.e. identity);
// db_part[blockIdx.y][c] = sum over this CTA's rows of dx[:, c].
template <typename T, int ACT>
__global__ void __launch_bounds__(256) bias_act_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                           const T* __restrict__ bias, T* __restrict__ dx,
                                                           float* __restrict__ db_part, int64_t rows, int N) {
  __shared__ float red[8][257];
  const int vec = N / 8;
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cg;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (c < vec) {
    float bb[8];
    if (ACT == 1) unpack8<T>(reinterpret_cast<const uint4*>(bias)[c], bb);
    for (int64_t r = (int64_t)blockIdx.y * 8 + rl; r < rows; r += (int64_t)gridDim.y * 8) {
      const int64_t idx = r * vec + c;
      float g[8];
      unpack8<T>(reinterpret_cast<const uint4*>(dy)[idx], g);
      if (ACT == 1) {
        float v[8], o[8];
        unpack8<T>(reinterpret_cast<const uint4*>(x)[idx], v);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          o[k] = g[k] * gelu_tanh_grad(v[k] + bb[k]);
          acc[k] += o[k];
        }
        reinterpret_cast<uint4*>(dx)[idx] = pack8<T>(o);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += g[k];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][cg * 8 + k] = acc[k];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) s += red[r][threadIdx.x];
    db_part[(int64_t)blockIdx.y * N + col] = s;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define FT_DISPATCH_16(dt, T, ...)                            \
  if (dt == kBF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else if (dt == kF16) { using T = __half; __VA_ARGS__; }     \
  else return -1;

template <typename T, bool LN>
void launch_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                     int64_t rows, int H, float eps, const void* res, void* sum_out, cudaStream_t s) {
  const int nvec = H / 8;
#define FT_NORM_FWD(THREADS)                                                                           \
  norm_fwd_kernel<T, LN, THREADS><<<(unsigned)rows, THREADS, 0, s>>>(                                 \
      (const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd, H, eps, (const T*)res, (T*)sum_out)
  if (nvec <= kNV * 256) FT_NORM_FWD(256);
  else if (nvec <= kNV * 512) FT_NORM_FWD(512);
  else FT_NORM_FWD(1024);
#undef FT_NORM_FWD
}

inline int round_up32(int v) { return (v + 31) / 32 * 32; }

// Shape of the backward launch for a hidden size: pieces per thread, rows per step, threads.
struct BwdShape { int nv, r, threads; };
inline BwdShape norm_bwd_shape(int H) {
  const int nvec = H / 8;
  if (nvec <= 640) return {1, 4, round_up32(nvec)};
  if (nvec <= 1024) return {2, 2, round_up32((nvec + 1) / 2)};
  return {4, 1, round_up32((nvec + 3) / 4)};
}

template <typename T, bool LN>
void launch_norm_bwd(const void* x, const void* w, const void* dy, const float* mean, const float* rstd,
                     void* dx, float* dw_part, float* db_part, int64_t rows, int H, int parts,
                     const void* dres, cudaStream_t s) {
  const BwdShape sh = norm_bwd_shape(H);
#define FT_NORM_BWD(NV, R, MAXT)                                                                      \
  norm_bwd_kernel<T, LN, NV, R, MAXT><<<parts, sh.threads, 0, s>>>(                                   \
      (const T*)x, (const T*)w, (const T*)dy, mean, rstd, (T*)dx, dw_part, db_part, rows, H, (const T*)dres)
  if (sh.nv == 1 && sh.threads <= 512) FT_NORM_BWD(1, 4, 512);
  else if (sh.nv == 1) FT_NORM_BWD(1, 4, 640);
  else if (sh.nv == 2) FT_NORM_BWD(2, 2, 512);
  else FT_NORM_BWD(4, 1, 512);
#undef FT_NORM_BWD
}

}  // namespace

extern "C" {

// Largest hidden size of ft_norm_fwd / ft_norm_bwd.
int ft_norm_max_hidden(int backward) { return backward ? 8 * 4 * 512 : 8 * kNV * 1024; }

// Number of partial rows ft_norm_bwd writes into dw_part / db_part (one per CTA, one CTA per SM).
int ft_norm_bwd_parts(int64_t rows, int H) {
  const int r = H % 8 == 0 && H > 0 ? norm_bwd_shape(H).r : 1;
  const int64_t groups = (rows + r - 1) / r;
  return groups < 148 ? (int)(groups < 1 ? 1 : groups) : 148;
}

// layernorm != 0: y = (x - mean) * rstd * w + b, mean and rstd saved per row.
// layernorm == 0: y = x * rstd * w (b, mean unused; may be null).
// With `res` (and `sum_out`) the row that is normalised is x + res, which is also written to
// sum_out in the tensors' dtype: the residual add before a norm costs no pass of its own.
int ft_add_norm_fwd(const void* x, const void* res, void* sum_out, const void* w, const void* b, void* y,
                    float* mean, float* rstd, int64_t rows, int H, float eps, int layernorm, int dt,
                    cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8 || H > ft_norm_max_hidden(0)) return -2;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (layernorm && !aligned16(b))) return -2;
  if ((res == nullptr) != (sum_out == nullptr)) return -2;
  if (res && (!aligned16(res) || !aligned16(sum_out))) return -2;
  if (rows > 0x7fffffffLL) return -2;
  FT_DISPATCH_16(dt, T, {
    if (layernorm) launch_norm_fwd<T, true>(x, w, b, y, mean, rstd, rows, H, eps, res, sum_out, s);
    else launch_norm_fwd<T, false>(x, w, nullptr, y, nullptr, rstd, rows, H, eps, res, sum_out, s);
  });
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                int64_t rows, int H, float eps, int layernorm, int dt, cudaStream_t s) {
  return ft_add_norm_fwd(x, nullptr, nullptr, w, b, y, mean, rstd, rows, H, eps, layernorm, dt, s);
}

// dw_part (and db_part for LayerNorm): ft_norm_bwd_parts(rows, H) * H floats of scratch.
// dw / db receive the column sums in the parameters' dtype `dt`.
// With `dres` ([rows, H], same dtype) dx = dres + (gradient through the norm): the sum of the two
// gradient branches that meet at the norm's input is formed here (dx and dres are distinct buffers).
int ft_add_norm_bwd(const void* x, const void* w, const void* dy, const void* dres, const float* mean,
                    const float* rstd, void* dx, void* dw, void* db, float* dw_part, float* db_part,
                    int64_t rows, int H, int layernorm, int dt, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8 || H > ft_norm_max_hidden(1)) return -2;
  if (!aligned16(x) || !aligned16(w) || !aligned16(dy) || !aligned16(dx) || !aligned16(dw_part) ||
      (layernorm && !aligned16(db_part)) || (dres && !aligned16(dres)))
    return -2;
  const int parts = ft_norm_bwd_parts(rows, H);
  FT_DISPATCH_16(dt, T, {
    if (layernorm) launch_norm_bwd<T, true>(x, w, dy, mean, rstd, dx, dw_part, db_part, rows, H, parts, dres, s);
    else launch_norm_bwd<T, false>(x, w, dy, nullptr, rstd, dx, dw_part, nullptr, rows, H, parts, dres, s);
    parts_reduce_kernel<T><<<(H + 255) / 256, 256, 0, s>>>(dw_part, (T*)dw, parts, H, 0);
    if (layernorm) parts_reduce_kernel<T><<<(H + 255) / 256, 256, 0, s>>>(db_part, (T*)db, parts, H, 0);
  });
  FT_LAUNCHED(layernorm ? 3 : 2);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_norm_bwd(const void* x, const void* w, const void* dy, const float* mean, const float* rstd,
                void* dx, void* dw, void* db, float* dw_part, float* db_part, int64_t rows, int H,
                int layernorm, int dt, cudaStream_t s) {
  return ft_add_norm_bwd(x, w, dy, nullptr, mean, rstd, dx, dw, db, dw_part, db_part, rows, H, layernorm,
                         dt, s);
}

// y = act(x + bias) over [rows, N]; y may be x.  act 0: identity, 1: tanh GELU.
int ft_bias_act_fwd(const void* x, const void* bias, void* y, int64_t rows, int N, int act, int dt,
                    cudaStream_t s) {
  if (rows <= 0) return 0;
  if (N % 8 || (act != 0 && act != 1)) return -2;
  if (!aligned16(x) || !aligned16(bias) || !aligned16(y)) return -2;
  const int grid = grid_for(rows * (N / 8), 256);
  FT_DISPATCH_16(dt, T, {
    if (act == 1) bias_act_fwd_kernel<T, 1><<<grid, 256, 0, s>>>((const T*)x, (const T*)bias, (T*)y, rows, N);
    else bias_act_fwd_kernel<T, 0><<<grid, 256, 0, s>>>((const T*)x, (const T*)bias, (T*)y, rows, N);
  });
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// Number of partial rows ft_bias_act_bwd writes for a [rows, N] problem.
int ft_bias_act_bwd_parts(int64_t rows, int N) {
  const int gx = (N + 255) / 256;
  int64_t parts = (148 * 8 + gx - 1) / gx;
  const int64_t by_rows = (rows + 7) / 8;
  if (parts > by_rows) parts = by_rows;
  if (parts > 64) parts = 64;
  if (parts < 1) parts = 1;
  return (int)parts;
}

// dx = dy * act'(x + bias) (act 1; for act 0 dx is dy itself and x, dx are unused),
// dbias (+)= column sums of dx.  db_part: ft_bias_act_bwd_parts(rows, N) * N floats.
int ft_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, void* dbias,
                    float* db_part, int64_t rows, int N, int act, int accumulate, int dt,
                    cudaStream_t s) {
  if (rows <= 0) return 0;
  if (N % 8 || (act != 0 && act != 1)) return -2;
  if (!aligned16(dy)) return -2;
  if (act == 1 && (!aligned16(x) || !aligned16(bias) || !aligned16(dx))) return -2;
  const int parts = ft_bias_act_bwd_parts(rows, N);
  const dim3 grid((N + 255) / 256, parts);
  FT_DISPATCH_16(dt, T, {
    if (act == 1)
      bias_act_bwd_kernel<T, 1><<<grid, 256, 0, s>>>((const T*)dy, (const T*)x, (const T*)bias, (T*)dx,
                                                      db_part, rows, N);
    else
      bias_act_bwd_kernel<T, 0><<<grid, 256, 0, s>>>((const T*)dy, nullptr, nullptr, nullptr, db_part, rows,
                                                      N);
    parts_reduce_kernel<T><<<(N + 255) / 256, 256, 0, s>>>(db_part, (T*)dbias, parts, N, accumulate);
  });
  FT_LAUNCHED(2);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

}  // extern "C"
