// bf16 / fp16 GEMM on the 5th-generation tensor cores (sm_100a):
//   C[M,N] (=|+=) sum_k A(m,k) * B(n,k),  fp32 accumulation in tensor memory.
//
// Persistent, warp-specialised CTAs, one per SM:
//   warp 0      TMA producer: 128B-swizzled operand tiles into a 4-stage
//               shared-memory ring (cp.async.bulk.tensor, no cluster multicast)
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 and
//               tcgen05.commit; also owns tensor-memory allocation
//   warps 2-5   epilogue: tcgen05.ld of the 128x256 fp32 accumulator, convert,
//               store (or read-modify-write when accumulating into C)
// Two accumulator buffers (2 x 256 TMEM columns) let the epilogue of tile i
// overlap the main loop of tile i+1.  Tiles are walked in groups of 16 M-blocks
// so one wave of 148 CTAs shares operand tiles through L2.
//
// Operand layouts: an operand is "K-major" when the reduction index is the
// contiguous one in global memory and "MN-major" otherwise.  The three Linear
// GEMMs map to: forward (A K-major, B K-major), input gradient (A K-major,
// B MN-major), weight gradient (A MN-major, B MN-major) - no transposes are
// ever materialised.
//
// Replaces the cuBLAS calls a PyTorch model issues through F.linear on the
// reference's path.  Every mbarrier wait is bounded; on expiry the kernel
// records a code in a device error word, releases its tensor memory and returns.
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "gemm2_kernel.cuh"
#include "gemm2_swiglu.cuh"
#include "gemm_host.h"

namespace {

using namespace ft;
using namespace ft::gemm;

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t inner, outer, ld;
  uint32_t box_inner, box_outer;
  int dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld &&
           box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    auto mix = [&](uint64_t v) { h ^= std::hash<uint64_t>()(v) + 0x9e3779b97f4a7c15ULL + (h << 6) + (h >> 2); };
    mix(k.inner); mix(k.outer); mix(k.ld); mix(k.box_inner); mix(k.box_outer); mix((uint64_t)k.dtype);
    return h;
  }
};

std::mutex g_map_mu;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;

}  // namespace

namespace ft {
namespace gemm {

// 2-D row-major tensor [outer, inner] with row stride ld (elements), 128B swizzle.
// dtype: kBF16 / kF16 (2-byte elements) or kF32.
int make_tmap(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
              uint32_t box_inner, uint32_t box_outer, int dtype) {
  MapKey key{ptr, inner, outer, ld, box_inner, box_outer, dtype};
  {
    std::lock_guard<std::mutex> lk(g_map_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -100;
  {
    // The driver entry point needs the primary context current in THIS thread; a
    // thread that has only used the runtime lazily (e.g. autograd's backward
    // thread) may not have bound it yet.
    int dev = 0;
    cudaGetDevice(&dev);
    cudaSetDevice(dev);
    cudaFree(nullptr);
  }
  const uint64_t esize = dtype == kF32 ? 4 : 2;
  if (((uintptr_t)ptr & 15) || ((ld * esize) & 15)) return -101;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == kF32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (getenv("FLEXTRAIN_DEBUG")) fprintf(stderr, "cuTensorMapEncodeTiled -> %d ptr=%p inner=%llu outer=%llu ld=%llu box=%u,%u\n", (int)r, ptr, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld, box_inner, box_outer);
    return -102;
  }
  std::lock_guard<std::mutex> lk(g_map_mu);
  if (g_maps.size() > 8192) g_maps.clear();
  g_maps[key] = *out;
  return 0;
}

static int* g_err_word[16] = {nullptr};
static int g_sm_count[16] = {0};

int* error_word(int dev) {
  if (!g_err_word[dev]) {
    cudaMalloc(&g_err_word[dev], sizeof(int));
    cudaMemset(g_err_word[dev], 0, sizeof(int));
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  return g_err_word[dev];
}

int sm_count(int dev) {
  error_word(dev);
  return g_sm_count[dev];
}

}  // namespace gemm
}  // namespace ft

namespace {

static_assert(SMEM_BYTES <= 232448 && P_SMEM_BYTES <= 232448 && P_SMEM_BYTES_GATHER <= 232448,
              "a GEMM kernel outgrew the 227 KB of dynamic shared memory of an SM");

template <typename T, bool A_MN, bool B_MN>
int launch_mode(int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int64_t ldc, int M, int N,
                int K, int* err, int grid, cudaStream_t s, const void* R, int64_t ldr) {
  GatherArgs side{};
  side.add_src = R;
  side.add_ld = ldr;
#define FT_LAUNCH(MODE)                                                                              \
  {                                                                                                  \
    auto kern = gemm_kernel<T, A_MN, B_MN, MODE>;                                                    \
    static bool configured = false;                                                                  \
    if (!configured) {                                                                               \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);           \
      configured = true;                                                                             \
    }                                                                                                \
    kern<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ta, tb, C, ldc, M, N, K, err, side);                  \
  }
  switch (mode) {
    case kStore16: FT_LAUNCH(kStore16); break;
    case kStore32: FT_LAUNCH(kStore32); break;
    case kAcc16: FT_LAUNCH(kAcc16); break;
    case kAcc32: FT_LAUNCH(kAcc32); break;
    default: return -3;
  }
#undef FT_LAUNCH
  return 0;
}

// ---- CTA-pair kernel (cluster of 2)
// Row blocks per group of the CTA-pair kernel's tile walk (FLEXTRAIN_GEMM_GROUP_M, default 16).
int pair_group_m() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FLEXTRAIN_GEMM_GROUP_M");
    v = e ? atoi(e) : GROUP_M;
    if (v < 1) v = GROUP_M;
  }
  return v;
}

template <typename T, bool A_MN, bool B_MN, int MODE>
int launch_pair_one(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int64_t ldc, int M, int N, int K,
                    int* err, int grid, cudaStream_t s, const void* R, int64_t ldr) {
  auto kern = gemm_pair_kernel<T, A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GatherArgs none{};
  none.group_m = pair_group_m();
  none.add_src = R;
  none.add_ld = ldr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, C, ldc, M, N, K, err, none);
  return e == cudaSuccess ? 0 : (int)e;
}

template <typename T, bool A_MN, bool B_MN>
int launch_pair_mode(int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int64_t ldc, int M,
                     int N, int K, int* err, int grid, cudaStream_t s, const void* R, int64_t ldr) {
  switch (mode) {
    case kStore16: return launch_pair_one<T, A_MN, B_MN, kStore16>(ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
    case kStore32: return launch_pair_one<T, A_MN, B_MN, kStore32>(ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
    case kAcc16: return launch_pair_one<T, A_MN, B_MN, kAcc16>(ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
    case kAcc32: return launch_pair_one<T, A_MN, B_MN, kAcc32>(ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
    default: return -3;
  }
}

template <typename T>
int launch_pair(int a_mn, int b_mn, int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C,
                int64_t ldc, int M, int N, int K, int* err, int grid, cudaStream_t s, const void* R,
                int64_t ldr) {
  if (!a_mn && !b_mn) return launch_pair_mode<T, false, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  if (!a_mn && b_mn) return launch_pair_mode<T, false, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  if (a_mn && b_mn) return launch_pair_mode<T, true, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  return launch_pair_mode<T, true, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
}

int g_use_pair = -1;   // -1: read FLEXTRAIN_GEMM_PAIR on first use

template <typename T>
int launch_pair_swiglu(const CUtensorMap& ta, const CUtensorMap& tb, void* act, int64_t ld_act, void* gu,
                       int64_t ld_gu, int M, int F, int K, int* err, int grid, cudaStream_t s) {
  auto kern = gemm_pair_swiglu_kernel<T>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, act, ld_act, gu, ld_gu, M, F, K, err);
  return e == cudaSuccess ? 0 : (int)e;
}

template <typename T>
int launch_layout(int a_mn, int b_mn, int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C,
                  int64_t ldc, int M, int N, int K, int* err, int grid, cudaStream_t s, const void* R,
                  int64_t ldr) {
  if (!a_mn && !b_mn) return launch_mode<T, false, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  if (!a_mn && b_mn) return launch_mode<T, false, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  if (a_mn && b_mn) return launch_mode<T, true, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
  return launch_mode<T, true, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s, R, ldr);
}

}  // namespace

extern "C" {

// C[M,N] (=|+=) A x B^T-like product with fp32 accumulation.
//   A: K-major -> stored [M,K] (row stride lda); MN-major (a_mn=1) -> stored [K,M].
//   B: K-major -> stored [N,K] (row stride ldb); MN-major (b_mn=1) -> stored [K,N].
//   C: [M,N], row stride ldc, dtype c_dtype (same 16-bit type as A/B, or fp32);
//      accumulate != 0 adds into C.
// Returns 0, a negative argument error, or a positive CUDA error code.
// C = A B + R: the accumulating epilogue of ft_gemm with the addend read from a matrix R of C's
// type and shape (row stride ldr) instead of from C.  R = nullptr gives C = A B (accumulate 0) or
// C += A B (accumulate 1).  R may not overlap C unless it is C.
int ft_gemm_add(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
                int64_t ldc, int c_dtype, int accumulate, const void* R, int64_t ldr, int M, int N, int K,
                int ab_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (R != nullptr) accumulate = 1;
  if (ab_dtype != kBF16 && ab_dtype != kF16) return -1;
  if (c_dtype != kF32 && c_dtype != ab_dtype) return -2;
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = error_word(dev);
  CUtensorMap ta, tb;
  int rc;
  if (g_use_pair < 0) {
    const char* e = getenv("FLEXTRAIN_GEMM_PAIR");
    g_use_pair = e ? atoi(e) : 1;
  }
  // The pair kernel's tile is 256 rows tall: below that half of it would be padding.
  const bool pair = g_use_pair != 0 && M > 128;
  const int b_box = pair ? 128 : BN;              // rows of B one CTA stages per k-block
  if (a_mn) rc = make_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK, ab_dtype);
  else rc = make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM, ab_dtype);
  if (rc) return rc;
  if (b_mn) rc = make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK, ab_dtype);
  else rc = make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, b_box, ab_dtype);
  if (rc) return rc;
  const int mode = c_dtype == kF32 ? (accumulate ? kAcc32 : kStore32) : (accumulate ? kAcc16 : kStore16);
  if (pair) {
    const int tiles = ((M + P_BM - 1) / P_BM) * ((N + P_BN - 1) / P_BN);
    const int pairs = sm_count(dev) / 2;
    const int grid = 2 * (tiles < pairs ? tiles : pairs);
    if (ab_dtype == kBF16)
      rc = launch_pair<__nv_bfloat16>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream, R, ldr);
    else
      rc = launch_pair<__half>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream, R, ldr);
  } else {
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sm_count(dev) ? tiles : sm_count(dev);
    if (ab_dtype == kBF16)
      rc = launch_layout<__nv_bfloat16>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream, R, ldr);
    else
      rc = launch_layout<__half>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream, R, ldr);
  }
  if (rc) return rc;
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

int ft_gemm(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
            int64_t ldc, int c_dtype, int accumulate, int M, int N, int K, int ab_dtype,
            cudaStream_t stream) {
  return ft_gemm_add(A, a_mn, lda, B, b_mn, ldb, C, ldc, c_dtype, accumulate, nullptr, 0, M, N, K, ab_dtype,
                     stream);
}

// act[M,F] = silu(X Wg^T) * (X Wu^T) with W = [Wg ; Wu] stored [2F, K] (row stride ldw), X stored
// [M, K] (row stride ldx); gu (optional, [M, 2F], row stride ld_gu) receives the two projections
// as the unfused path would have stored them.  Returns -4 when the shape is not covered (F not a
// multiple of 128, fewer than 129 rows): the caller then runs ft_gemm + the activation kernel.
int ft_gemm_swiglu(const void* X, int64_t ldx, const void* W, int64_t ldw, void* act, int64_t ld_act,
                   void* gu, int64_t ld_gu, int M, int F, int K, int dtype, cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if (dtype != kBF16 && dtype != kF16) return -1;
  if (F % 128 || M <= 128) return -4;
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = error_word(dev);
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, X, (uint64_t)K, (uint64_t)M, (uint64_t)ldx, BK, BM, dtype);
  if (rc) return rc;
  rc = make_tmap(&tb, W, (uint64_t)K, (uint64_t)(2 * F), (uint64_t)ldw, BK, 128, dtype);
  if (rc) return rc;
  const int tiles = ((M + P_BM - 1) / P_BM) * (F / 128);
  const int pairs = sm_count(dev) / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  if (dtype == kBF16)
    rc = launch_pair_swiglu<__nv_bfloat16>(ta, tb, act, ld_act, gu, ld_gu, M, F, K, err, grid, stream);
  else
    rc = launch_pair_swiglu<__half>(ta, tb, act, ld_act, gu, ld_gu, M, F, K, err, grid, stream);
  if (rc) return rc;
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

// Selects the CTA-pair kernel (1) or the single-CTA kernel (0) for later ft_gemm calls.
void ft_gemm_set_pair(int on) { g_use_pair = on ? 1 : 0; }
int ft_gemm_get_pair() { return g_use_pair > 0 ? 1 : 0; }

// Reads (and clears) the device error word: 0 = no bounded wait ever expired.
// Synchronises the device; meant for tests and health checks.
int ft_gemm_error() {
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = error_word(dev);
  int host = 0;
  if (cudaMemcpy(&host, err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (host) cudaMemset(err, 0, sizeof(int));
  return host;
}

}  // extern "C"
