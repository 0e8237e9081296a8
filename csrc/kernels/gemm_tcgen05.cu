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

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace ft;
using namespace ft::sm100;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

enum OutMode : int { kStore16 = 0, kStore32 = 1, kAcc16 = 2, kAcc32 = 3 };

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort;
};

__device__ __forceinline__ void tile_coords(int t, int mt, int nt, int& mb, int& nb) {
  const int group_size = GROUP_M * nt;
  const int group = t / group_size;
  const int first_m = group * GROUP_M;
  const int gm = min(mt - first_m, GROUP_M);
  const int in_group = t - group * group_size;
  mb = first_m + in_group % gm;
  nb = in_group / gm;
}

template <typename T, int MODE>
__device__ __forceinline__ void store_chunk(const uint32_t (&acc)[32], void* C, int64_t ldc, int row,
                                            int col0, int M, int N) {
  if (row >= M) return;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
  if constexpr (MODE == kStore32 || MODE == kAcc32) {
    float* p = reinterpret_cast<float*>(C) + (int64_t)row * ldc + col0;
    if (col0 + 32 <= N && (ldc % 4 == 0)) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if constexpr (MODE == kAcc32) {
          float4 old = reinterpret_cast<float4*>(p)[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(p)[q] = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j) p[j] = (MODE == kAcc32 ? p[j] : 0.f) + v[j];
    }
  } else {
    T* p = reinterpret_cast<T*>(C) + (int64_t)row * ldc + col0;
    if (col0 + 32 <= N && (ldc % 8 == 0)) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[8 * q + j];
        if constexpr (MODE == kAcc16) {
          float old[8];
          unpack8<T>(reinterpret_cast<uint4*>(p)[q], old);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += old[j];
        }
        reinterpret_cast<uint4*>(p)[q] = pack8<T>(o);
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; ++j)
        p[j] = from_float<T>((MODE == kAcc16 ? to_float(p[j]) : 0.f) + v[j]);
    }
  }
}

template <typename T, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            void* __restrict__ C, int64_t ldc, int M, int N, int K, int* __restrict__ err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (M + BM - 1) / BM, nt = (N + BN - 1) / BN, kt = (K + BK - 1) / BK;
  const int num_tiles = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 4);
    }
    bars->abort = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile uint32_t* abort_flag = &bars->abort;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, mt, nt, mb, nb);
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 1);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tmap_a, &bars->full[stage], mb * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tmap_a, &bars->full[stage], kb * BK, mb * BM);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tmap_b, &bars->full[stage], nb * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, &bars->full[stage], kb * BK, nb * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc =
          make_idesc_f16(sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0, A_MN ? 1 : 0,
                         B_MN ? 1 : 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicCAS(err, 0, 2);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < kt; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase)) {
            *abort_flag = 1;
            atomicCAS(err, 0, 3);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sa + k * (UK * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * (UK * 128), 64 * BK * 2, 1024)
                                     : make_smem_desc(sb + k * (UK * 2), 16, 1024);
            umma_f16(tmem_d, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&bars->empty[stage]);          // frees the stage once the MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        umma_commit(&bars->tmem_full[acc]);          // accumulator complete
      }
    }
  } else {
    // ---------------------------------------------------------- epilogue
    const int quarter = warp & 3;                    // TMEM lane quarter this warp may read
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(t, mt, nt, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase)) {
        *abort_flag = 1;
        atomicCAS(err, 0, 4);
        break;
      }
      tc_fence_after();
      const int row = mb * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = nb * BN + c * 32;
        if (col0 >= N) break;                        // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_chunk<T, MODE>(r, C, ldc, row, col0, M, N);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

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

// 2-D row-major tensor [outer, inner] with row stride ld (elements), 128B swizzle.
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
  if (((uintptr_t)ptr & 15) || ((ld * 2) & 15)) return -101;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
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

int* g_err_word[16] = {nullptr};
int g_sm_count[16] = {0};

int* error_word(int dev) {
  if (!g_err_word[dev]) {
    cudaMalloc(&g_err_word[dev], sizeof(int));
    cudaMemset(g_err_word[dev], 0, sizeof(int));
    cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  }
  return g_err_word[dev];
}

template <typename T, bool A_MN, bool B_MN>
int launch_mode(int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C, int64_t ldc, int M, int N,
                int K, int* err, int grid, cudaStream_t s) {
#define FT_LAUNCH(MODE)                                                                              \
  {                                                                                                  \
    auto kern = gemm_kernel<T, A_MN, B_MN, MODE>;                                                    \
    static bool configured = false;                                                                  \
    if (!configured) {                                                                               \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);           \
      configured = true;                                                                             \
    }                                                                                                \
    kern<<<grid, NUM_THREADS, SMEM_BYTES, s>>>(ta, tb, C, ldc, M, N, K, err);                        \
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

template <typename T>
int launch_layout(int a_mn, int b_mn, int mode, const CUtensorMap& ta, const CUtensorMap& tb, void* C,
                  int64_t ldc, int M, int N, int K, int* err, int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_mode<T, false, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s);
  if (!a_mn && b_mn) return launch_mode<T, false, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s);
  if (a_mn && b_mn) return launch_mode<T, true, true>(mode, ta, tb, C, ldc, M, N, K, err, grid, s);
  return launch_mode<T, true, false>(mode, ta, tb, C, ldc, M, N, K, err, grid, s);
}

}  // namespace

extern "C" {

// C[M,N] (=|+=) A x B^T-like product with fp32 accumulation.
//   A: K-major -> stored [M,K] (row stride lda); MN-major (a_mn=1) -> stored [K,M].
//   B: K-major -> stored [N,K] (row stride ldb); MN-major (b_mn=1) -> stored [K,N].
//   C: [M,N], row stride ldc, dtype c_dtype (same 16-bit type as A/B, or fp32);
//      accumulate != 0 adds into C.
// Returns 0, a negative argument error, or a positive CUDA error code.
int ft_gemm(const void* A, int a_mn, int64_t lda, const void* B, int b_mn, int64_t ldb, void* C,
            int64_t ldc, int c_dtype, int accumulate, int M, int N, int K, int ab_dtype,
            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (ab_dtype != kBF16 && ab_dtype != kF16) return -1;
  if (c_dtype != kF32 && c_dtype != ab_dtype) return -2;
  int dev = 0;
  cudaGetDevice(&dev);
  int* err = error_word(dev);
  CUtensorMap ta, tb;
  int rc;
  if (a_mn) rc = make_tmap(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BK, ab_dtype);
  else rc = make_tmap(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, BM, ab_dtype);
  if (rc) return rc;
  if (b_mn) rc = make_tmap(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BK, ab_dtype);
  else rc = make_tmap(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, BN, ab_dtype);
  if (rc) return rc;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_sm_count[dev] ? tiles : g_sm_count[dev];
  const int mode = c_dtype == kF32 ? (accumulate ? kAcc32 : kStore32) : (accumulate ? kAcc16 : kStore16);
  if (ab_dtype == kBF16)
    rc = launch_layout<__nv_bfloat16>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream);
  else
    rc = launch_layout<__half>(a_mn, b_mn, mode, ta, tb, C, ldc, M, N, K, err, grid, stream);
  if (rc) return rc;
  FT_LAUNCHED(1);
  FT_CUDA_RETURN_IF_ERROR();
  return 0;
}

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
