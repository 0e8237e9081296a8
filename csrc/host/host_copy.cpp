// Host-side staging helpers.
//
//   ft_host_memcpy      multi-threaded DRAM -> DRAM copy with non-temporal stores
//                       (AVX-512 when the CPU has it, AVX2 otherwise).  Used for
//                       staging between pinned pools where the destination is
//                       not read again by the CPU soon, so it should not evict
//                       the optimizer's working set from the caches.
//   ft_locked_alloc /   page-aligned, mlock'ed host buffers with a registry, for
//   ft_locked_free  /   processes that have no CUDA context (the CUDA library has
//   ft_locked_is_managed  the cudaHostAlloc-based pool for those that do).
//
// Counterparts in the reference: ops/csrc/aio/py_lib/deepspeed_py_copy.cpp:25-135
// (an 8/4/1-way unrolled float copy) and deepspeed_pin_tensor.cpp:23-61
// (posix_memalign + mlock behind at::from_blob).  Everything returns status codes.
#include <immintrin.h>
#include "omp_compat.h"
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr size_t kBlock = 1u << 20;   // work item of one thread

__attribute__((target("avx512f"))) void stream_copy_512(uint8_t* d, const uint8_t* s, size_t n) {
  size_t i = 0;
  for (; i + 256 <= n; i += 256) {
    __m512i a = _mm512_loadu_si512(s + i), b = _mm512_loadu_si512(s + i + 64);
    __m512i c = _mm512_loadu_si512(s + i + 128), e = _mm512_loadu_si512(s + i + 192);
    _mm512_stream_si512(reinterpret_cast<__m512i*>(d + i), a);
    _mm512_stream_si512(reinterpret_cast<__m512i*>(d + i + 64), b);
    _mm512_stream_si512(reinterpret_cast<__m512i*>(d + i + 128), c);
    _mm512_stream_si512(reinterpret_cast<__m512i*>(d + i + 192), e);
  }
  for (; i + 64 <= n; i += 64)
    _mm512_stream_si512(reinterpret_cast<__m512i*>(d + i), _mm512_loadu_si512(s + i));
  if (i < n) memcpy(d + i, s + i, n - i);
}

void stream_copy_256(uint8_t* d, const uint8_t* s, size_t n) {
  size_t i = 0;
  for (; i + 128 <= n; i += 128) {
    __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(s + i));
    __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(s + i + 32));
    __m256i c = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(s + i + 64));
    __m256i e = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(s + i + 96));
    _mm256_stream_si256(reinterpret_cast<__m256i*>(d + i), a);
    _mm256_stream_si256(reinterpret_cast<__m256i*>(d + i + 32), b);
    _mm256_stream_si256(reinterpret_cast<__m256i*>(d + i + 64), c);
    _mm256_stream_si256(reinterpret_cast<__m256i*>(d + i + 96), e);
  }
  if (i < n) memcpy(d + i, s + i, n - i);
}

// One block: bring the destination to a 64-byte boundary with a plain copy, then
// stream (non-temporal stores need an aligned destination).
void copy_block(uint8_t* d, const uint8_t* s, size_t n, bool avx512) {
  const size_t mis = reinterpret_cast<uintptr_t>(d) & 63;
  if (mis) {
    size_t head = 64 - mis;
    if (head > n) head = n;
    memcpy(d, s, head);
    d += head; s += head; n -= head;
  }
  if (n == 0) return;
  if (avx512) stream_copy_512(d, s, n);
  else stream_copy_256(d, s, n);
}

std::mutex g_mu;
std::unordered_map<void*, size_t> g_locked;   // address -> bytes

}  // namespace

extern "C" {

// Copies `nbytes` from `src` to `dst` (no overlap) with up to `threads` OpenMP
// threads (0: the OpenMP default).  Returns 0, or -1 on bad arguments.
int ft_host_memcpy(void* dst, const void* src, size_t nbytes, int threads) {
  if ((!dst || !src) && nbytes) return -1;
  if (nbytes == 0 || dst == src) return 0;
  uint8_t* d = static_cast<uint8_t*>(dst);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  if ((d < s + nbytes) && (s < d + nbytes)) return -1;   // overlapping ranges
  const bool avx512 = __builtin_cpu_supports("avx512f");
  const long blocks = (long)((nbytes + kBlock - 1) / kBlock);
  int nt = threads > 0 ? threads : omp_get_max_threads();
  if (nt > blocks) nt = (int)blocks;
  if (nt < 1) nt = 1;
#pragma omp parallel for schedule(static) num_threads(nt)
  for (long b = 0; b < blocks; ++b) {
    const size_t off = (size_t)b * kBlock;
    const size_t n = off + kBlock <= nbytes ? kBlock : nbytes - off;
    copy_block(d + off, s + off, n, avx512);
  }
  _mm_sfence();
  return 0;
}

// Page-aligned allocation of `nbytes`, mlock'ed when the process's limit allows.
// `*locked` (optional) reports whether mlock succeeded.  nullptr on failure.
void* ft_locked_alloc(size_t nbytes, int* locked) {
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  const size_t size = ((nbytes ? nbytes : 1) + page - 1) / page * page;
  void* p = nullptr;
  if (posix_memalign(&p, page, size) != 0) return nullptr;
  const int ok = mlock(p, size) == 0;
  if (locked) *locked = ok;
  std::lock_guard<std::mutex> g(g_mu);
  g_locked[p] = ok ? size : 0;
  return p;
}

int ft_locked_is_managed(const void* p) {
  std::lock_guard<std::mutex> g(g_mu);
  return g_locked.count(const_cast<void*>(p)) ? 1 : 0;
}

// 0 on success, -1 when `p` did not come from ft_locked_alloc.
int ft_locked_free(void* p) {
  size_t size = 0;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_locked.find(p);
    if (it == g_locked.end()) return -1;
    size = it->second;
    g_locked.erase(it);
  }
  if (size) munlock(p, size);
  free(p);
  return 0;
}

}  // extern "C"
