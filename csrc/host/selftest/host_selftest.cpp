// Stand-alone driver of the host library's C ABI (Adam, streaming copy, locked
// allocations, NVMe engine) for sanitizer builds: it is compiled together with
// the library sources under -fsanitize=address,undefined and under
// -fsanitize=thread and must finish with exit code 0 and no sanitizer report.
// The reference ships no such harness (its C++ is compiled with asserts and -g
// only, flextrain/ops/op_builder/cpu_adam.py:31-36, async_io.py:43-60).
//
//   host_selftest <scratch directory>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <string>
#include <thread>
#include <vector>

extern "C" {
int ft_adam_update(int64_t step, float lr, float beta1, float beta2, float eps, float weight_decay, int adamw,
                   int bias_correction, float grad_scale, float* param, const void* grad, int grad_dtype,
                   float* exp_avg, float* exp_avg_sq, int64_t n, void* out_copy, int copy_dtype, int threads,
                   int force_scalar);
int ft_has_nonfinite(const void* grad, int grad_dtype, int64_t n, int threads);
int ft_host_memcpy(void* dst, const void* src, size_t nbytes, int threads);
void* ft_locked_alloc(size_t nbytes, int* locked);
int ft_locked_is_managed(const void* p);
int ft_locked_free(void* p);
void* ft_nvme_create(int64_t block_size, int queue_depth, int threads, int engine_kind, int use_odirect);
void ft_nvme_destroy(void* h);
int64_t ft_nvme_submit(void* h, const char* path, void* buffer, int64_t nbytes, int64_t file_offset,
                       int is_write);
int ft_nvme_wait_op(void* h, int64_t id);
int64_t ft_nvme_wait(void* h);
int ft_nvme_sync_rw(void* h, const char* path, void* buffer, int64_t nbytes, int64_t file_offset, int is_write);
int ft_nvme_forget(void* h, const char* path);
void ft_nvme_inject_fault(void* h, int kind, int count);
int ft_nvme_register_buffers(void* h, void* const* ptrs, const int64_t* lens, int n);
int64_t ft_nvme_fixed_ops(void* h);
}

static int g_failed = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
      ++g_failed;                                                          \
    }                                                                      \
  } while (0)

static void test_adam() {
  const int64_t n = 100003;                       // odd size: vector body and scalar tail
  std::vector<float> p(n), g(n), m(n, 0.f), v(n, 0.f), p2, m2, v2;
  for (int64_t i = 0; i < n; ++i) { p[i] = 0.01f * (float)(i % 97); g[i] = 0.001f * (float)((i * 7) % 31) - 0.01f; }
  p2 = p; m2 = m; v2 = v;
  std::vector<uint16_t> copy(n);
  CHECK(ft_adam_update(1, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, 1, 1.f, p.data(), g.data(), 0, m.data(),
                       v.data(), n, copy.data(), 1, 4, 0) == 0);
  CHECK(ft_adam_update(1, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f, 1, 1, 1.f, p2.data(), g.data(), 0, m2.data(),
                       v2.data(), n, nullptr, 0, 1, 1) == 0);
  double worst = 0;
  for (int64_t i = 0; i < n; ++i) worst = std::fmax(worst, std::fabs((double)p[i] - (double)p2[i]));
  CHECK(worst < 1e-6);
  g[n / 2] = INFINITY;
  CHECK(ft_has_nonfinite(g.data(), 0, n, 3) == 1);
  // concurrent updates of disjoint slices from several caller threads (what the
  // engine's host worker and a user thread may do)
  std::vector<std::thread> th;
  std::atomic<int> bad{0};
  g[n / 2] = 0.f;
  for (int t = 0; t < 4; ++t)
    th.emplace_back([&, t] {
      const int64_t lo = t * (n / 4), len = n / 4;
      if (ft_adam_update(2, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.f, 1, 1, 0.5f, p.data() + lo, g.data() + lo, 0,
                         m.data() + lo, v.data() + lo, len, nullptr, 0, 2, 0) != 0)
        ++bad;
    });
  for (auto& x : th) x.join();
  CHECK(bad == 0);
}

static void test_copy_and_locked() {
  const size_t n = (3u << 20) + 77;
  std::vector<uint8_t> src(n), dst(n + 64, 0);
  for (size_t i = 0; i < n; ++i) src[i] = (uint8_t)(i * 131u);
  CHECK(ft_host_memcpy(dst.data() + 3, src.data(), n, 5) == 0);      // misaligned destination
  CHECK(memcmp(dst.data() + 3, src.data(), n) == 0);
  CHECK(dst[2] == 0 && dst[n + 3] == 0);
  CHECK(ft_host_memcpy(src.data() + 1, src.data(), 100, 1) == -1);   // overlap is refused
  int locked = -1;
  void* a = ft_locked_alloc(10000, &locked);
  CHECK(a != nullptr && (locked == 0 || locked == 1));
  CHECK(ft_locked_is_managed(a) == 1);
  memset(a, 7, 10000);
  CHECK(ft_locked_free(a) == 0);
  CHECK(ft_locked_free(a) == -1);
}

static void test_nvme(const std::string& dir, int kind) {
  void* h = ft_nvme_create(1 << 16, 4, 2, kind, 0);
  if (!h) { CHECK(kind != 3); return; }           // only the portable engine must always exist
  const int64_t n = (1 << 20) + 4096;
  std::vector<uint8_t> out(n), in(n, 0);
  for (int64_t i = 0; i < n; ++i) out[i] = (uint8_t)(i * 17u + (unsigned)kind);
  const std::string f1 = dir + "/selftest_" + std::to_string(kind) + "_a.swp";
  const std::string f2 = dir + "/selftest_" + std::to_string(kind) + "_b.swp";
  CHECK(ft_nvme_sync_rw(h, f1.c_str(), out.data(), n, 0, 1) == 0);
  CHECK(ft_nvme_sync_rw(h, f1.c_str(), in.data(), n, 0, 0) == 0);
  CHECK(memcmp(in.data(), out.data(), n) == 0);
  // several operations in flight, then one collective wait
  std::vector<int64_t> ids;
  for (int k = 0; k < 4; ++k) ids.push_back(ft_nvme_submit(h, f2.c_str(), out.data() + k * 65536, 65536, k * 65536, 1));
  for (auto id : ids) CHECK(id > 0);
  CHECK(ft_nvme_wait(h) >= 0);
  std::fill(in.begin(), in.end(), 0);
  int64_t rid = ft_nvme_submit(h, f2.c_str(), in.data(), 4 * 65536, 0, 0);
  CHECK(rid > 0 && ft_nvme_wait_op(h, rid) == 0);
  CHECK(memcmp(in.data(), out.data(), 4 * 65536) == 0);
  // registered staging buffer: same data path with fixed-buffer requests where the kernel
  // accepts the registration (io_uring engine only)
  {
    void* ptrs[1] = {out.data()};
    int64_t lens[1] = {n};
    const int holders = ft_nvme_register_buffers(h, ptrs, lens, 1);
    CHECK(holders >= 0);
    CHECK(ft_nvme_sync_rw(h, f1.c_str(), out.data(), n, 0, 1) == 0);
    std::fill(in.begin(), in.end(), 0);
    CHECK(ft_nvme_sync_rw(h, f1.c_str(), in.data(), n, 0, 0) == 0);
    CHECK(memcmp(in.data(), out.data(), n) == 0);
    if (holders > 0) CHECK(ft_nvme_fixed_ops(h) > 0);
    CHECK(ft_nvme_register_buffers(h, nullptr, nullptr, 0) == 0);
  }
  // an injected I/O error surfaces as a status code, and the engine keeps working
  ft_nvme_inject_fault(h, 1, 1);
  CHECK(ft_nvme_sync_rw(h, f1.c_str(), in.data(), 65536, 0, 0) != 0);
  CHECK(ft_nvme_sync_rw(h, f1.c_str(), in.data(), 65536, 0, 0) == 0);
  CHECK(ft_nvme_sync_rw(h, (dir + "/does_not_exist.swp").c_str(), in.data(), 4096, 0, 0) != 0);
  ft_nvme_forget(h, f1.c_str());
  ft_nvme_forget(h, f2.c_str());
  ft_nvme_destroy(h);
  unlink(f1.c_str());
  unlink(f2.c_str());
}

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  test_adam();
  test_copy_and_locked();
  for (int kind = 1; kind <= 3; ++kind) test_nvme(dir, kind);
  if (g_failed) { fprintf(stderr, "host_selftest: %d check(s) failed\n", g_failed); return 1; }
  printf("host_selftest: ok\n");
  return 0;
}
