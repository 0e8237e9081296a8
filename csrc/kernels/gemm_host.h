// Host-side helpers shared by the GEMM launchers: cached TMA tensor maps, the
// per-device error word and the SM count.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace ft {
namespace gemm {

// 2-D row-major tensor [outer, inner] of 16-bit (or, with dtype kF32, 32-bit)
// elements with row stride ld (elements), 128-byte swizzle.  Returns 0 or a negative error.
int make_tmap(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
              uint32_t box_inner, uint32_t box_outer, int dtype);
int* error_word(int dev);
int sm_count(int dev);

}  // namespace gemm
}  // namespace ft
