// Warp-level tensor-core helpers shared by the 8x8 block kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {
namespace bsr8 {

constexpr int kWarps = 8;
constexpr int kThreadsBsr = kWarps * 32;

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool BF16>
__device__ __forceinline__ void mma_16bit(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// 16-byte asynchronous copy global -> shared, bypassing L1; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// x = hi + lo with hi holding the top 10 mantissa bits (what a tf32 operand keeps); the tensor
// core ignores the low 13 bits of a tf32 register, so `lo` is passed as it is.
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = __float_as_uint(x) & 0xffffe000u;
  lo = __float_as_uint(x - __uint_as_float(hi));
}

// Work item of a warp -> (group of block rows, feature tile).  Default order: tile index fastest;
// with tile_major_groups > 0 all groups of tile 0 come first, then tile 1, ...  The common
// shapes avoid the 64-bit division (a warp's whole job is a few thousand cycles; a software
// division is a measurable part of that).
__device__ __forceinline__ void split_work(int64_t work, int tiles, int64_t tile_major_groups, int64_t& grp, int& tile) {
  if (tile_major_groups > 0) {
    if ((work | tile_major_groups) >> 32) {
      grp = work % tile_major_groups;
      tile = (int)(work / tile_major_groups);
    } else {
      const uint32_t q = (uint32_t)work / (uint32_t)tile_major_groups;
      tile = (int)q;
      grp = (uint32_t)work - q * (uint32_t)tile_major_groups;
    }
  } else if (tiles == 1) {
    grp = work;
    tile = 0;
  } else if (work >> 32) {
    grp = work / tiles;
    tile = (int)(work % tiles);
  } else {
    const uint32_t q = (uint32_t)work / (uint32_t)tiles;
    grp = q;
    tile = (int)((uint32_t)work - q * (uint32_t)tiles);
  }
}

}  // namespace bsr8
}  // namespace lf
