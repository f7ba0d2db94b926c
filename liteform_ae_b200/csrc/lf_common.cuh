// Shared host/device helpers for the liteform_b200 library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "liteform_b200.h"

namespace lf {

// Thread-local message behind lf_last_error().
char* error_buffer();
int fail(int status, const char* fmt, ...);

#define LF_CUDA_CHECK(expr)                                                                   \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return lf::fail(LF_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                      __FILE__, __LINE__);                                                    \
  } while (0)

#define LF_REQUIRE(cond, ...)                                            \
  do {                                                                   \
    if (!(cond)) return lf::fail(LF_ERR_INVALID_ARGUMENT, __VA_ARGS__);  \
  } while (0)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

constexpr int kBucketAlign = 64;  // elements; bucket starts inside the rows/cols/vals arenas

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ceil(log2(d)) for d >= 1, on integers (the reference uses math.ceil(math.log2(d))).
__device__ __forceinline__ int ceil_log2_u32(uint32_t d) { return d <= 1 ? 0 : 32 - __clz(d - 1); }

// Warp-level inclusive scan.
__device__ __forceinline__ int warp_inclusive_scan(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Exclusive scan of one int per thread over a block of kThreads (multiple of 32, <= 1024).
// `smem` needs kThreads/32 + 1 ints.  Returns the exclusive prefix; *total gets the block sum.
template <int kThreads>
__device__ __forceinline__ int block_exclusive_scan(int v, int* smem, int* total) {
  constexpr int kWarps = kThreads / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = warp_inclusive_scan(v);
  if (lane == 31) smem[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kWarps ? smem[lane] : 0;
    int winc = warp_inclusive_scan(w);
    if (lane < kWarps) smem[lane] = winc - w;
    if (lane == kWarps - 1) smem[kWarps] = winc;
  }
  __syncthreads();
  int res = inc - v + smem[warp];
  *total = smem[kWarps];
  __syncthreads();
  return res;
}

}  // namespace lf
