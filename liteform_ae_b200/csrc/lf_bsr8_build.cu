// CSR -> 8x8 block-sparse rows on the device.
//
// The reference converts on the host with SciPy (MTX.tobsr_with_padding,
// playground_pipline/format_matrix_market.py:116-138: pad the shape, scipy.sparse.bsr_matrix).
// Here eight lanes own one block row, one lane per matrix row.  Columns are sorted inside a CSR
// row, so the block columns of a block row come out of an eight-way merge: the lanes agree on
// the smallest block column any of them still has, that is the next block, and every lane
// consumes its entries inside it (at most 8).  The same walk runs twice: once counting blocks
// (lf_bsr8_plan, followed by a scan that turns the counts into the block-row pointer), once
// writing block columns and the dense 8x8 tiles (lf_bsr8_fill).  Rows past M (the padding up to
// a multiple of 8) are empty; a tile holds zeros wherever the matrix has no entry, as SciPy's.
// The CSR input is canonical (sorted columns, no duplicate entry in a row), as everywhere in
// this library.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lf_common.cuh"

namespace lf {
namespace {

constexpr int kBuildThreads = 256;
constexpr int kRowsPerCta = kBuildThreads / 8;   // block rows per thread block
constexpr int kNoBlock = 0x7fffffff;

__device__ __forceinline__ int group_min8(int v) {
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = min(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
__device__ __forceinline__ uint32_t bits(float x) { return __float_as_uint(x); }
__device__ __forceinline__ uint32_t bits(__nv_bfloat16 x) { return __bfloat16_as_ushort(x); }
__device__ __forceinline__ uint32_t bits(__half x) { return __half_as_ushort(x); }

// FILL = false: counts[I + 1] = number of blocks of block row I.
// FILL = true: writes block columns and tiles at bsr_indptr[I] + k for the k-th block.
template <bool FILL, typename T>
__global__ void __launch_bounds__(kBuildThreads)
bsr8_walk_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                 const float* __restrict__ data, int64_t M, int64_t Mb, int64_t* __restrict__ bsr_indptr,
                 int32_t* __restrict__ bsr_indices, T* __restrict__ blocks) {
  const int l = threadIdx.x & 7;
  // whole warps stay in the loop together (the shuffles name all 32 lanes): block rows past Mb
  // simply have nothing to merge
  const int64_t I = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 3);
  const int64_t row = I * 8 + l;
  const bool live = I < Mb && row < M;
  int64_t pos = live ? indptr[row] : 0;
  const int64_t end = live ? indptr[row + 1] : 0;
  int64_t out = (FILL && I < Mb) ? bsr_indptr[I] : 0;
  int count = 0;
  for (;;) {
    const int mine = pos < end ? (indices[pos] >> 3) : kNoBlock;
    const int J = group_min8(mine);
    if (__all_sync(0xffffffffu, J == kNoBlock)) break;
    if (J == kNoBlock) continue;   // this group is done, another group of the warp is not
    if (FILL) {
      T tile_row[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) tile_row[c] = from_float<T>(0.f);
      while (pos < end) {
        const int col = indices[pos];
        if ((col >> 3) != J) break;
        const T v = from_float<T>(data ? data[pos] : 1.0f);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if ((col & 7) == c) tile_row[c] = v;
        ++pos;
      }
      if (l == 0) bsr_indices[out] = J;
      T* dst = blocks + out * 64 + l * 8;
      uint32_t w[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) w[c] = bits(tile_row[c]);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      if (sizeof(T) == 4) {
        d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
        d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
      } else {
        d4[0] = make_uint4(w[0] | (w[1] << 16), w[2] | (w[3] << 16), w[4] | (w[5] << 16), w[6] | (w[7] << 16));
      }
      ++out;
    } else {
      while (pos < end && (indices[pos] >> 3) == J) ++pos;
      ++count;
    }
  }
  if (!FILL && l == 0 && I < Mb) bsr_indptr[I + 1] = count;
}

// In-place inclusive scan of v[1..n] by one thread block (v[0] = 0): 8 elements per thread and
// step, no inter-block hand-off to wait for.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
scan_counts_kernel(int64_t* __restrict__ v, int64_t n) {
  __shared__ int s_scan[kScanThreads / 32 + 1];
  int64_t running = 0;
  if (threadIdx.x == 0) v[0] = 0;
  for (int64_t base = 0; base < n; base += (int64_t)kScanThreads * 8) {
    const int64_t i0 = base + (int64_t)threadIdx.x * 8;
    int x[8], sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      x[k] = i0 + k < n ? (int)v[1 + i0 + k] : 0;
      sum += x[k];
    }
    int tot;
    int64_t acc = running + block_exclusive_scan<kScanThreads>(sum, s_scan, &tot);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      acc += x[k];
      if (i0 + k < n) v[1 + i0 + k] = acc;
    }
    running += tot;
  }
}

}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

int lf_bsr8_plan(const int64_t* indptr, const int32_t* indices, int64_t M, int64_t* bsr_indptr,
                 int64_t* num_blocks, void* stream) {
  LF_REQUIRE(indptr && bsr_indptr && num_blocks, "null pointer argument");
  LF_REQUIRE(M >= 0, "bad row count");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t Mb = ceil_div64(M, 8);
  *num_blocks = 0;
  if (Mb == 0) {
    LF_CUDA_CHECK(cudaMemsetAsync(bsr_indptr, 0, sizeof(int64_t), st));
    LF_CUDA_CHECK(cudaStreamSynchronize(st));
    return LF_OK;
  }
  const int64_t grid = ceil_div64(Mb, kRowsPerCta);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  int64_t h_nnz = 0;
  LF_CUDA_CHECK(cudaMemcpyAsync(&h_nnz, indptr + M, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  bsr8_walk_kernel<false, float><<<(unsigned)grid, kBuildThreads, 0, st>>>(indptr, indices, nullptr, M, Mb, bsr_indptr,
                                                                           nullptr, nullptr);
  LF_CUDA_CHECK(cudaGetLastError());
  scan_counts_kernel<<<1, kScanThreads, 0, st>>>(bsr_indptr, Mb);
  LF_CUDA_CHECK(cudaGetLastError());
  LF_CUDA_CHECK(cudaMemcpyAsync(num_blocks, bsr_indptr + Mb, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  if (h_nnz > 0x7fffffffll) return fail(LF_ERR_UNSUPPORTED, "more than 2^31-1 stored entries are not supported");
  return LF_OK;
}

int lf_bsr8_fill(const int64_t* indptr, const int32_t* indices, const float* data, int64_t M,
                 const int64_t* bsr_indptr, int32_t* bsr_indices, void* blocks, int32_t dtype, void* stream) {
  LF_REQUIRE(indptr && bsr_indptr, "null pointer argument");
  LF_REQUIRE(M >= 0, "bad row count");
  LF_REQUIRE(dtype >= LF_DTYPE_F32 && dtype <= LF_DTYPE_F16, "unknown dtype %d", dtype);
  const int64_t Mb = ceil_div64(M, 8);
  if (Mb == 0) return LF_OK;
  if (!bsr_indices || !blocks) {
    // legal only when the plan found no block at all; the kernel then writes nothing
    LF_REQUIRE(!bsr_indices && !blocks, "block arrays missing");
  }
  LF_REQUIRE((uintptr_t)blocks % 16 == 0, "blocks must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t grid = ceil_div64(Mb, kRowsPerCta);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  int64_t* ptr = const_cast<int64_t*>(bsr_indptr);
  switch (dtype) {
    case LF_DTYPE_F32:
      bsr8_walk_kernel<true, float><<<(unsigned)grid, kBuildThreads, 0, st>>>(indptr, indices, data, M, Mb, ptr,
                                                                              bsr_indices, (float*)blocks);
      break;
    case LF_DTYPE_BF16:
      bsr8_walk_kernel<true, __nv_bfloat16><<<(unsigned)grid, kBuildThreads, 0, st>>>(
          indptr, indices, data, M, Mb, ptr, bsr_indices, (__nv_bfloat16*)blocks);
      break;
    default:
      bsr8_walk_kernel<true, __half><<<(unsigned)grid, kBuildThreads, 0, st>>>(indptr, indices, data, M, Mb, ptr,
                                                                               bsr_indices, (__half*)blocks);
      break;
  }
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

}  // extern "C"
