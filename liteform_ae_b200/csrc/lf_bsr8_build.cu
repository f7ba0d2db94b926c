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

// ---------------------------------------------------------------------------------------------
// Coarse blocks (R x C, both multiples of 8) -> 8x8 tiles.  The reference's block path hands over
// 32x32 fp16 blocks (bench_bsrmm(bsr_mat, x, block_size=32), format_algos.py:1562-1643); the
// product kernels here take 8x8 tiles, and the zero padding inside coarse blocks must not become
// tiles.  Three launches: flag the candidate tiles that hold a nonzero; count them per fine block
// row and scan; write block columns and tiles in order (coarse column, then sub-column).
// A candidate tile is (coarse block b, sub-row a, sub-column c), flag index (b * R/8 + a) * C/8 + c.
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }

template <typename T>
__global__ void __launch_bounds__(256)
split8_flag_kernel(const T* __restrict__ data, int64_t candidates, int R, int C, uint8_t* __restrict__ flags) {
  const int Ra = R / 8, Cc = C / 8;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < candidates; q += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(q % Cc);
    const int64_t t = q / Cc;
    const int a = (int)(t % Ra);
    const int64_t b = t / Ra;
    const T* src = data + (b * R + a * 8) * C + c * 8;
    bool any = false;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) any |= to_float<T>(src[i * C + j]) != 0.f;
    flags[q] = any ? 1 : 0;
  }
}

// counts[f + 1] = tiles of fine block row f = I * R/8 + a
__global__ void __launch_bounds__(256)
split8_count_kernel(const int64_t* __restrict__ indptr, const uint8_t* __restrict__ flags, int64_t fine_rows, int Ra,
                    int Cc, int64_t* __restrict__ out_indptr) {
  const int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= fine_rows) return;
  const int64_t I = f / Ra;
  const int a = (int)(f % Ra);
  int64_t n = 0;
  for (int64_t b = indptr[I]; b < indptr[I + 1]; ++b) {
    const uint8_t* fl = flags + (b * Ra + a) * Cc;
    for (int c = 0; c < Cc; ++c) n += fl[c];
  }
  out_indptr[f + 1] = n;
}

// One warp per fine block row: walks its candidate tiles in order, 32 at a time; the kept ones get
// consecutive output positions (ballot prefix) and are copied by the whole warp, two elements per
// lane, converted to the output type.  Zeros are written as +0 (what a rebuild from the nonzero
// entries produces).
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
split8_fill_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices, const TI* __restrict__ data,
                   const uint8_t* __restrict__ flags, int64_t fine_rows, int R, int C,
                   const int64_t* __restrict__ out_indptr, int32_t* __restrict__ out_indices, TO* __restrict__ out_blocks) {
  const int Ra = R / 8, Cc = C / 8;
  const int lane = threadIdx.x & 31;
  const int64_t f = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (f >= fine_rows) return;
  const int64_t I = f / Ra;
  const int a = (int)(f % Ra);
  const int64_t b0 = indptr[I];
  const int64_t cand = (indptr[I + 1] - b0) * Cc;
  int64_t out = out_indptr[f];
  for (int64_t q0 = 0; q0 < cand; q0 += 32) {
    const int64_t q = q0 + lane;
    int64_t b = 0;
    int c = 0;
    bool keep = false;
    if (q < cand) {
      b = b0 + q / Cc;
      c = (int)(q % Cc);
      keep = flags[(b * Ra + a) * Cc + c] != 0;
    }
    const unsigned kept = __ballot_sync(0xffffffffu, keep);
    if (keep) out_indices[out + __popc(kept & ((1u << lane) - 1u))] = indices[b] * Cc + c;
    int k = 0;
    for (unsigned todo = kept; todo; todo &= todo - 1, ++k) {
      const int src_lane = __ffs(todo) - 1;
      const int64_t sb = __shfl_sync(0xffffffffu, b, src_lane);
      const int sc = __shfl_sync(0xffffffffu, c, src_lane);
      const TI* src = data + (sb * R + a * 8) * C + sc * 8;
      TO* dst = out_blocks + (out + k) * 64;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int e = lane + 32 * h;           // element of the tile: row e / 8, column e % 8
        const float x = to_float<TI>(src[(e >> 3) * C + (e & 7)]);
        dst[e] = from_float<TO>(x == 0.f ? 0.f : x);
      }
    }
    out += __popc(kept);
  }
}

template <typename TI>
int split8_fill_launch(int out_dtype, const int64_t* indptr, const int32_t* indices, const TI* data, const uint8_t* flags,
                       int64_t fine_rows, int R, int C, const int64_t* out_indptr, int32_t* out_indices, void* out_blocks,
                       cudaStream_t st) {
  const int64_t grid = ceil_div64(fine_rows, 8);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  switch (out_dtype) {
    case LF_DTYPE_F32:
      split8_fill_kernel<TI, float><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, data, flags, fine_rows, R, C,
                                                                    out_indptr, out_indices, (float*)out_blocks);
      break;
    case LF_DTYPE_BF16:
      split8_fill_kernel<TI, __nv_bfloat16><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, data, flags, fine_rows, R, C,
                                                                            out_indptr, out_indices, (__nv_bfloat16*)out_blocks);
      break;
    default:
      split8_fill_kernel<TI, __half><<<(unsigned)grid, 256, 0, st>>>(indptr, indices, data, flags, fine_rows, R, C,
                                                                     out_indptr, out_indices, (__half*)out_blocks);
      break;
  }
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

int check_split8(const void* indptr, const void* data, int64_t block_rows, int64_t num_blocks, int R, int C, int in_dtype) {
  LF_REQUIRE(indptr && block_rows >= 0 && num_blocks >= 0, "bad arguments");
  LF_REQUIRE(R >= 8 && C >= 8 && R % 8 == 0 && C % 8 == 0 && R <= 1024 && C <= 1024,
             "block shape %d x %d is not a multiple of 8 (or exceeds 1024)", R, C);
  LF_REQUIRE(in_dtype >= LF_DTYPE_F32 && in_dtype <= LF_DTYPE_F16, "unknown dtype %d", in_dtype);
  LF_REQUIRE(num_blocks == 0 || data, "block data missing");
  LF_REQUIRE(num_blocks * (int64_t)(R / 8) * (C / 8) < (1ll << 31), "more than 2^31-1 candidate tiles are not supported");
  return LF_OK;
}

}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

size_t lf_bsr_split8_scratch_bytes(int64_t num_blocks, int32_t R, int32_t C) {
  if (num_blocks < 0 || R < 8 || C < 8) return 0;
  return align_up((size_t)num_blocks * (size_t)(R / 8) * (size_t)(C / 8) + 1, 256);
}

int lf_bsr_split8_plan(const int64_t* indptr, const void* data, int32_t in_dtype, int64_t block_rows,
                       int64_t num_blocks, int32_t R, int32_t C, void* scratch, size_t scratch_bytes,
                       int64_t* out_indptr, int64_t* num_tiles, void* stream) {
  if (int s = check_split8(indptr, data, block_rows, num_blocks, R, C, in_dtype)) return s;
  LF_REQUIRE(scratch && out_indptr && num_tiles, "null pointer argument");
  if (scratch_bytes < lf_bsr_split8_scratch_bytes(num_blocks, R, C)) return fail(LF_ERR_WORKSPACE_TOO_SMALL, "split scratch too small");
  cudaStream_t st = (cudaStream_t)stream;
  const int Ra = R / 8, Cc = C / 8;
  const int64_t fine_rows = block_rows * Ra;
  const int64_t candidates = num_blocks * Ra * Cc;
  uint8_t* flags = (uint8_t*)scratch;
  *num_tiles = 0;
  if (candidates > 0) {
    const int64_t want = ceil_div64(candidates, 256);
    const unsigned grid = (unsigned)(want > 148 * 64 ? 148 * 64 : want);
    if (in_dtype == LF_DTYPE_F32) split8_flag_kernel<float><<<grid, 256, 0, st>>>((const float*)data, candidates, R, C, flags);
    else if (in_dtype == LF_DTYPE_BF16) split8_flag_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)data, candidates, R, C, flags);
    else split8_flag_kernel<__half><<<grid, 256, 0, st>>>((const __half*)data, candidates, R, C, flags);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  if (fine_rows == 0) {
    LF_CUDA_CHECK(cudaMemsetAsync(out_indptr, 0, sizeof(int64_t), st));
    LF_CUDA_CHECK(cudaStreamSynchronize(st));
    return LF_OK;
  }
  LF_REQUIRE(ceil_div64(fine_rows, 256) < (1ll << 31), "too many block rows");
  split8_count_kernel<<<(unsigned)ceil_div64(fine_rows, 256), 256, 0, st>>>(indptr, flags, fine_rows, Ra, Cc, out_indptr);
  LF_CUDA_CHECK(cudaGetLastError());
  scan_counts_kernel<<<1, kScanThreads, 0, st>>>(out_indptr, fine_rows);
  LF_CUDA_CHECK(cudaGetLastError());
  LF_CUDA_CHECK(cudaMemcpyAsync(num_tiles, out_indptr + fine_rows, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  return LF_OK;
}

int lf_bsr_split8_fill(const int64_t* indptr, const int32_t* indices, const void* data, int32_t in_dtype,
                       int64_t block_rows, int64_t num_blocks, int32_t R, int32_t C, const void* scratch,
                       const int64_t* out_indptr, int32_t* out_indices, void* out_blocks, int32_t out_dtype,
                       void* stream) {
  if (int s = check_split8(indptr, data, block_rows, num_blocks, R, C, in_dtype)) return s;
  LF_REQUIRE(out_dtype >= LF_DTYPE_F32 && out_dtype <= LF_DTYPE_F16, "unknown dtype %d", out_dtype);
  LF_REQUIRE(scratch && out_indptr, "null pointer argument");
  const int64_t fine_rows = block_rows * (R / 8);
  if (fine_rows == 0 || num_blocks == 0) return LF_OK;
  LF_REQUIRE(indices, "block columns missing");
  if (!out_indices || !out_blocks) {   // legal only when the plan found no tile; the kernel then writes nothing
    LF_REQUIRE(!out_indices && !out_blocks, "output arrays missing");
  }
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* flags = (const uint8_t*)scratch;
  if (in_dtype == LF_DTYPE_F32)
    return split8_fill_launch<float>(out_dtype, indptr, indices, (const float*)data, flags, fine_rows, R, C, out_indptr,
                                     out_indices, out_blocks, st);
  if (in_dtype == LF_DTYPE_BF16)
    return split8_fill_launch<__nv_bfloat16>(out_dtype, indptr, indices, (const __nv_bfloat16*)data, flags, fine_rows, R,
                                             C, out_indptr, out_indices, out_blocks, st);
  return split8_fill_launch<__half>(out_dtype, indptr, indices, (const __half*)data, flags, fine_rows, R, C, out_indptr,
                                    out_indices, out_blocks, st);
}

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
