// Launchers of the 8x8 block kernels that copy through the tensor memory accelerator
// (lf_spmm_bsr8_tma.cu); arguments are those of the public entry points, already validated.
// rows = false: tiled copies of swizzled boxes through a tensor map; true: one bulk copy per B row.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lf {

extern int g_bsr_copy_engine;   // LF_OPT_BSR_COPY_ENGINE
extern int g_bsr_tile_order;    // LF_OPT_BSR_TILE_ORDER

int bsr8_f32_tma_launch(bool rows, const int64_t* indptr, const int32_t* indices, const float* blocks, int64_t r0, int64_t r1,
                        const float* B, int64_t ldb, float* C, int64_t ldc, int N, int stages, int rows_per_warp,
                        bool tile_major, cudaStream_t st);

int bsr8_16bit_tma_launch(bool rows, bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                          int64_t r0, int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int N,
                          int stages, int rows_per_warp, cudaStream_t st);

// The thread-block-wide pipeline (lf_spmm_bsr8_pipe.cu): a producer warp issues one tiled copy per
// block, consumer warps run the MMAs.  shape = blocks per stage * 10 + stages (0 = default).
int bsr8_f32_pipe_launch(const int64_t* indptr, const int32_t* indices, const float* blocks, int64_t r0, int64_t r1,
                         const float* B, int64_t ldb, float* C, int64_t ldc, int N, int shape, int rows_per_cta,
                         bool tile_major, bool allow_3d, cudaStream_t st);
int bsr8_16bit_pipe_launch(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks, int64_t r0,
                           int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int N, int shape,
                           int rows_per_cta, bool allow_3d, cudaStream_t st);
int bsr8_pipe_timeouts(cudaStream_t st, int* count);

// Tensor map over B (memory of this GPU) for one tiled copy per block: 3-D {128 bytes of features,
// rows, feature slices} when N is a whole number of slices and the driver accepts the view
// (*boxes_per_block = 1), else 2-D {N, rows} with one copy per slice (*boxes_per_block = slices).
int bsr8_make_b_map(CUtensorMap* map, int* boxes_per_block, const void* B, int64_t ldb, int N, int elem_bytes,
                    int slices, bool allow_3d);

// 16-bit inputs on the 5th-generation tensor cores (lf_spmm_bsr8_umma.cu): tcgen05.mma with the
// accumulators in tensor memory, fed by the same tiled copies.  shape as above.
// producer: 0 = one warp issuing tiled bulk copies, 2 / 4 = that many warps issuing per-lane cp.async
int bsr8_16bit_umma_launch(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks, int64_t r0,
                           int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int N, int shape,
                           int rows_per_cta, bool allow_3d, int producer, cudaStream_t st);
extern int g_bsr_umma_producer;   // LF_OPT_BSR_UMMA_PRODUCER
int bsr8_umma_timeouts(cudaStream_t st, int* count);

extern int g_bsr_block_warps;   // LF_OPT_BSR_BLOCK_WARPS
extern int g_bsr_pipe_shape;    // LF_OPT_BSR_PIPE_SHAPE
extern int g_bsr_pipe_3d;       // LF_OPT_BSR_PIPE_3D

// Synchronises the stream, then returns (and clears) the number of warps that gave up waiting
// for a copy since the last call.
int bsr8_tma_timeouts(cudaStream_t st, int* count);

}  // namespace lf
