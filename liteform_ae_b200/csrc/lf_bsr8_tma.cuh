// Launchers of the 8x8 block kernels that copy through the tensor memory accelerator
// (lf_spmm_bsr8_tma.cu); arguments are those of the public entry points, already validated.
// rows = false: tiled copies of swizzled boxes through a tensor map; true: one bulk copy per B row.
#pragma once

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

// Synchronises the stream, then returns (and clears) the number of warps that gave up waiting
// for a copy since the last call.
int bsr8_tma_timeouts(cudaStream_t st, int* count);

}  // namespace lf
