// Block-sparse SpMM for 8x8 blocks: C[I*8 + i, :] = sum over blocks (I, J) of A_IJ[i, :] * B[J*8 : J*8+8, :].
//
// Takes over the kernel of the reference's bench_bsrmm (playground_pipline/format_algos.py:1562-1643;
// arithmetic format_algos.py:1204-1213), which multiplies 32x32 fp16 blocks with wmma 16x16x16
// fragments and fp16 accumulators (format_algos.py:1226-1233, 1272-1288).  Here blocks are 8x8 (a
// coarser blocking is re-blocked by the caller), accumulation is always fp32, and the tensor cores
// are driven with warp-level mma.sync: the product is computed transposed, D[feature, row] =
// sum_k B^T[feature, k] * A^T[k, row], so that the 16-wide M dimension of the instruction runs
// over features (always plentiful) and the 8-wide N dimension is exactly the 8 rows of a block --
// no lane of the instruction is wasted on padding.  tcgen05.mma does not fit this shape: its
// smallest tile (M = 64, N = 8) would put one block row on a whole CTA-wide instruction with its
// operands staged through shared memory, for a kernel whose limit is L2/HBM bandwidth.
//
//   * float32 path: every operand is split x = hi + lo into two tf32 numbers and three
//     m16n8k8 tf32 MMAs (hi*hi + lo*hi + hi*lo) reproduce the fp32 product to ~2^-21 relative.
//   * 16-bit path (bf16 or fp16 inputs): m16n8k16 over a pair of blocks, fp32 accumulate.
//
// Data movement.  One warp owns a few consecutive block rows and one feature tile.  The 8 rows of B that a
// block needs (and the block itself) are copied global -> shared with 16-byte cp.async, one
// fully coalesced row (or two half rows) per instruction, into a warp-private ring of D stages,
// so D-1 blocks are in flight per warp without holding registers; the warp then reads its MMA
// fragments from shared memory with 128-bit loads.  A fragment read needs rows 2t/2t+1 for
// t = 0..3 inside every quarter warp, which would be a 4-way bank conflict on plain row-major
// rows, so the 16-byte chunks of row r are stored XOR-swizzled by r (chunk c -> c ^ (r & 7)).
// Loading fragments straight from global memory was measured at 4x the L1 wavefronts for the
// same reason (a quarter warp touches four 128-byte lines per 128-bit load).
//
// Because M and K of an MMA are only summation/placement indices, both are permuted so that every
// shared-memory access is a full 128-bit vector: a lane's four (float32) or eight (16-bit)
// consecutive features of one B row feed four / eight different MMA tiles, and the k-slots of a
// lane map to adjacent block columns so that its two A values are one 64-bit (32-bit) load.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "lf_bsr8_mma.cuh"
#include "lf_bsr8_tma.cuh"
#include "lf_common.cuh"

namespace lf {
namespace {

using namespace bsr8;

// 1 = per-lane cp.async into warp-private rings, 4 = thread-block pipeline fed by tiled bulk copies
constexpr int kDefaultCopyEngine = 1;

// ---------------------------------------------------------------------------------------------
// float32 in / float32 out, 3xTF32.  One warp = one block row x one tile of 64*T features.
// Lane (g = lane / 4, t = lane % 4).  MMA index maps:
//   k-slot t   <-> block column 2t      k-slot t+4 <-> block column 2t+1
//   MMA tile j of unit q: m = g   <-> feature F + 64q + 4g + j
//                         m = g+8 <-> feature F + 64q + 32 + 4g + j
//   n <-> row of the block; a lane ends with C[row 2t / 2t+1][4 consecutive features] as float4.
// Stage layout: 8 rows of 64*T floats (16*T chunks of 16 bytes, chunk c of row r at c ^ r),
// then the 8x8 block (256 bytes).
// ---------------------------------------------------------------------------------------------
template <int T, int D>
struct F32Cfg {
  static constexpr int kRowBytes = 256 * T;
  static constexpr int kStage = 8 * kRowBytes + 256;   // a thread block of W warps takes W * D stages
};

// A warp walks the blocks of R consecutive block rows as one stream, so the copy ring stays full
// across row boundaries; lane l keeps indptr[I0 + l] and a sliding window of 32 block columns.
template <int T, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_f32_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                     const float* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                     const float* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                     int tiles, int rows_per_warp, int64_t tile_major_groups) {
  using Cfg = F32Cfg<T, D>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  // Default order: tile index fastest, so the tiles of one block row are resident together and
  // the A blocks they share come from HBM once.  With many tiles the B rows all of them gather
  // (band x N) outgrow the L2; then (tile_major_groups > 0) all row groups of tile 0 run first,
  // then tile 1, ...: B is read from HBM once per tile and A once per tile.
  const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;   // 8 warps per block or fewer
  int64_t grp;
  int tile;
  split_work(work, tiles, tile_major_groups, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end || tile >= tiles) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * (64 * T);
  uint8_t* ring = smem_raw + warp * (D * Cfg::kStage);
  const uint32_t ring_u32 = smem_u32(ring);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];              // lane l <= R: start of row l
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;   // first block held in my_idx (none yet)
  int64_t ib = row_start(0);    // issue cursor (runs D-1 blocks ahead of the consumer)
  int slot_in = 0;

  // copy the next block of the stream (if any) into the next ring slot
  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      if (b >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const uint32_t dst = ring_u32 + slot_in * Cfg::kStage;
      const float* src = B + (int64_t)J * 8 * ldb + F;
      if (T == 2) {
        const int ok = (F + 4 * lane < N) ? 16 : 0;   // lane = chunk of the row
#pragma unroll
        for (int r = 0; r < 8; ++r)
          cp_async16(dst + r * Cfg::kRowBytes + (((lane & ~7) | ((lane ^ r) & 7)) << 4),
                     src + (int64_t)r * ldb + (ok ? 4 * lane : 0), ok);
      } else {
        const int c = lane & 15, rr = lane >> 4;      // two rows per instruction
        const int ok = (F + 4 * c < N) ? 16 : 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = 2 * i + rr;
          cp_async16(dst + r * Cfg::kRowBytes + (((c & ~7) | ((c ^ r) & 7)) << 4),
                     src + (int64_t)r * ldb + (ok ? 4 * c : 0), ok);
        }
      }
      if (lane < 16) cp_async16(dst + 8 * Cfg::kRowBytes + lane * 16, blocks + b * 64 + lane * 4, 16);
      ib = b + 1;
      slot_in = slot_in + 1 == D ? 0 : slot_in + 1;
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  int slot_out = 0;
  for (int r = 0; r < R; ++r) {
    float acc[T][4][4];
#pragma unroll
    for (int q = 0; q < T; ++q)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q][j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; ++b) {
      cp_async_wait<D - 2>();
      __syncwarp();
      issue_next();   // refills the slot consumed in the previous iteration

      const uint8_t* st = ring + slot_out * Cfg::kStage;
      slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
      const float2 av = *reinterpret_cast<const float2*>(st + 8 * Cfg::kRowBytes + (g * 8 + 2 * t) * 4);
      uint32_t b0h, b0l, b1h, b1l;
      split_tf32(av.x, b0h, b0l);
      split_tf32(av.y, b1h, b1l);
      const uint8_t* row0 = st + (2 * t) * Cfg::kRowBytes;
      const uint8_t* row1 = row0 + Cfg::kRowBytes;
      const int sw0 = ((g ^ (2 * t)) & 7) << 4, sw1 = ((g ^ (2 * t + 1)) & 7) << 4;
#pragma unroll
      for (int q = 0; q < T; ++q) {
        const float4 x0 = *reinterpret_cast<const float4*>(row0 + q * 256 + sw0);        // k = t,   m = g
        const float4 x1 = *reinterpret_cast<const float4*>(row0 + q * 256 + 128 + sw0);  // k = t,   m = g+8
        const float4 y0 = *reinterpret_cast<const float4*>(row1 + q * 256 + sw1);        // k = t+4, m = g
        const float4 y1 = *reinterpret_cast<const float4*>(row1 + q * 256 + 128 + sw1);  // k = t+4, m = g+8
        const float a_f[4][4] = {{x0.x, x1.x, y0.x, y1.x}, {x0.y, x1.y, y0.y, y1.y},
                                 {x0.z, x1.z, y0.z, y1.z}, {x0.w, x1.w, y0.w, y1.w}};
        uint32_t ah[4][4], al[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) split_tf32(a_f[j][i], ah[j][i], al[j][i]);
        // the three products of one tile depend on each other through the accumulator: issue
        // them tile-interleaved so that consecutive MMAs are independent
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[q][j], al[j], b0h, b1h);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[q][j], ah[j], b0l, b1l);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_tf32(acc[q][j], ah[j], b0h, b1h);
      }
    }

    float* c0 = C + ((I0 + r - block_row_begin) * 8 + 2 * t) * ldc + F + 4 * g;
    float* c1 = c0 + ldc;
#pragma unroll
    for (int q = 0; q < T; ++q) {
      if (F + 64 * q + 4 * g < N) {
        __stcs(reinterpret_cast<float4*>(c0 + 64 * q), make_float4(acc[q][0][0], acc[q][1][0], acc[q][2][0], acc[q][3][0]));
        __stcs(reinterpret_cast<float4*>(c1 + 64 * q), make_float4(acc[q][0][1], acc[q][1][1], acc[q][2][1], acc[q][3][1]));
      }
      if (F + 64 * q + 32 + 4 * g < N) {
        __stcs(reinterpret_cast<float4*>(c0 + 64 * q + 32), make_float4(acc[q][0][2], acc[q][1][2], acc[q][2][2], acc[q][3][2]));
        __stcs(reinterpret_cast<float4*>(c1 + 64 * q + 32), make_float4(acc[q][0][3], acc[q][1][3], acc[q][2][3], acc[q][3][3]));
      }
    }
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// float32, narrow tile: 32 features per warp, for N <= 32.  The 64-feature unit above would leave
// the upper half of every MMA (rows m = g + 8) on padding; here both halves carry features:
//   MMA tile j (j = 0, 1): m = g <-> feature F + 4g + j,  m = g + 8 <-> feature F + 4g + 2 + j
// so one 128-bit shared load per B row feeds both tiles, and a block costs 6 MMAs instead of 12.
// A stage is 8 rows of 128 bytes (chunk c of row r at c ^ r) plus the block: 1280 bytes, which
// lets the ring be twice as deep at three thread blocks per SM -- with so little work per block
// the kernel lives on the number of blocks in flight.
// ---------------------------------------------------------------------------------------------
template <int D>
struct F32NarrowCfg {
  static constexpr int kStage = 8 * 128 + 256;
  static constexpr int kSmem = kWarps * D * kStage;
};

template <int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_f32_narrow_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                            const float* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                            const float* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                            int tiles, int rows_per_warp) {
  using Cfg = F32NarrowCfg<D>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * kWarps + warp;
  int64_t grp;
  int tile;
  split_work(work, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 32;
  uint8_t* ring = smem_raw + warp * (D * Cfg::kStage);
  const uint32_t ring_u32 = smem_u32(ring);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  int64_t ib = row_start(0);
  int slot_in = 0;
  const int cc = lane & 7, rr = lane >> 3;                // chunk of the row, row within a group of four
  const int ok = (F + 4 * cc < N) ? 16 : 0;

  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      if (b >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const uint32_t dst = ring_u32 + slot_in * Cfg::kStage;
      const float* src = B + (int64_t)J * 8 * ldb + F + (ok ? 4 * cc : 0);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = 4 * i + rr;
        cp_async16(dst + r * 128 + ((cc ^ r) << 4), src + (int64_t)r * ldb, ok);
      }
      if (lane < 16) cp_async16(dst + 8 * 128 + lane * 16, blocks + b * 64 + lane * 4, 16);
      ib = b + 1;
      slot_in = slot_in + 1 == D ? 0 : slot_in + 1;
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  int slot_out = 0;
  for (int r = 0; r < R; ++r) {
    float acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; ++b) {
      cp_async_wait<D - 2>();
      __syncwarp();
      issue_next();

      const uint8_t* st = ring + slot_out * Cfg::kStage;
      slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
      const float2 av = *reinterpret_cast<const float2*>(st + 8 * 128 + (g * 8 + 2 * t) * 4);
      uint32_t b0h, b0l, b1h, b1l;
      split_tf32(av.x, b0h, b0l);
      split_tf32(av.y, b1h, b1l);
      const float4 x = *reinterpret_cast<const float4*>(st + (2 * t) * 128 + (((g ^ (2 * t)) & 7) << 4));          // k = t
      const float4 y = *reinterpret_cast<const float4*>(st + (2 * t + 1) * 128 + (((g ^ (2 * t + 1)) & 7) << 4));  // k = t+4
      const float a_f[2][4] = {{x.x, x.z, y.x, y.z}, {x.y, x.w, y.y, y.w}};
      uint32_t ah[2][4], al[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) split_tf32(a_f[j][i], ah[j][i], al[j][i]);
#pragma unroll
      for (int j = 0; j < 2; ++j) mma_tf32(acc[j], al[j], b0h, b1h);
#pragma unroll
      for (int j = 0; j < 2; ++j) mma_tf32(acc[j], ah[j], b0l, b1l);
#pragma unroll
      for (int j = 0; j < 2; ++j) mma_tf32(acc[j], ah[j], b0h, b1h);
    }

    if (F + 4 * g < N) {
      float* c0 = C + ((I0 + r - block_row_begin) * 8 + 2 * t) * ldc + F + 4 * g;
      __stcs(reinterpret_cast<float4*>(c0), make_float4(acc[0][0], acc[1][0], acc[0][2], acc[1][2]));
      __stcs(reinterpret_cast<float4*>(c0 + ldc), make_float4(acc[0][1], acc[1][1], acc[0][3], acc[1][3]));
    }
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// 16-bit in (bf16 or fp16) / float32 out.  One warp = one block row x one tile of 128 features;
// two blocks per m16n8k16 MMA.  Index maps:
//   k-slots 2t, 2t+1   <-> block 0, columns 2t, 2t+1      k-slots 2t+8, 2t+9 <-> block 1, same columns
//   MMA tile j: m = g   <-> feature F + 8g + j
//               m = g+8 <-> feature F + 64 + 8g + j
// A lane reads 8 consecutive 16-bit features (128 bits) of each of its four B rows and interleaves
// rows pairwise with byte permutes to form the packed k-pairs the MMA wants.
// Stage layout: 16 rows (8 of block 0, 8 of block 1) of 128 features (16 chunks, chunk c of row r
// at c ^ (r & 7)), then the two 8x8 blocks (2 x 128 bytes).
// ---------------------------------------------------------------------------------------------
template <int D>
struct H16Cfg {
  static constexpr int kRowBytes = 256;
  static constexpr int kStage = 16 * kRowBytes + 256;   // a thread block of W warps takes W * D stages
};

template <bool BF16, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_16bit_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                       const uint16_t* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                       const uint16_t* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                       int tiles, int rows_per_warp) {
  using Cfg = H16Cfg<D>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;   // 8 warps per block or fewer
  int64_t grp;
  int tile;
  split_work(work, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 128;
  uint8_t* ring = smem_raw + warp * (D * Cfg::kStage);
  const uint32_t ring_u32 = smem_u32(ring);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];              // lane l <= R: start of row l
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  // issue cursor: pairs never straddle a row (an odd row ends with a half-empty pair)
  int ir = 0;
  int64_t ib = row_start(0), ire = row_start(1);
  while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
  int slot_in = 0;

  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      const bool two = b + 1 < ire;
      if (b + 1 >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J0 = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const int J1 = __shfl_sync(0xffffffffu, my_idx, (int)(b + 1 - win));
      const uint32_t dst = ring_u32 + slot_in * Cfg::kStage;
      const int c = lane & 15, rr = lane >> 4;   // two rows per instruction, 16 chunks of 8 features each
      const bool in = F + 8 * c < N;
      const uint16_t* s0 = B + (int64_t)J0 * 8 * ldb + F + (in ? 8 * c : 0);
      const uint16_t* s1 = B + (int64_t)(two ? J1 : J0) * 8 * ldb + F + (in ? 8 * c : 0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 2 * i + rr;
        const uint32_t off = r * Cfg::kRowBytes + (((c & ~7) | ((c ^ r) & 7)) << 4);
        cp_async16(dst + off, s0 + (int64_t)r * ldb, in ? 16 : 0);
        cp_async16(dst + 8 * Cfg::kRowBytes + off, s1 + (int64_t)r * ldb, (in && two) ? 16 : 0);
      }
      // the two blocks: 2 x 128 bytes = 16 chunks; the second is zero-filled for a half-empty pair
      if (lane < 16)
        cp_async16(dst + 16 * Cfg::kRowBytes + lane * 16,
                   blocks + (b + ((lane >= 8 && two) ? 1 : 0)) * 64 + (lane & 7) * 8, (lane < 8 || two) ? 16 : 0);
      ib = two ? b + 2 : b + 1;
      while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
      slot_in = slot_in + 1 == D ? 0 : slot_in + 1;
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  int slot_out = 0;
  for (int r = 0; r < R; ++r) {
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; b += 2) {
      cp_async_wait<D - 2>();
      __syncwarp();
      issue_next();

      const uint8_t* st = ring + slot_out * Cfg::kStage;
      slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(st + 16 * Cfg::kRowBytes + (g * 8 + 2 * t) * 2);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(st + 16 * Cfg::kRowBytes + 128 + (g * 8 + 2 * t) * 2);
      const int sw0 = ((g ^ (2 * t)) & 7) << 4, sw1 = ((g ^ (2 * t + 1)) & 7) << 4;
      // [row][half]: rows = (blk0 col 2t), (blk0 col 2t+1), (blk1 col 2t), (blk1 col 2t+1)
      uint4 v[4][2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        v[0][h] = *reinterpret_cast<const uint4*>(st + (2 * t) * Cfg::kRowBytes + h * 128 + sw0);
        v[1][h] = *reinterpret_cast<const uint4*>(st + (2 * t + 1) * Cfg::kRowBytes + h * 128 + sw1);
        v[2][h] = *reinterpret_cast<const uint4*>(st + (8 + 2 * t) * Cfg::kRowBytes + h * 128 + sw0);
        v[3][h] = *reinterpret_cast<const uint4*>(st + (8 + 2 * t + 1) * Cfg::kRowBytes + h * 128 + sw1);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // feature j of the lane's 8: 32-bit word j/2, half-word j%2 of each 128-bit load
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;  // (hi,hi) or (lo,lo) halves of two words
        auto word = [&](const uint4& u) { return j < 2 ? u.x : (j < 4 ? u.y : (j < 6 ? u.z : u.w)); };
        uint32_t a[4];
        a[0] = __byte_perm(word(v[0][0]), word(v[1][0]), sel);  // m = g,   k = 2t, 2t+1
        a[1] = __byte_perm(word(v[0][1]), word(v[1][1]), sel);  // m = g+8, k = 2t, 2t+1
        a[2] = __byte_perm(word(v[2][0]), word(v[3][0]), sel);  // m = g,   k = 2t+8, 2t+9
        a[3] = __byte_perm(word(v[2][1]), word(v[3][1]), sel);  // m = g+8, k = 2t+8, 2t+9
        mma_16bit<BF16>(acc[j], a, b0, b1);
      }
    }

    float* c0 = C + ((I0 + r - block_row_begin) * 8 + 2 * t) * ldc + F + 8 * g;
    float* c1 = c0 + ldc;
#pragma unroll
    for (int h = 0; h < 2; ++h) {  // features 8g + 4h .. +3
      if (F + 8 * g < N) {
        __stcs(reinterpret_cast<float4*>(c0 + 4 * h), make_float4(acc[4 * h][0], acc[4 * h + 1][0], acc[4 * h + 2][0], acc[4 * h + 3][0]));
        __stcs(reinterpret_cast<float4*>(c1 + 4 * h), make_float4(acc[4 * h][1], acc[4 * h + 1][1], acc[4 * h + 2][1], acc[4 * h + 3][1]));
      }
      if (F + 64 + 8 * g < N) {
        __stcs(reinterpret_cast<float4*>(c0 + 64 + 4 * h), make_float4(acc[4 * h][2], acc[4 * h + 1][2], acc[4 * h + 2][2], acc[4 * h + 3][2]));
        __stcs(reinterpret_cast<float4*>(c1 + 64 + 4 * h), make_float4(acc[4 * h][3], acc[4 * h + 1][3], acc[4 * h + 2][3], acc[4 * h + 3][3]));
      }
    }
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// 16-bit, narrow tile: 32 features per warp, for N <= 32 (the 128-feature tile above would spend
// three quarters of every MMA on padding).  As in the float32 narrow kernel both halves of an
// MMA carry features:  tile j (j = 0, 1): m = g <-> feature F + 4g + j,  m = g + 8 <-> F + 4g + 2 + j,
// so a lane needs 4 consecutive 16-bit features (64 bits) of each of its four B rows and a block
// pair costs 2 MMAs.  Stage: 16 rows of 64 bytes cut into 32-byte pieces (piece h of row r holds
// features 16h .. 16h + 15) plus the two blocks, 1280 bytes.  Piece (r, h) lies in 128-byte line
// (r & 1) + 2h + 4(r >> 3) at byte 32 ((r >> 1) & 3): the 16 lanes of one 64-bit load phase
// (g = 0..3 or 4..7, t = 0..3) then read one whole line, each its own 8 bytes.
// ---------------------------------------------------------------------------------------------
template <int D>
struct H16NarrowCfg {
  static constexpr int kStage = 16 * 64 + 256;
  static constexpr int kSmem = kWarps * D * kStage;
};

__device__ __forceinline__ int narrow16_offset(int r, int h) {
  return ((r & 1) + 2 * h + 4 * (r >> 3)) * 128 + ((r >> 1) & 3) * 32;
}

template <bool BF16, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_16bit_narrow_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                              const uint16_t* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                              const uint16_t* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                              int tiles, int rows_per_warp) {
  using Cfg = H16NarrowCfg<D>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * kWarps + warp;
  int64_t grp;
  int tile;
  split_work(work, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 32;
  uint8_t* ring = smem_raw + warp * (D * Cfg::kStage);
  const uint32_t ring_u32 = smem_u32(ring);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  int ir = 0;
  int64_t ib = row_start(0), ire = row_start(1);
  while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
  int slot_in = 0;
  const int cc = lane & 3, rl = lane >> 2;      // 16-byte chunk of a 64-byte row, row of the block
  const bool in = F + 8 * cc < N;
  // chunk cc = piece cc >> 1, second half of the piece when cc is odd
  const uint32_t off0 = narrow16_offset(rl, cc >> 1) + (cc & 1) * 16;
  const uint32_t off1 = narrow16_offset(8 + rl, cc >> 1) + (cc & 1) * 16;

  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      const bool two = b + 1 < ire;
      if (b + 1 >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J0 = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const int J1 = __shfl_sync(0xffffffffu, my_idx, (int)(b + 1 - win));
      const uint32_t dst = ring_u32 + slot_in * Cfg::kStage;
      const int64_t col = F + (in ? 8 * cc : 0);
      cp_async16(dst + off0, B + ((int64_t)J0 * 8 + rl) * ldb + col, in ? 16 : 0);
      cp_async16(dst + off1, B + ((int64_t)(two ? J1 : J0) * 8 + rl) * ldb + col, (in && two) ? 16 : 0);
      if (lane < 16)
        cp_async16(dst + 1024 + lane * 16, blocks + (b + ((lane >= 8 && two) ? 1 : 0)) * 64 + (lane & 7) * 8,
                   (lane < 8 || two) ? 16 : 0);
      ib = two ? b + 2 : b + 1;
      while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
      slot_in = slot_in + 1 == D ? 0 : slot_in + 1;
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  // where this lane reads: rows 2t, 2t+1 of block 0 and of block 1, piece g >> 2, 8 bytes at 8 (g & 3)
  const int rd0 = narrow16_offset(2 * t, g >> 2) + (g & 3) * 8;
  const int rd1 = narrow16_offset(2 * t + 1, g >> 2) + (g & 3) * 8;
  const int rd2 = narrow16_offset(8 + 2 * t, g >> 2) + (g & 3) * 8;
  const int rd3 = narrow16_offset(8 + 2 * t + 1, g >> 2) + (g & 3) * 8;

  int slot_out = 0;
  for (int r = 0; r < R; ++r) {
    float acc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; b += 2) {
      cp_async_wait<D - 2>();
      __syncwarp();
      issue_next();

      const uint8_t* st = ring + slot_out * Cfg::kStage;
      slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(st + 1024 + (g * 8 + 2 * t) * 2);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(st + 1024 + 128 + (g * 8 + 2 * t) * 2);
      const uint2 v0 = *reinterpret_cast<const uint2*>(st + rd0);   // block 0, column 2t:   features 4g .. 4g+3
      const uint2 v1 = *reinterpret_cast<const uint2*>(st + rd1);   // block 0, column 2t+1
      const uint2 v2 = *reinterpret_cast<const uint2*>(st + rd2);   // block 1, column 2t
      const uint2 v3 = *reinterpret_cast<const uint2*>(st + rd3);   // block 1, column 2t+1
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t sel = j ? 0x7632u : 0x5410u;   // second / first feature of each 32-bit word
        uint32_t a[4];
        a[0] = __byte_perm(v0.x, v1.x, sel);   // m = g   (feature 4g + j),     k = 2t, 2t+1
        a[1] = __byte_perm(v0.y, v1.y, sel);   // m = g+8 (feature 4g + 2 + j), k = 2t, 2t+1
        a[2] = __byte_perm(v2.x, v3.x, sel);   // m = g,   k = 2t+8, 2t+9
        a[3] = __byte_perm(v2.y, v3.y, sel);   // m = g+8, k = 2t+8, 2t+9
        mma_16bit<BF16>(acc[j], a, b0, b1);
      }
    }

    if (F + 4 * g < N) {
      float* c0 = C + ((I0 + r - block_row_begin) * 8 + 2 * t) * ldc + F + 4 * g;
      __stcs(reinterpret_cast<float4*>(c0), make_float4(acc[0][0], acc[1][0], acc[0][2], acc[1][2]));
      __stcs(reinterpret_cast<float4*>(c0 + ldc), make_float4(acc[0][1], acc[1][1], acc[0][3], acc[1][3]));
    }
  }
  cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// 16-bit, 64 features per warp, for 32 < N <= 64 (the 128-feature tile would leave the upper half
// of every MMA on padding and, with its 4.3 KB stages, only two thread blocks of three stages
// per SM).  tile j (j = 0..3): m = g <-> feature F + 8g + j,  m = g + 8 <-> F + 8g + 4 + j: one
// 128-bit load per B row, 4 MMAs per block pair.  Stage: 16 rows of 128 bytes (chunk c of row r
// at c ^ (r & 7)) plus the two blocks, 2304 bytes; four stages, three thread blocks per SM.
// ---------------------------------------------------------------------------------------------
template <int D>
struct H16MidCfg {
  static constexpr int kStage = 16 * 128 + 256;
  static constexpr int kSmem = kWarps * D * kStage;
};

template <bool BF16, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_16bit_mid_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                           const uint16_t* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                           const uint16_t* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                           int tiles, int rows_per_warp) {
  using Cfg = H16MidCfg<D>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * kWarps + warp;
  int64_t grp;
  int tile;
  split_work(work, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 64;
  uint8_t* ring = smem_raw + warp * (D * Cfg::kStage);
  const uint32_t ring_u32 = smem_u32(ring);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  int ir = 0;
  int64_t ib = row_start(0), ire = row_start(1);
  while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
  int slot_in = 0;
  const int cc = lane & 7, rr = lane >> 3;      // chunk of a 128-byte row, row within a group of four
  const bool in = F + 8 * cc < N;

  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      const bool two = b + 1 < ire;
      if (b + 1 >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J0 = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const int J1 = __shfl_sync(0xffffffffu, my_idx, (int)(b + 1 - win));
      const uint32_t dst = ring_u32 + slot_in * Cfg::kStage;
      const uint16_t* s0 = B + (int64_t)J0 * 8 * ldb + F + (in ? 8 * cc : 0);
      const uint16_t* s1 = B + (int64_t)(two ? J1 : J0) * 8 * ldb + F + (in ? 8 * cc : 0);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = 4 * i + rr;
        const uint32_t off = r * 128 + ((cc ^ r) << 4);
        cp_async16(dst + off, s0 + (int64_t)r * ldb, in ? 16 : 0);
        cp_async16(dst + 8 * 128 + off, s1 + (int64_t)r * ldb, (in && two) ? 16 : 0);
      }
      if (lane < 16)
        cp_async16(dst + 16 * 128 + lane * 16, blocks + (b + ((lane >= 8 && two) ? 1 : 0)) * 64 + (lane & 7) * 8,
                   (lane < 8 || two) ? 16 : 0);
      ib = two ? b + 2 : b + 1;
      while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
      slot_in = slot_in + 1 == D ? 0 : slot_in + 1;
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  const int rd0 = (2 * t) * 128 + (((g ^ (2 * t)) & 7) << 4);
  const int rd1 = (2 * t + 1) * 128 + (((g ^ (2 * t + 1)) & 7) << 4);

  int slot_out = 0;
  for (int r = 0; r < R; ++r) {
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; b += 2) {
      cp_async_wait<D - 2>();
      __syncwarp();
      issue_next();

      const uint8_t* st = ring + slot_out * Cfg::kStage;
      slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(st + 16 * 128 + (g * 8 + 2 * t) * 2);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(st + 16 * 128 + 128 + (g * 8 + 2 * t) * 2);
      const uint4 v0 = *reinterpret_cast<const uint4*>(st + rd0);             // block 0, column 2t: features 8g .. 8g+7
      const uint4 v1 = *reinterpret_cast<const uint4*>(st + rd1);             // block 0, column 2t+1
      const uint4 v2 = *reinterpret_cast<const uint4*>(st + 8 * 128 + rd0);   // block 1, column 2t
      const uint4 v3 = *reinterpret_cast<const uint4*>(st + 8 * 128 + rd1);   // block 1, column 2t+1
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
        auto lo = [&](const uint4& u) { return j < 2 ? u.x : u.y; };   // features 8g + j
        auto hi = [&](const uint4& u) { return j < 2 ? u.z : u.w; };   // features 8g + 4 + j
        uint32_t a[4];
        a[0] = __byte_perm(lo(v0), lo(v1), sel);   // m = g,   k = 2t, 2t+1
        a[1] = __byte_perm(hi(v0), hi(v1), sel);   // m = g+8, k = 2t, 2t+1
        a[2] = __byte_perm(lo(v2), lo(v3), sel);   // m = g,   k = 2t+8, 2t+9
        a[3] = __byte_perm(hi(v2), hi(v3), sel);   // m = g+8, k = 2t+8, 2t+9
        mma_16bit<BF16>(acc[j], a, b0, b1);
      }
    }

    if (F + 8 * g < N) {
      float* c0 = C + ((I0 + r - block_row_begin) * 8 + 2 * t) * ldc + F + 8 * g;
      float* c1 = c0 + ldc;
      __stcs(reinterpret_cast<float4*>(c0), make_float4(acc[0][0], acc[1][0], acc[2][0], acc[3][0]));
      __stcs(reinterpret_cast<float4*>(c0 + 4), make_float4(acc[0][2], acc[1][2], acc[2][2], acc[3][2]));
      __stcs(reinterpret_cast<float4*>(c1), make_float4(acc[0][1], acc[1][1], acc[2][1], acc[3][1]));
      __stcs(reinterpret_cast<float4*>(c1 + 4), make_float4(acc[0][3], acc[1][3], acc[2][3], acc[3][3]));
    }
  }
  cp_async_wait<0>();
}

// tuning state of the block kernels (lf_bsr_set_tuning)
int g_bsr_feat_units = 0;   // 0 = automatic, 1 or 2 = features per warp / 64 of the float32 kernel
int g_bsr_stages = 0;       // 0 = automatic, 3 or 4 = depth of the per-warp copy ring
int g_bsr_rows_per_warp = 0;  // 0 = automatic (4 float32, 8 16-bit); block rows one warp streams through, 1..31

int check_common(const void* indptr, const void* indices, const void* blocks, int64_t r0, int64_t r1,
                 const void* B, int64_t ldb, const void* C, int64_t ldc, int N, int feat_align) {
  LF_REQUIRE(indptr && B && C, "null pointer argument");
  LF_REQUIRE(0 <= r0 && r0 <= r1, "bad block-row range");
  // a matrix without any block has no block arrays (NULL): the product is a zero C
  LF_REQUIRE(N >= 1 && ldb >= N && ldc >= N && ldb < (1ll << 31), "bad dense operands");
  if (N % feat_align != 0 || ldb % feat_align != 0 || ldc % 4 != 0 || (uintptr_t)B % 16 != 0 ||
      (uintptr_t)C % 16 != 0 || (uintptr_t)blocks % 16 != 0)
    return fail(LF_ERR_UNSUPPORTED,
                "the 8x8 block kernel needs N and ldb to be multiples of %d elements, ldc a multiple of 4 and "
                "16-byte aligned blocks, B and C (use the composed-format or CSR entry points otherwise)", feat_align);
  return LF_OK;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  LF_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return LF_OK;
}

}  // namespace

// 0 = automatic, 1 = per-lane cp.async, 2 = tiled bulk copies, 3 = one bulk copy per B row
// (LF_OPT_BSR_COPY_ENGINE)
int g_bsr_copy_engine = 0;
// 0 = automatic (one after the other from four feature tiles on), 1 = the feature tiles of a block
// row together, 2 = one tile after the other (LF_OPT_BSR_TILE_ORDER)
int g_bsr_tile_order = 0;
// thread-block pipeline: blocks per stage * 10 + stages (0 = default), and whether one 3-D tiled
// copy per block may be used (1) or one 2-D copy per feature slice (0)
int g_bsr_pipe_shape = 0;
// warps per thread block of the cp.async-ring kernels for more than 64 features (LF_OPT_BSR_BLOCK_WARPS)
int g_bsr_block_warps = 0;
static int block_warps(int automatic) { return g_bsr_block_warps ? g_bsr_block_warps : automatic; }
int g_bsr_pipe_3d = 1;
// tcgen05 path: who fills shared memory: 0 one warp issuing tiled bulk copies, 2 / 4 that many warps issuing cp.async
int g_bsr_umma_producer = 0;

namespace {
int copy_engine() {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("LF_BSR_COPY_ENGINE");
    env = e ? atoi(e) : 0;
  }
  const int v = g_bsr_copy_engine ? g_bsr_copy_engine : env;
  return v >= 1 && v <= 5 ? v : kDefaultCopyEngine;
}
// A block matrix that holds no block at all (the caller passes no block arrays): C = 0.
int clear_c(float* C, int64_t ldc, int N, int64_t rows, cudaStream_t st) {
  LF_CUDA_CHECK(cudaMemset2DAsync(C, sizeof(float) * ldc, 0, sizeof(float) * N, (size_t)rows, st));
  return LF_OK;
}
}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

int lf_bsr_set_tuning(int32_t feat_units, int32_t stages, int32_t rows_per_warp) {
  LF_REQUIRE(feat_units >= 0 && feat_units <= 2 && (stages == 0 || stages == 3 || stages == 4) &&
                 rows_per_warp >= 0 && rows_per_warp <= 31, "bad tuning values");
  g_bsr_feat_units = feat_units;
  g_bsr_stages = stages;
  g_bsr_rows_per_warp = rows_per_warp;
  return LF_OK;
}

int lf_bsr_copy_status(void* stream) {
  int n = 0, m = 0;
  if (int s = bsr8_tma_timeouts((cudaStream_t)stream, &n)) return s;
  if (int s = bsr8_pipe_timeouts((cudaStream_t)stream, &m)) return s;
  n += m;
  if (int s = bsr8_umma_timeouts((cudaStream_t)stream, &m)) return s;
  n += m;
  if (n) return fail(LF_ERR_KERNEL_TIMEOUT, "%d warps of a block kernel gave up waiting for a copy", n);
  return LF_OK;
}

int lf_spmm_bsr8_f32(const int64_t* indptr, const int32_t* indices, const float* blocks,
                     int64_t block_row_begin, int64_t block_row_end, const float* B, int64_t ldb,
                     float* C, int64_t ldc, int32_t N, void* stream) {
  if (int s = check_common(indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N, 4)) return s;
  if (block_row_begin == block_row_end) return LF_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (!indices || !blocks) {
    LF_REQUIRE(!indices && !blocks, "one of the block arrays is missing");
    return clear_c(C, ldc, N, (block_row_end - block_row_begin) * 8, st);
  }
  const int64_t rows = block_row_end - block_row_begin;
  const int T = g_bsr_feat_units ? g_bsr_feat_units : (N > 64 ? 2 : 1);
  const int D = g_bsr_stages ? g_bsr_stages : (T == 2 ? 3 : 4);
  const int tiles = (N + 64 * T - 1) / (64 * T);
  const int rpw = g_bsr_rows_per_warp ? g_bsr_rows_per_warp : 4;
  const int64_t groups = ceil_div64(rows, rpw);
  const int64_t grid = ceil_div64(groups * tiles, kWarps);
  // measured on the banded benchmark matrix: no difference up to three tiles (N <= 384), 10 %
  // faster with four (N = 512), where the B rows of all tiles together no longer fit the L2
  const int64_t tile_major = (g_bsr_tile_order == 0 ? tiles > 3 : g_bsr_tile_order == 2) ? groups : 0;
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  if (N <= 32 && !g_bsr_feat_units) {   // narrow tile: both halves of every MMA carry features
    const int ntiles = (N + 31) / 32;
    const int64_t ngrid = ceil_div64(groups * ntiles, kWarps);
    auto k = bsr8_spmm_f32_narrow_kernel<6, 3>;
    if (int s = set_smem(k, F32NarrowCfg<6>::kSmem)) return s;
    k<<<(unsigned)ngrid, kThreadsBsr, F32NarrowCfg<6>::kSmem, st>>>(indptr, indices, blocks, block_row_begin,
                                                                    block_row_end, B, (int)ldb, C, ldc, N, ntiles, rpw);
    LF_CUDA_CHECK(cudaGetLastError());
    return LF_OK;
  }
  if ((copy_engine() == 4 || copy_engine() == 5) && N > 32)
    return bsr8_f32_pipe_launch(indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N,
                                g_bsr_pipe_shape, g_bsr_rows_per_warp, (N + 127) / 128 > 3 ? g_bsr_tile_order != 1 : g_bsr_tile_order == 2,
                                g_bsr_pipe_3d != 0, st);
  if (T == 2 && (copy_engine() == 2 || copy_engine() == 3))
    return bsr8_f32_tma_launch(copy_engine() == 3, indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N, D, rpw,
                               tile_major > 0, st);
  const int W = block_warps(8);   // float32: no gain from smaller thread blocks (0.92 / 0.95 ms at N = 128)
  const int64_t wgrid = ceil_div64(groups * tiles, W);
  LF_REQUIRE(wgrid < (1ll << 31), "too many thread blocks");
#define LF_BSR(T_, D_, M_)                                                                                   \
  do {                                                                                                       \
    auto k = bsr8_spmm_f32_kernel<T_, D_, M_>;                                                               \
    const int smem = W * D_ * F32Cfg<T_, D_>::kStage;                                                        \
    if (int s = set_smem(k, smem)) return s;                                                                 \
    k<<<(unsigned)wgrid, W * 32, smem, st>>>(indptr, indices, blocks, block_row_begin, block_row_end, B,    \
                                             (int)ldb, C, ldc, N, tiles, rpw, tile_major);                   \
  } while (0)
  if (T == 2) { if (D == 3) LF_BSR(2, 3, 2); else LF_BSR(2, 4, 1); }
  else        { if (D == 3) LF_BSR(1, 3, 3); else LF_BSR(1, 4, 3); }
#undef LF_BSR
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

static int launch_16bit(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                        int64_t r0, int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int32_t N,
                        void* stream) {
  if (int s = check_common(indptr, indices, blocks, r0, r1, B, ldb, C, ldc, N, 8)) return s;
  if (r0 == r1) return LF_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (!indices || !blocks) {
    LF_REQUIRE(!indices && !blocks, "one of the block arrays is missing");
    return clear_c(C, ldc, N, (r1 - r0) * 8, st);
  }
  const int tiles = (N + 127) / 128;
  const int rpw = g_bsr_rows_per_warp ? g_bsr_rows_per_warp : 8;
  const int64_t grid = ceil_div64(ceil_div64(r1 - r0, rpw) * tiles, kWarps);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  const int D = g_bsr_stages ? g_bsr_stages : 3;
  if (N <= 32 && !g_bsr_stages) {   // narrow tile: both halves of every MMA carry features
    const int ntiles = (N + 31) / 32;
    const int64_t ngrid = ceil_div64(ceil_div64(r1 - r0, rpw) * ntiles, kWarps);
    if (bf16) {
      auto k = bsr8_spmm_16bit_narrow_kernel<true, 6, 3>;
      if (int s = set_smem(k, H16NarrowCfg<6>::kSmem)) return s;
      k<<<(unsigned)ngrid, kThreadsBsr, H16NarrowCfg<6>::kSmem, st>>>(indptr, indices, blocks, r0, r1, B, (int)ldb, C,
                                                                      ldc, N, ntiles, rpw);
    } else {
      auto k = bsr8_spmm_16bit_narrow_kernel<false, 6, 3>;
      if (int s = set_smem(k, H16NarrowCfg<6>::kSmem)) return s;
      k<<<(unsigned)ngrid, kThreadsBsr, H16NarrowCfg<6>::kSmem, st>>>(indptr, indices, blocks, r0, r1, B, (int)ldb, C,
                                                                      ldc, N, ntiles, rpw);
    }
    LF_CUDA_CHECK(cudaGetLastError());
    return LF_OK;
  }
  if (N <= 64 && !g_bsr_stages) {   // 64 features per warp
    const int64_t ngrid = ceil_div64(ceil_div64(r1 - r0, rpw), kWarps);
    if (bf16) {
      auto k = bsr8_spmm_16bit_mid_kernel<true, 4, 3>;
      if (int s = set_smem(k, H16MidCfg<4>::kSmem)) return s;
      k<<<(unsigned)ngrid, kThreadsBsr, H16MidCfg<4>::kSmem, st>>>(indptr, indices, blocks, r0, r1, B, (int)ldb, C, ldc,
                                                                   N, 1, rpw);
    } else {
      auto k = bsr8_spmm_16bit_mid_kernel<false, 4, 3>;
      if (int s = set_smem(k, H16MidCfg<4>::kSmem)) return s;
      k<<<(unsigned)ngrid, kThreadsBsr, H16MidCfg<4>::kSmem, st>>>(indptr, indices, blocks, r0, r1, B, (int)ldb, C, ldc,
                                                                   N, 1, rpw);
    }
    LF_CUDA_CHECK(cudaGetLastError());
    return LF_OK;
  }
  if (copy_engine() == 5)
    return bsr8_16bit_umma_launch(bf16, indptr, indices, blocks, r0, r1, B, ldb, C, ldc, N, g_bsr_pipe_shape,
                                  g_bsr_rows_per_warp, g_bsr_pipe_3d != 0, g_bsr_umma_producer, st);
  if (copy_engine() == 4)
    return bsr8_16bit_pipe_launch(bf16, indptr, indices, blocks, r0, r1, B, ldb, C, ldc, N, g_bsr_pipe_shape,
                                  g_bsr_rows_per_warp, g_bsr_pipe_3d != 0, st);
  if (copy_engine() == 2 || copy_engine() == 3) return bsr8_16bit_tma_launch(copy_engine() == 3, bf16, indptr, indices, blocks, r0, r1, B, ldb, C, ldc, N, D, rpw, st);
  // Warps per thread block: the ring of a warp takes D stages of shared memory, so smaller thread
  // blocks pack the SM in finer steps (four blocks of four warps instead of two of eight) and
  // leave and enter it in smaller units.  Measured on the banded benchmark matrix (bf16, 8 / 4
  // warps): N = 128 0.532 / 0.516 ms, N = 256 1.039 / 1.050 ms, N = 512 2.219 / 2.348 ms.
  const int W = block_warps(tiles == 1 ? 4 : 8);
  const int64_t wgrid = ceil_div64(ceil_div64(r1 - r0, rpw) * tiles, W);
  LF_REQUIRE(wgrid < (1ll << 31), "too many thread blocks");
#define LF_BSR16(B_, D_, M_)                                                                                  \
  do {                                                                                                        \
    auto k = bsr8_spmm_16bit_kernel<B_, D_, M_>;                                                              \
    const int smem = W * D_ * H16Cfg<D_>::kStage;                                                             \
    if (int s = set_smem(k, smem)) return s;                                                                  \
    k<<<(unsigned)wgrid, W * 32, smem, st>>>(indptr, indices, blocks, r0, r1, B, (int)ldb, C, ldc, N, tiles, rpw); \
  } while (0)
  if (bf16) { if (D == 3) LF_BSR16(true, 3, 2); else LF_BSR16(true, 4, 1); }
  else      { if (D == 3) LF_BSR16(false, 3, 2); else LF_BSR16(false, 4, 1); }
#undef LF_BSR16
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

int lf_spmm_bsr8_bf16(const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                      int64_t block_row_begin, int64_t block_row_end, const uint16_t* B, int64_t ldb,
                      float* C, int64_t ldc, int32_t N, void* stream) {
  return launch_16bit(true, indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N, stream);
}

int lf_spmm_bsr8_f16(const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                     int64_t block_row_begin, int64_t block_row_end, const uint16_t* B, int64_t ldb,
                     float* C, int64_t ldc, int32_t N, void* stream) {
  return launch_16bit(false, indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N, stream);
}

}  // extern "C"
