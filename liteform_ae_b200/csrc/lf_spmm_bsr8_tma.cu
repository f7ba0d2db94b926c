// C = A @ B for A in 8x8 block-sparse rows: the variant whose B rows and A blocks travel into
// shared memory through the tensor memory accelerator instead of per-lane cp.async.
//
// Work split, index maps and the MMA sequence are those of the cp.async kernels
// (lf_spmm_bsr8.cu): a warp streams the blocks of a few consecutive block rows through a private
// ring of D stages.  What changes is who moves the bytes:
//   * B: one tiled 2-D copy (cp.async.bulk.tensor.2d) per box of 8 rows x 128 bytes, swizzle mode
//     128B, so that chunk c (16 bytes) of row r lands at chunk c ^ r of its row: the same
//     conflict-free pattern the cp.async kernels build by hand.  One elected lane issues the
//     four boxes of a stage; no lane computes addresses or spends LSU wavefronts on the copy.
//   * A: one untiled bulk copy (cp.async.bulk) of the 256-byte block (pair).
//   * completion: one mbarrier per stage, armed with the byte count of the stage
//     (arrive.expect_tx) and waited on by parity.  Every wait is bounded: a warp that gives up
//     records it in a device flag, still waits (bounded again) for the copies it has in flight,
//     and returns; lf_bsr_copy_status reports the flag to the host.
// The tensor map describes B as it lies in memory ({N, rows} with the row pitch ldb); features
// beyond N read as zeros (out-of-bounds fill), so no lane masks the tail.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "lf_bsr8_mma.cuh"
#include "lf_bsr8_tma.cuh"
#include "lf_common.cuh"

namespace lf {
namespace {

using namespace bsr8;

__device__ int g_copy_timeouts;   // number of warps that gave up waiting for a stage

constexpr long long kWaitCycles = 2000000000ll;   // about a second at the boost clock

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// false when the phase did not complete within kWaitCycles
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - t0 > kWaitCycles) return false;
  return true;
}
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Shared memory of one thread block: [warp][stage] B data (DATA bytes: four swizzled 1024-byte
// boxes, or the pitched rows; the region starts on a 1024-byte boundary so that the swizzle of a
// box depends on the row only), then [warp][stage] A blocks (256 bytes), then [warp][stage]
// mbarriers.
template <int D, int DATA>
struct TmaCfg {
  static constexpr int kData = DATA;
  static constexpr int kOffA = kWarps * D * kData;
  static constexpr int kOffBar = kOffA + kWarps * D * 256;
  static constexpr int kSmem = kOffBar + kWarps * D * 8 + 1024;   // + slack for the alignment
};

// What both kernels share: the warp's ring, its barriers and the bounded wait / drain logic.
template <int D, int DATA>
struct Ring {
  using Cfg = TmaCfg<D, DATA>;
  uint32_t data, blk, bar;   // shared-memory addresses of stage 0
  const uint8_t* data_ptr;
  const uint8_t* blk_ptr;
  int slot_in = 0, slot_out = 0, in_flight = 0;
  uint32_t parity = 0;

  __device__ __forceinline__ Ring(uint8_t* raw, int warp, int lane) {
    const uint32_t raw_u32 = smem_u32(raw);
    const uint32_t pad = ((raw_u32 + 1023u) & ~1023u) - raw_u32;
    uint8_t* base = raw + pad;
    data_ptr = base + warp * (D * Cfg::kData);
    blk_ptr = base + Cfg::kOffA + warp * (D * 256);
    data = smem_u32(data_ptr);
    blk = smem_u32(blk_ptr);
    bar = smem_u32(base + Cfg::kOffBar + warp * (D * 8));
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < D; ++s) mbar_init(bar + 8 * s, 1);
      mbar_fence_init();
    }
    __syncwarp();
  }
  __device__ __forceinline__ void advance_in() { slot_in = slot_in + 1 == D ? 0 : slot_in + 1; ++in_flight; }
  // waits for the oldest stage; false after a timeout (recorded)
  __device__ __forceinline__ bool wait_oldest(int lane) {
    const bool ok = mbar_wait_bounded(bar + 8 * slot_out, parity);
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0) atomicAdd(&g_copy_timeouts, 1);
      return false;
    }
    return true;
  }
  __device__ __forceinline__ int pop() {
    const int s = slot_out;
    slot_out = slot_out + 1 == D ? 0 : slot_out + 1;
    if (slot_out == 0) parity ^= 1u;
    --in_flight;
    return s;
  }
  // after a timeout: give the copies still in flight a bounded chance to land before the warp
  // (and with it, perhaps, the thread block and its shared memory) goes away
  __device__ __forceinline__ void drain() {
    while (in_flight > 0) {
      mbar_wait_bounded(bar + 8 * slot_out, parity);
      pop();
    }
  }
};

// Two ways to lay a stage out, chosen by ROWS:
//   ROWS = false  tiled copies.  Box 2q + h (1024 bytes) = the 8 rows x features F + 64q + 32h .. + 31,
//                 swizzled; a lane finds (row, 16-byte chunk c) of a box at row * 128 + ((c ^ row) << 4).
//   ROWS = true   one untiled bulk copy per B row (512 bytes float32, 256 bytes 16-bit), rows kept
//                 16 bytes apart from a multiple of 128 (pitch 528 / 272), which spreads the four
//                 rows a quarter-warp reads over all banks; no tensor map is needed.
struct F32Layout {
  static constexpr int kTiledData = 4 * 1024;
  static constexpr int kRowPitch = 512 + 16;
  static constexpr int kRowsData = 8 * kRowPitch;
};
struct H16Layout {
  static constexpr int kTiledData = 4 * 1024;
  static constexpr int kRowPitch = 256 + 16;
  static constexpr int kRowsData = 16 * kRowPitch;
};

// ---------------------------------------------------------------------------------------------
// float32, 3xTF32, 128 features per warp; half h of unit q feeds MMA rows m = g + 8h.
// ---------------------------------------------------------------------------------------------
template <bool ROWS, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_f32_tma_kernel(const __grid_constant__ CUtensorMap mapB, const int64_t* __restrict__ indptr,
                         const int32_t* __restrict__ indices, const float* __restrict__ blocks,
                         int64_t block_row_begin, int64_t block_row_end, const float* __restrict__ B, int ldb,
                         float* __restrict__ C, int64_t ldc, int N, int tiles, int rows_per_warp,
                         int64_t tile_major_groups) {
  constexpr int kData = ROWS ? F32Layout::kRowsData : F32Layout::kTiledData;
  constexpr int kPitch = ROWS ? F32Layout::kRowPitch : 128;   // bytes between the rows a lane reads
  constexpr int kHalf = ROWS ? 128 : 1024;                     // bytes between 32-feature halves
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * kWarps + warp;
  int64_t grp;
  int tile;
  split_work(work, tiles, tile_major_groups, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end || tile >= tiles) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 128;
  const int boxes = min(4, (N - F + 31) / 32);   // boxes past N feed only outputs nobody stores
  const uint32_t row_bytes = (uint32_t)min(128, N - F) * 4;   // ROWS: bytes of one B row inside N
  Ring<D, kData> ring(smem_raw, warp, lane);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  int64_t ib = row_start(0);

  auto issue_next = [&]() {
    if (ib < stream_end) {
      const int64_t b = ib;
      if (b >= win + 32) {
        win = b;
        my_idx = (b + lane < stream_end) ? indices[b + lane] : 0;
      }
      const int J = __shfl_sync(0xffffffffu, my_idx, (int)(b - win));
      const uint32_t bar = ring.bar + 8 * ring.slot_in;
      const uint32_t dst = ring.data + ring.slot_in * kData;
      if (ROWS) {
        if (lane == 0) mbar_expect_tx(bar, 8 * row_bytes + 256);
        __syncwarp();
        if (lane < 8) bulk_load(dst + lane * kPitch, B + ((int64_t)J * 8 + lane) * ldb + F, row_bytes, bar);
        if (lane == 8) bulk_load(ring.blk + ring.slot_in * 256, blocks + b * 64, 256, bar);
      } else if (lane == 0) {
        mbar_expect_tx(bar, boxes * 1024 + 256);
        for (int bx = 0; bx < boxes; ++bx) tma_load_box(dst + bx * 1024, &mapB, F + 32 * bx, J * 8, bar);
        bulk_load(ring.blk + ring.slot_in * 256, blocks + b * 64, 256, bar);
      }
      ib = b + 1;
      ring.advance_in();
    }
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  for (int r = 0; r < R; ++r) {
    float acc[2][4][4];
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[q][j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; ++b) {
      if (!ring.wait_oldest(lane)) {
        ring.drain();
        return;
      }
      __syncwarp();
      issue_next();   // refills the stage consumed in the previous iteration

      const int s = ring.pop();
      const uint8_t* st = ring.data_ptr + s * kData;
      const float2 av = *reinterpret_cast<const float2*>(ring.blk_ptr + s * 256 + (g * 8 + 2 * t) * 4);
      uint32_t b0h, b0l, b1h, b1l;
      split_tf32(av.x, b0h, b0l);
      split_tf32(av.y, b1h, b1l);
      const uint8_t* row0 = st + (2 * t) * kPitch + ((ROWS ? g : (g ^ (2 * t)) & 7) << 4);
      const uint8_t* row1 = st + (2 * t + 1) * kPitch + ((ROWS ? g : (g ^ (2 * t + 1)) & 7) << 4);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const float4 x0 = *reinterpret_cast<const float4*>(row0 + (2 * q) * kHalf);       // k = t,   m = g
        const float4 x1 = *reinterpret_cast<const float4*>(row0 + (2 * q + 1) * kHalf);   // k = t,   m = g+8
        const float4 y0 = *reinterpret_cast<const float4*>(row1 + (2 * q) * kHalf);       // k = t+4, m = g
        const float4 y1 = *reinterpret_cast<const float4*>(row1 + (2 * q + 1) * kHalf);   // k = t+4, m = g+8
        const float a_f[4][4] = {{x0.x, x1.x, y0.x, y1.x}, {x0.y, x1.y, y0.y, y1.y},
                                 {x0.z, x1.z, y0.z, y1.z}, {x0.w, x1.w, y0.w, y1.w}};
        uint32_t ah[4][4], al[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) split_tf32(a_f[j][i], ah[j][i], al[j][i]);
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
    for (int q = 0; q < 2; ++q) {
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
}

// ---------------------------------------------------------------------------------------------
// 16-bit in (bf16 or fp16), 128 features per warp, two blocks per MMA.  Tiled stage: box
// 2 * blk + h = rows of block blk, features F + 64h .. + 63; row-wise stage: row 8 * blk + r.  The
// last pair of an odd row has no second block: nothing is copied for it and the lanes feed zeros.
// ---------------------------------------------------------------------------------------------
template <bool ROWS, bool BF16, int D, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_16bit_tma_kernel(const __grid_constant__ CUtensorMap mapB, const int64_t* __restrict__ indptr,
                           const int32_t* __restrict__ indices, const uint16_t* __restrict__ blocks,
                           int64_t block_row_begin, int64_t block_row_end, const uint16_t* __restrict__ B, int ldb,
                           float* __restrict__ C, int64_t ldc, int N, int tiles, int rows_per_warp) {
  constexpr int kData = ROWS ? H16Layout::kRowsData : H16Layout::kTiledData;
  constexpr int kPitch = ROWS ? H16Layout::kRowPitch : 128;   // bytes between the rows a lane reads
  constexpr int kHalf = ROWS ? 128 : 1024;                     // bytes between 64-feature halves
  constexpr int kBlk = ROWS ? 8 * H16Layout::kRowPitch : 2048; // bytes between the two blocks of a pair
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3, warp = threadIdx.x >> 5;
  const int64_t work = (int64_t)blockIdx.x * kWarps + warp;
  int64_t grp;
  int tile;
  split_work(work, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_warp;
  if (I0 >= block_row_end) return;
  const int R = (int)min((int64_t)rows_per_warp, block_row_end - I0);
  const int F = tile * 128;
  const int halves = min(2, (N - F + 63) / 64);
  const uint32_t row_bytes = (uint32_t)min(128, N - F) * 2;   // ROWS: bytes of one B row inside N
  Ring<D, kData> ring(smem_raw, warp, lane);

  const int64_t my_ptr = indptr[I0 + min(lane, R)];
  const int64_t stream_end = __shfl_sync(0xffffffffu, my_ptr, R);
  auto row_start = [&](int r) { return __shfl_sync(0xffffffffu, my_ptr, r); };

  int my_idx = 0;
  int64_t win = -(int64_t)64;
  int ir = 0;
  int64_t ib = row_start(0), ire = row_start(1);
  while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }

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
      const uint32_t bar = ring.bar + 8 * ring.slot_in;
      const uint32_t dst = ring.data + ring.slot_in * kData;
      if (ROWS) {
        if (lane == 0) mbar_expect_tx(bar, (two ? 2 : 1) * (8 * row_bytes + 128));
        __syncwarp();
        if (lane < (two ? 16 : 8))
          bulk_load(dst + lane * kPitch, B + ((int64_t)(lane < 8 ? J0 : J1) * 8 + (lane & 7)) * ldb + F, row_bytes, bar);
        if (lane == 16) bulk_load(ring.blk + ring.slot_in * 256, blocks + b * 64, two ? 256 : 128, bar);
      } else if (lane == 0) {
        mbar_expect_tx(bar, (two ? 2 : 1) * (halves * 1024 + 128));
        for (int h = 0; h < halves; ++h) tma_load_box(dst + h * 1024, &mapB, F + 64 * h, J0 * 8, bar);
        if (two)
          for (int h = 0; h < halves; ++h) tma_load_box(dst + (2 + h) * 1024, &mapB, F + 64 * h, J1 * 8, bar);
        bulk_load(ring.blk + ring.slot_in * 256, blocks + b * 64, two ? 256 : 128, bar);
      }
      ib = two ? b + 2 : b + 1;
      while (ib == ire && ir + 1 < R) { ++ir; ire = row_start(ir + 1); }
      ring.advance_in();
    }
  };

#pragma unroll
  for (int s = 0; s < D - 1; ++s) issue_next();

  for (int r = 0; r < R; ++r) {
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    const int64_t be = row_start(r + 1);
    for (int64_t b = row_start(r); b < be; b += 2) {
      if (!ring.wait_oldest(lane)) {
        ring.drain();
        return;
      }
      __syncwarp();
      issue_next();

      const int s = ring.pop();
      const bool two = b + 1 < be;
      const uint8_t* st = ring.data_ptr + s * kData;
      const uint8_t* ab = ring.blk_ptr + s * 256 + (g * 8 + 2 * t) * 2;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(ab);
      const uint32_t b1 = two ? *reinterpret_cast<const uint32_t*>(ab + 128) : 0u;
      const uint8_t* row0 = st + (2 * t) * kPitch + ((ROWS ? g : (g ^ (2 * t)) & 7) << 4);
      const uint8_t* row1 = st + (2 * t + 1) * kPitch + ((ROWS ? g : (g ^ (2 * t + 1)) & 7) << 4);
      // [row][half]: rows = (blk0 col 2t), (blk0 col 2t+1), (blk1 col 2t), (blk1 col 2t+1)
      uint4 v[4][2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        v[0][h] = *reinterpret_cast<const uint4*>(row0 + h * kHalf);
        v[1][h] = *reinterpret_cast<const uint4*>(row1 + h * kHalf);
        v[2][h] = two ? *reinterpret_cast<const uint4*>(row0 + kBlk + h * kHalf) : make_uint4(0, 0, 0, 0);
        v[3][h] = two ? *reinterpret_cast<const uint4*>(row1 + kBlk + h * kHalf) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
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
    for (int h = 0; h < 2; ++h) {
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
}

// ---- host side ---------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's encoder, looked up through the runtime (the library does not link libcuda).
EncodeTiledFn encode_tiled_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> lock(mu);
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// B as a 2-D tensor {N features, rows} with pitch ldb; boxes of 8 rows x 128 bytes.  The number of
// rows of B is not an argument of the product (A's block columns index it), so the map claims the
// largest row count whose last row still has a 32-bit coordinate; a copy touches only the rows
// its coordinates name.
int make_b_map(CUtensorMap* map, const void* B, int64_t ldb, int N, int elem_bytes) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(LF_ERR_UNSUPPORTED, "the driver does not export cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)1 << 31};
  const cuuint64_t strides[1] = {(cuuint64_t)ldb * elem_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), 8};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                         const_cast<void*>(B), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LF_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return LF_OK;
}

template <typename K>
int set_smem(K kernel, int bytes) {
  LF_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return LF_OK;
}

}  // namespace

int bsr8_f32_tma_launch(bool rows, const int64_t* indptr, const int32_t* indices, const float* blocks, int64_t r0,
                        int64_t r1, const float* B, int64_t ldb, float* C, int64_t ldc, int N, int stages,
                        int rows_per_warp, bool tile_major, cudaStream_t st) {
  CUtensorMap map = {};
  if (!rows)
    if (int s = make_b_map(&map, B, ldb, N, 4)) return s;
  const int tiles = (N + 127) / 128;
  const int64_t groups = ceil_div64(r1 - r0, rows_per_warp);
  const int64_t grid = ceil_div64(groups * tiles, kWarps);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  const int64_t tm = tile_major ? groups : 0;
#define LF_TMA32(R_, D_, M_, DATA_)                                                                              \
  do {                                                                                                           \
    auto k = bsr8_spmm_f32_tma_kernel<R_, D_, M_>;                                                               \
    constexpr int smem = TmaCfg<D_, DATA_>::kSmem;                                                               \
    if (int s = set_smem(k, smem)) return s;                                                                     \
    k<<<(unsigned)grid, kThreadsBsr, smem, st>>>(map, indptr, indices, blocks, r0, r1, B, (int)ldb, C, ldc, N,   \
                                                 tiles, rows_per_warp, tm);                                      \
  } while (0)
  if (rows) { if (stages == 4) LF_TMA32(true, 4, 1, F32Layout::kRowsData); else LF_TMA32(true, 3, 2, F32Layout::kRowsData); }
  else      { if (stages == 4) LF_TMA32(false, 4, 1, F32Layout::kTiledData); else LF_TMA32(false, 3, 2, F32Layout::kTiledData); }
#undef LF_TMA32
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

int bsr8_16bit_tma_launch(bool rows, bool bf16, const int64_t* indptr, const int32_t* indices,
                          const uint16_t* blocks, int64_t r0, int64_t r1, const uint16_t* B, int64_t ldb, float* C,
                          int64_t ldc, int N, int stages, int rows_per_warp, cudaStream_t st) {
  CUtensorMap map = {};
  if (!rows)
    if (int s = make_b_map(&map, B, ldb, N, 2)) return s;
  const int tiles = (N + 127) / 128;
  const int64_t grid = ceil_div64(ceil_div64(r1 - r0, rows_per_warp) * tiles, kWarps);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
#define LF_TMA16(R_, B_, D_, M_, DATA_)                                                                          \
  do {                                                                                                           \
    auto k = bsr8_spmm_16bit_tma_kernel<R_, B_, D_, M_>;                                                         \
    constexpr int smem = TmaCfg<D_, DATA_>::kSmem;                                                               \
    if (int s = set_smem(k, smem)) return s;                                                                     \
    k<<<(unsigned)grid, kThreadsBsr, smem, st>>>(map, indptr, indices, blocks, r0, r1, B, (int)ldb, C, ldc, N,   \
                                                 tiles, rows_per_warp);                                          \
  } while (0)
#define LF_TMA16_D(R_, B_, DATA_) \
  do { if (stages == 4) LF_TMA16(R_, B_, 4, 1, DATA_); else LF_TMA16(R_, B_, 3, 2, DATA_); } while (0)
  if (rows) { if (bf16) LF_TMA16_D(true, true, H16Layout::kRowsData); else LF_TMA16_D(true, false, H16Layout::kRowsData); }
  else      { if (bf16) LF_TMA16_D(false, true, H16Layout::kTiledData); else LF_TMA16_D(false, false, H16Layout::kTiledData); }
#undef LF_TMA16_D
#undef LF_TMA16
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

int bsr8_tma_timeouts(cudaStream_t st, int* count) {
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  int n = 0;
  LF_CUDA_CHECK(cudaMemcpyFromSymbol(&n, g_copy_timeouts, sizeof(int)));
  if (n) {
    const int zero = 0;
    LF_CUDA_CHECK(cudaMemcpyToSymbol(g_copy_timeouts, &zero, sizeof(int)));
  }
  *count = n;
  return LF_OK;
}

}  // namespace lf
