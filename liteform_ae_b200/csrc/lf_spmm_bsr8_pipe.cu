// C = A @ B for A in 8x8 block-sparse rows: the thread-block-wide pipeline.
//
// Takes over the kernel of the reference's bench_bsrmm (playground_pipline/format_algos.py:1562-1643;
// arithmetic format_algos.py:1204-1213).  Index maps of the MMAs and the shared-memory layout a
// consumer reads are those of the per-warp kernels (lf_spmm_bsr8.cu); what differs is who moves
// the bytes and how the work of a thread block is organised:
//
//   * one PRODUCER warp per thread block walks the blocks of a run of consecutive block rows and,
//     per block, issues ONE tiled bulk copy (cp.async.bulk.tensor through a tensor map over B):
//     the 8 rows of B the block needs, all feature slices of the thread block's tile at once, land
//     as swizzled 8 x 128-byte boxes ([slice][row][128 bytes], 16-byte chunk c of row r at c ^ r).
//     The A blocks of a stage are contiguous in memory and come with one untiled bulk copy.  No
//     lane computes copy addresses or spends load/store-unit slots on the copy;
//   * a stage holds up to SB blocks of ONE block row; stages form a ring of D; a stage is handed
//     to the consumers through an mbarrier armed with its byte count (arrive.expect_tx) and handed
//     back through a second mbarrier on which every consumer warp arrives once;
//   * NCW CONSUMER warps each own one feature slice (32 float32 or 64 16-bit features) of every
//     block: conflict-free 128-bit fragment loads from the swizzled boxes, mma.sync with fp32
//     accumulators kept across the stages of a block row, streaming float4 stores of C;
//   * producer and consumers derive the same stage sequence from the block-row pointers, so no
//     control word travels through shared memory.
// Per block the consumers execute about half the instructions of the per-warp kernels (no copy
// issue, no copy addressing, no per-block ring bookkeeping), which is what bounds those.
//
// Every wait is bounded (about a second); a warp that gives up raises a flag that makes all waits
// of its thread block return, the producer gives its copies in flight a bounded chance to land,
// and the host reads the count through lf_bsr_copy_status.  No copy uses cluster multicast and the
// tensor map covers memory of this GPU only.
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

__device__ int g_pipe_timeouts;   // thread blocks that gave up waiting for a stage

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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Waits for the phase with the given parity.  Returns false when the thread block is giving up:
// this wait ran out of time (it then raises `abort_flag`), or another warp already did.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Shared memory of one thread block (offsets from a 1024-byte aligned base):
//   [D][SB][NCW] boxes of 1024 bytes  (B rows; box = 8 rows x 128 bytes, swizzled)
//   [D][SB] A blocks of kABytes
//   [D] full barriers, [D] empty barriers, abort flag
template <int NCW, int SB, int D, int A_BYTES>
struct PipeCfg {
  static constexpr int kBlockB = NCW * 1024;
  static constexpr int kStageB = SB * kBlockB;
  static constexpr int kStageA = SB * A_BYTES;
  static constexpr int kOffA = D * kStageB;
  static constexpr int kOffBar = kOffA + D * kStageA;
  static constexpr int kSmem = kOffBar + 2 * D * 8 + 16 + 1024;   // + slack for the alignment
  static constexpr int kThreads = (NCW + 1) * 32;
};

// The stage sequence both sides walk: block rows I0 .. I0+R-1 in order, each cut into chunks of up
// to SB blocks; a block row without blocks is one empty stage (its rows of C still get written).
// lane l <= R holds row pointer I0 + l.
struct RowPtrs {
  int64_t mine;
  __device__ __forceinline__ int64_t at(int r) const { return __shfl_sync(0xffffffffu, mine, r); }
};

// ---------------------------------------------------------------------------------------------
// Producer: one warp.  Lane 0 issues the copies; all lanes keep a window of 32 block columns.
// boxes_per_block = 1: the tensor map is 3-D {features of a slice, rows, slices} and one copy
// brings all NCW slices of a block; = NCW: the map is 2-D {features, rows}, one copy per slice.
// ---------------------------------------------------------------------------------------------
template <typename Cfg, int NCW, int SB, int D, int A_BYTES, int ELEMS_PER_SLICE>
__device__ __forceinline__ void produce(const CUtensorMap* mapB, const RowPtrs& ptrs, int R,
                                        const int32_t* __restrict__ indices, const uint8_t* __restrict__ blocks,
                                        int tile, int boxes_per_block, uint32_t smem_base, volatile int* abort_flag,
                                        int lane) {
  const uint32_t bar_full = smem_base + Cfg::kOffBar, bar_empty = bar_full + D * 8;
  const int64_t stream_begin = ptrs.at(0), stream_end = ptrs.at(R);
  int64_t win = stream_begin;
  int idx_cur = (win + lane < stream_end) ? indices[win + lane] : 0;
  int idx_nxt = (win + 32 + lane < stream_end) ? indices[win + 32 + lane] : 0;
  int q = 0;          // stages armed so far: stage q uses slot q % D for the (q / D)-th time
  bool ok = true;
  for (int r = 0; r < R && ok; ++r) {
    int64_t b = ptrs.at(r);
    const int64_t be = ptrs.at(r + 1);
    do {
      const int n = (int)min((int64_t)SB, be - b);
      const int slot = q % D;
      const uint32_t round = (uint32_t)(q / D);
      if (round > 0) {   // the consumers must have released this slot
        ok = mbar_wait(bar_empty + 8 * slot, (round - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const uint32_t full = bar_full + 8 * slot;
      if (lane == 0) mbar_expect_tx(full, (uint32_t)n * (Cfg::kBlockB + A_BYTES));
      ++q;
      if (n > 0) {
        const uint32_t dstB = smem_base + slot * Cfg::kStageB;
        for (int k = 0; k < n; ++k) {
          if (b + k >= win + 32) {   // slide the window; the one after it is requested now
            win += 32;
            idx_cur = idx_nxt;
            idx_nxt = (win + 32 + lane < stream_end) ? indices[win + 32 + lane] : 0;
          }
          const int J = __shfl_sync(0xffffffffu, idx_cur, (int)(b + k - win));
          if (lane == 0) {
            if (boxes_per_block == 1) {
              tma_load_3d(dstB + k * Cfg::kBlockB, mapB, 0, J * 8, tile * NCW, full);
            } else {
#pragma unroll
              for (int s = 0; s < NCW; ++s)
                tma_load_2d(dstB + k * Cfg::kBlockB + s * 1024, mapB, (tile * NCW + s) * ELEMS_PER_SLICE, J * 8, full);
            }
          }
        }
        if (lane == 0)
          bulk_load(smem_base + Cfg::kOffA + slot * Cfg::kStageA, blocks + b * A_BYTES, (uint32_t)n * A_BYTES, full);
      }
      b += n;
    } while (b < be);
  }
  if (!ok) {
    // giving up: let the copies already issued land (bounded) before the shared memory goes away
    for (int p = q - 1; p >= 0 && p >= q - D; --p) {
      const long long t0 = clock64();
      while (!mbar_try_wait(bar_full + 8 * (p % D), (uint32_t)(p / D) & 1u) && clock64() - t0 < kWaitCycles) {}
    }
  }
}

// ---------------------------------------------------------------------------------------------
// float32 consumer: 32 features (one box per block), 3xTF32.  Lane (g = lane / 4, t = lane % 4);
//   k-slot t <-> block column 2t, k-slot t+4 <-> block column 2t+1;
//   MMA tile j (j = 0, 1): m = g <-> feature 4g + j,  m = g + 8 <-> feature 4g + 2 + j;
//   n <-> row of the block: a lane ends with C[row 2t / 2t+1][4 consecutive features].
// ---------------------------------------------------------------------------------------------
struct F32Consumer {
  static constexpr int kABytes = 256;
  static constexpr int kFeat = 32;
  float acc[2][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  }
  // boxes: first box of this warp's slice in the stage (stride between blocks: block_stride bytes)
  __device__ __forceinline__ void blocks(const uint8_t* box, int block_stride, const uint8_t* a_blocks, int n, int g, int t) {
    const int off0 = (2 * t) * 128 + (((g ^ (2 * t)) & 7) << 4);
    const int off1 = (2 * t + 1) * 128 + (((g ^ (2 * t + 1)) & 7) << 4);
#pragma unroll 4
    for (int k = 0; k < n; ++k) {
      const float2 av = *reinterpret_cast<const float2*>(a_blocks + k * 256 + (g * 8 + 2 * t) * 4);
      const float4 x = *reinterpret_cast<const float4*>(box + k * block_stride + off0);   // k = t
      const float4 y = *reinterpret_cast<const float4*>(box + k * block_stride + off1);   // k = t + 4
      uint32_t b0h, b0l, b1h, b1l;
      split_tf32(av.x, b0h, b0l);
      split_tf32(av.y, b1h, b1l);
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
  }
  __device__ __forceinline__ void store(float* c_row0, int64_t ldc, int F, int N, int g, int t) {
    if (F + 4 * g < N) {
      float* c0 = c_row0 + (2 * t) * ldc + F + 4 * g;
      __stcs(reinterpret_cast<float4*>(c0), make_float4(acc[0][0], acc[1][0], acc[0][2], acc[1][2]));
      __stcs(reinterpret_cast<float4*>(c0 + ldc), make_float4(acc[0][1], acc[1][1], acc[0][3], acc[1][3]));
    }
  }
};

// ---------------------------------------------------------------------------------------------
// 16-bit consumer (bf16 or fp16): 64 features (one box per block), m16n8k16 over pairs of blocks.
//   k-slots 2t, 2t+1 <-> block 0, columns 2t, 2t+1;  k-slots 2t+8, 2t+9 <-> block 1, same columns;
//   MMA tile j (j = 0..3): m = g <-> feature 8g + j,  m = g + 8 <-> feature 8g + 4 + j.
// An odd block at the end of a stage pairs with zeros (its partner's box is never read).
// ---------------------------------------------------------------------------------------------
template <bool BF16>
struct H16Consumer {
  static constexpr int kABytes = 128;
  static constexpr int kFeat = 64;
  float acc[4][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  }
  __device__ __forceinline__ void blocks(const uint8_t* box, int block_stride, const uint8_t* a_blocks, int n, int g, int t) {
    const int rd0 = (2 * t) * 128 + (((g ^ (2 * t)) & 7) << 4);
    const int rd1 = (2 * t + 1) * 128 + (((g ^ (2 * t + 1)) & 7) << 4);
#pragma unroll 2
    for (int k = 0; k < n; k += 2) {
      const bool two = k + 1 < n;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(a_blocks + k * 128 + (g * 8 + 2 * t) * 2);
      const uint32_t b1 = two ? *reinterpret_cast<const uint32_t*>(a_blocks + (k + 1) * 128 + (g * 8 + 2 * t) * 2) : 0u;
      const uint8_t* t0 = box + k * block_stride;
      const uint8_t* t1 = t0 + block_stride;
      const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
      const uint4 v0 = *reinterpret_cast<const uint4*>(t0 + rd0);              // block 0, column 2t: features 8g .. 8g+7
      const uint4 v1 = *reinterpret_cast<const uint4*>(t0 + rd1);              // block 0, column 2t+1
      const uint4 v2 = two ? *reinterpret_cast<const uint4*>(t1 + rd0) : zero4;   // block 1, column 2t
      const uint4 v3 = two ? *reinterpret_cast<const uint4*>(t1 + rd1) : zero4;   // block 1, column 2t+1
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
  }
  __device__ __forceinline__ void store(float* c_row0, int64_t ldc, int F, int N, int g, int t) {
    if (F + 8 * g < N) {
      float* c0 = c_row0 + (2 * t) * ldc + F + 8 * g;
      float* c1 = c0 + ldc;
      __stcs(reinterpret_cast<float4*>(c0), make_float4(acc[0][0], acc[1][0], acc[2][0], acc[3][0]));
      __stcs(reinterpret_cast<float4*>(c0 + 4), make_float4(acc[0][2], acc[1][2], acc[2][2], acc[3][2]));
      __stcs(reinterpret_cast<float4*>(c1), make_float4(acc[0][1], acc[1][1], acc[2][1], acc[3][1]));
      __stcs(reinterpret_cast<float4*>(c1 + 4), make_float4(acc[0][3], acc[1][3], acc[2][3], acc[3][3]));
    }
  }
};

// grid.x = groups of block rows x feature tiles (tile index fastest, or all groups of tile 0 first
// when tile_major_groups > 0: then the B rows of one tile stay in the L2 while it is worked on).
template <typename Consumer, int NCW, int SB, int D, int MINB>
__global__ void __launch_bounds__((NCW + 1) * 32, MINB)
bsr8_spmm_pipe_kernel(const __grid_constant__ CUtensorMap mapB, const int64_t* __restrict__ indptr,
                      const int32_t* __restrict__ indices, const uint8_t* __restrict__ blocks,
                      int64_t block_row_begin, int64_t block_row_end, float* __restrict__ C, int64_t ldc, int N,
                      int tiles, int rows_per_cta, int64_t tile_major_groups, int boxes_per_block) {
  using Cfg = PipeCfg<NCW, SB, D, Consumer::kABytes>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t grp;
  int tile;
  split_work((int64_t)blockIdx.x, tiles, tile_major_groups, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_cta;
  if (I0 >= block_row_end || tile >= tiles) return;
  const int R = (int)min((int64_t)rows_per_cta, block_row_end - I0);   // <= 31

  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t pad = ((raw_u32 + 1023u) & ~1023u) - raw_u32;
  uint8_t* base = smem_raw + pad;
  const uint32_t base_u32 = raw_u32 + pad;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base + Cfg::kOffBar + 2 * D * 8);
  const uint32_t bar_full = base_u32 + Cfg::kOffBar, bar_empty = bar_full + D * 8;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
#pragma unroll
    for (int s = 0; s < D; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, NCW);
    }
    mbar_fence_init();
  }
  __syncthreads();

  RowPtrs ptrs;
  ptrs.mine = indptr[I0 + min(lane, R)];

  if (warp == NCW) {
    produce<Cfg, NCW, SB, D, Consumer::kABytes, Consumer::kFeat>(&mapB, ptrs, R, indices, blocks, tile, boxes_per_block,
                                                                 base_u32, abort_flag, lane);
    if (*abort_flag && lane == 0) atomicAdd(&g_pipe_timeouts, 1);
    return;
  }

  // ---- consumers ------------------------------------------------------------------------------
  const int g = lane >> 2, t = lane & 3;
  const int F = (tile * NCW + warp) * Consumer::kFeat;   // first feature of this warp's slice
  Consumer cons;
  int slot = 0;
  uint32_t round = 0;
  for (int r = 0; r < R; ++r) {
    cons.zero();
    int64_t b = ptrs.at(r);
    const int64_t be = ptrs.at(r + 1);
    do {
      const int n = (int)min((int64_t)SB, be - b);
      bool ok = mbar_wait(bar_full + 8 * slot, round & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {   // unfinished rows of C stay unwritten; the host learns through lf_bsr_copy_status
        if (warp == 0 && lane == 0) atomicAdd(&g_pipe_timeouts, 1);
        return;
      }
      cons.blocks(base + slot * Cfg::kStageB + warp * 1024, Cfg::kBlockB, base + Cfg::kOffA + slot * Cfg::kStageA, n, g, t);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
      b += n;
      if (++slot == D) { slot = 0; ++round; }
    } while (b < be);
    cons.store(C + (I0 + r - block_row_begin) * 8 * ldc, ldc, F, N, g, t);
  }
}

// ---- host side ---------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

// B as a tensor of this GPU's memory.  3-D view {features of a slice (128 bytes), rows, slices}: the
// slice index walks along a row in steps of 128 bytes, so one box {128 bytes, 8 rows, NCW slices}
// is the whole tile of a block, laid down slice after slice.  Needs N to be a whole number of
// slices.  Otherwise (or when the driver refuses the 3-D view) the 2-D view {N, rows} with one
// box {128 bytes, 8 rows} per slice; features beyond N read as zeros.  The number of rows of B is
// not an argument of the product (A's block columns index it), so the map claims the largest row
// count a 32-bit coordinate can name; a copy touches only the rows its coordinates name.
}  // namespace

int bsr8_make_b_map(CUtensorMap* map, int* boxes_per_block, const void* B, int64_t ldb, int N, int elem_bytes, int ncw,
                    bool allow_3d) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(LF_ERR_UNSUPPORTED, "the driver does not export cuTensorMapEncodeTiled");
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
  const cuuint32_t per_slice = (cuuint32_t)(128 / elem_bytes);
  if (allow_3d && N % (int)per_slice == 0) {
    const cuuint64_t dims[3] = {per_slice, (cuuint64_t)1 << 31, (cuuint64_t)(N / (int)per_slice)};
    const cuuint64_t strides[2] = {(cuuint64_t)ldb * elem_bytes, 128};
    const cuuint32_t box[3] = {per_slice, 8, (cuuint32_t)ncw};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, dt, 3, const_cast<void*>(B), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
      *boxes_per_block = 1;
      return LF_OK;
    }
  }
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)1 << 31};
  const cuuint64_t strides[1] = {(cuuint64_t)ldb * elem_bytes};
  const cuuint32_t box[2] = {per_slice, 8};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void*>(B), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LF_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  *boxes_per_block = ncw;
  return LF_OK;
}

namespace {

template <typename Consumer, int NCW, int SB, int D, int MINB>
int launch(const CUtensorMap& map, int boxes, const int64_t* indptr, const int32_t* indices, const void* blocks, int64_t r0,
           int64_t r1, float* C, int64_t ldc, int N, int rows_per_cta, bool tile_major, cudaStream_t st) {
  using Cfg = PipeCfg<NCW, SB, D, Consumer::kABytes>;
  const int tile_feat = NCW * Consumer::kFeat;
  const int tiles = (N + tile_feat - 1) / tile_feat;
  const int64_t groups = ceil_div64(r1 - r0, rows_per_cta);
  const int64_t grid = groups * tiles;
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  auto k = bsr8_spmm_pipe_kernel<Consumer, NCW, SB, D, MINB>;
  LF_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  k<<<(unsigned)grid, Cfg::kThreads, Cfg::kSmem, st>>>(map, indptr, indices, (const uint8_t*)blocks, r0, r1, C, ldc, N, tiles,
                                                      rows_per_cta, tile_major ? groups : 0, boxes);
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

}  // namespace

// shape: blocks per stage * 10 + stages; 0 or an unknown value = 4 blocks, 4 stages
int bsr8_f32_pipe_launch(const int64_t* indptr, const int32_t* indices, const float* blocks, int64_t r0, int64_t r1,
                         const float* B, int64_t ldb, float* C, int64_t ldc, int N, int shape, int rows_per_cta,
                         bool tile_major, bool allow_3d, cudaStream_t st) {
  CUtensorMap map = {};
  int boxes = 0;
  if (int s = bsr8_make_b_map(&map, &boxes, B, ldb, N, 4, 4, allow_3d)) return s;
  const int rpc = rows_per_cta >= 1 && rows_per_cta <= 31 ? rows_per_cta : 31;
  switch (shape) {
    case 83: return launch<F32Consumer, 4, 8, 3, 2>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, tile_major, st);
    case 43: return launch<F32Consumer, 4, 4, 3, 4>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, tile_major, st);
    case 26: return launch<F32Consumer, 4, 2, 6, 4>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, tile_major, st);
    default: return launch<F32Consumer, 4, 4, 4, 3>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, tile_major, st);
  }
}

int bsr8_16bit_pipe_launch(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks, int64_t r0,
                           int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int N, int shape,
                           int rows_per_cta, bool allow_3d, cudaStream_t st) {
  CUtensorMap map = {};
  int boxes = 0;
  const int ncw = N > 128 ? 4 : 2;   // 256 features per thread block when there are that many, else 128
  if (int s = bsr8_make_b_map(&map, &boxes, B, ldb, N, 2, ncw, allow_3d)) return s;
  const int rpc = rows_per_cta >= 1 && rows_per_cta <= 31 ? rows_per_cta : 31;
#define LF_PIPE16(NCW_, SB_, D_, M_)                                                                                  \
  (bf16 ? launch<H16Consumer<true>, NCW_, SB_, D_, M_>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, false, st) \
        : launch<H16Consumer<false>, NCW_, SB_, D_, M_>(map, boxes, indptr, indices, blocks, r0, r1, C, ldc, N, rpc, false, st))
  if (ncw == 4) {
    switch (shape) {
      case 83: return LF_PIPE16(4, 8, 3, 2);
      case 43: return LF_PIPE16(4, 4, 3, 4);
      default: return LF_PIPE16(4, 4, 4, 3);
    }
  }
  switch (shape) {
    case 83: return LF_PIPE16(2, 8, 3, 4);
    case 43: return LF_PIPE16(2, 4, 3, 8);
    default: return LF_PIPE16(2, 4, 4, 6);
  }
#undef LF_PIPE16
}

int bsr8_pipe_timeouts(cudaStream_t st, int* count) {
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  int n = 0;
  LF_CUDA_CHECK(cudaMemcpyFromSymbol(&n, g_pipe_timeouts, sizeof(int)));
  if (n) {
    const int zero = 0;
    LF_CUDA_CHECK(cudaMemcpyToSymbol(g_pipe_timeouts, &zero, sizeof(int)));
  }
  *count = n;
  return LF_OK;
}

}  // namespace lf
