// C = A @ B for A in 8x8 block-sparse rows, 16-bit inputs: the 5th-generation tensor-core path
// (tcgen05.mma with the accumulator in tensor memory).
//
// Takes over the kernel of the reference's bench_bsrmm (playground_pipline/format_algos.py:1562-1643;
// arithmetic format_algos.py:1204-1213; the reference multiplies 32x32 fp16 blocks with wmma and
// fp16 accumulators, format_algos.py:1226-1233).  The product is computed transposed, one block row
// at a time:  D[feature, row] = sum over the blocks (I, J) of the block row of
//     Bt_J[feature, k] * At_IJ[k, row],      k = 0..7 the rows of B that block column J names,
// so that features run along the M dimension of the instruction (64 per MMA), the 8 rows of a
// block row are its N dimension, and two blocks make one K = 16 step.  Nothing is rearranged on
// the way:
//   * the MMA's A operand (M x K, "MN-major": features contiguous) is exactly the box a tiled bulk
//     copy writes for a block: 8 rows of B x 128 bytes, swizzle mode 128B.  The next block's box is
//     the K-direction neighbour (stride byte offset = size of a block's boxes);
//   * the MMA's B operand (N x K, K-major, no swizzle) is the 8x8 tile as BSR stores it: 8 rows of
//     16 bytes = one core matrix; the next tile in memory is the next K step (leading byte offset
//     128).  The tiles of a stage are contiguous in memory and arrive with one bulk copy;
//   * the accumulator D (64 features x 8 rows, fp32) lives in 8 columns of tensor memory; a block
//     row of a 128-feature tile uses two accumulators, a ring of accumulator stages lets the
//     epilogue of one block row overlap the MMAs of the next.
// Thread block = 6 warps: warps 0-3 read accumulators back (tcgen05.ld, each warp its quarter of the
// tensor-memory lanes) and store C; warp 4 issues the copies (one tiled copy per block); one lane
// of warp 5 issues the MMAs and commits them to mbarriers (tcgen05.commit), which is also what
// returns a shared-memory stage to the producer.  All three derive the same sequence of stages
// from the block-row pointers.  No warp computes a copy address, loads a fragment or issues a
// warp-level MMA: per block the thread block executes a few dozen instructions.
//
// An odd block at the end of a stage is paired with a zero tile (written by the producer, made
// visible to the tensor core with a proxy fence) and a duplicate of its own B rows.
//
// Two producers, chosen at launch.  (a) One warp issuing tiled bulk copies (TMA) as described.
// (b) NP warps copying the same bytes with per-lane 16-byte cp.async into the same swizzled
// layout (chunk c of row r at c ^ r, written by hand): the tiled copies deliver scattered 128-byte
// rows at about 22-26 bytes per clock and SM whatever the ring looks like, 32 lanes issuing the
// same rows with one instruction get more.  cp.async writes through the generic proxy, the tensor
// core reads through the async proxy: a producer warp waits for its own copies of a stage
// (cp.async.wait_group), issues fence.proxy.async, then arrives on the stage's mbarrier; padding
// (a missing pair partner, features beyond N) is zero-filled by the copy itself.
// Every wait is bounded; a thread block that gives up raises a flag, drains its copies, frees its
// tensor memory and returns; the host reads the count through lf_bsr_copy_status.  No copy and no
// commit uses cluster multicast; the tensor map covers memory of this GPU only.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "lf_bsr8_mma.cuh"
#include "lf_bsr8_tma.cuh"
#include "lf_common.cuh"

namespace lf {
namespace {

using namespace bsr8;

__device__ int g_umma_timeouts;   // thread blocks that gave up waiting

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

// ---- tensor memory and tcgen05 ----------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {        // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// the mbarrier gets one arrival once every MMA this thread issued so far has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 8 consecutive 32-bit columns: thread l of the warp gets lane (taddr.lane + l)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (64 bits): start address >> 4 in bits [0,14), leading byte offset
// >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), layout type in
// [61,64) (0 = no swizzle, 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((uint64_t)layout_type << 61);
}
// Instruction descriptor (32 bits) of kind::f16: D format fp32 (1 at bit 4), A / B element type at bits
// 7 / 10 (0 = fp16, 1 = bf16), A MN-major (bit 15), B K-major (bit 16 = 0), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, int M, int N) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (1u << 15) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// Shared memory of one thread block (offsets from a 1024-byte aligned base):
//   [D][SB][NS] boxes of 1024 bytes   B rows: box = 8 rows x 64 features, swizzled
//   [D][SB] tiles of 128 bytes        A blocks
//   barriers: full[D], empty[D], acc_full[AS], acc_empty[AS]; tensor-memory base; abort flag
template <int NS, int SB, int D, int AS>
struct UmmaCfg {
  static constexpr int kBlockB = NS * 1024;
  static constexpr int kStageB = SB * kBlockB;
  static constexpr int kStageA = SB * 128;
  static constexpr int kOffA = D * kStageB;
  static constexpr int kOffBar = kOffA + D * kStageA;
  static constexpr int kBars = 2 * D + 2 * AS;
  static constexpr int kOffMisc = kOffBar + kBars * 8;
  static constexpr int kSmem = kOffMisc + 16 + 1024;   // + slack for the alignment
  static constexpr int kTmemCols = AS * NS * 8 < 32 ? 32 : AS * NS * 8;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "tensor-memory columns must be a power of two");
  static_assert(SB % 2 == 0, "a stage holds whole pairs of blocks");
};

struct RowPtrs {
  int64_t mine;   // lane l <= R holds row pointer I0 + l
  __device__ __forceinline__ int64_t at(int r) const { return __shfl_sync(0xffffffffu, mine, r); }
};

// NP = 0: one producer warp issuing tiled bulk copies; NP > 0: NP producer warps issuing cp.async.
// Warps 0-3 epilogue, then the producer warp(s), then the MMA warp.
template <bool BF16, int NS, int SB, int D, int AS, int MINB, int NP>
__global__ void __launch_bounds__((5 + (NP > 0 ? NP : 1)) * 32, MINB)
bsr8_spmm_umma_kernel(const __grid_constant__ CUtensorMap mapB, const int64_t* __restrict__ indptr,
                      const int32_t* __restrict__ indices, const uint8_t* __restrict__ blocks,
                      const uint16_t* __restrict__ Bmat, int ldb,
                      int64_t block_row_begin, int64_t block_row_end, float* __restrict__ C, int64_t ldc, int N,
                      int tiles, int rows_per_cta, int boxes_per_block) {
  constexpr int kProducers = NP > 0 ? NP : 1;
  constexpr int kMmaWarp = 4 + kProducers;
  using Cfg = UmmaCfg<NS, SB, D, AS>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t grp;
  int tile;
  split_work((int64_t)blockIdx.x, tiles, 0, grp, tile);
  const int64_t I0 = block_row_begin + grp * rows_per_cta;
  if (I0 >= block_row_end || tile >= tiles) return;
  const int R = (int)min((int64_t)rows_per_cta, block_row_end - I0);   // <= 31

  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t pad = ((raw_u32 + 1023u) & ~1023u) - raw_u32;
  uint8_t* base = smem_raw + pad;
  const uint32_t base_u32 = raw_u32 + pad;
  const uint32_t bar_full = base_u32 + Cfg::kOffBar, bar_empty = bar_full + D * 8;
  const uint32_t bar_acc_full = bar_empty + D * 8, bar_acc_empty = bar_acc_full + AS * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base + Cfg::kOffMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base + Cfg::kOffMisc + 8);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
#pragma unroll
    for (int s = 0; s < D; ++s) {
      mbar_init(bar_full + 8 * s, kProducers);   // one arrival per producer warp (the TMA producer adds its byte count)
      mbar_init(bar_empty + 8 * s, 1);
    }
#pragma unroll
    for (int s = 0; s < AS; ++s) {
      mbar_init(bar_acc_full + 8 * s, 1);
      mbar_init(bar_acc_empty + 8 * s, 4);
    }
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(base_u32 + Cfg::kOffMisc, Cfg::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  RowPtrs ptrs;
  ptrs.mine = indptr[I0 + min(lane, R)];

  if (NP > 0 && warp >= 4 && warp < kMmaWarp) {
    // ---- producers (cp.async): NP warps copy every stage together, 16 bytes per lane and instruction --
    constexpr int LAG = 2;                      // stages a producer warp keeps in flight before it waits
    static_assert(D >= LAG + 2, "the ring must hold the stages in flight plus one being multiplied");
    constexpr int PL = (NP > 0 ? NP : 1) * 32;  // producer lanes
    const int pl = (warp - 4) * 32 + lane;
    const int64_t stream_end = ptrs.at(R);
    int64_t win = ptrs.at(0);
    int idx_cur = (win + lane < stream_end) ? indices[win + lane] : 0;
    int q = 0;
    bool ok = true;
    auto publish = [&](int stage) {             // this warp's copies of `stage` have landed: hand them over
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_full + 8 * (stage % D));
    };
    for (int r = 0; r < R && ok; ++r) {
      int64_t b = ptrs.at(r);
      const int64_t be = ptrs.at(r + 1);
      while (b < be) {
        const int n = (int)min((int64_t)SB, be - b);
        const int n_pad = (n + 1) & ~1;
        const int slot = q % D;
        const uint32_t round = (uint32_t)(q / D);
        if (round > 0) {
          ok = mbar_wait(bar_empty + 8 * slot, (round - 1) & 1u, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (b + SB > win + 32) {   // keep the block columns of the whole stage inside the window
          win = b;
          idx_cur = (win + lane < stream_end) ? indices[win + lane] : 0;
        }
        const uint32_t dstB = base_u32 + slot * Cfg::kStageB;
        // B rows: 16-byte chunk c of the stage = (block k, slice s, row r8, chunk j)
        for (int c = pl; c < n_pad * NS * 64; c += PL) {
          const int k = c / (NS * 64), w = c % (NS * 64);
          const int sl = w >> 6, r8 = (w >> 3) & 7, j = w & 7;
          const int J = __shfl_sync(0xffffffffu, idx_cur, (int)(b - win) + (k < n ? k : n - 1));
          const int f = (tile * NS + sl) * 64 + j * 8;
          const bool live = k < n && f < N;
          const uint16_t* src = Bmat + ((int64_t)J * 8 + r8) * ldb + (live ? f : 0);
          cp_async16(dstB + k * Cfg::kBlockB + sl * 1024 + r8 * 128 + ((j ^ r8) << 4), src, live ? 16 : 0);
        }
        // A tiles: 8 chunks per block, contiguous in memory
        if (pl < n_pad * 8) {
          const int k = pl >> 3;
          cp_async16(base_u32 + Cfg::kOffA + slot * Cfg::kStageA + pl * 16, blocks + (b + (k < n ? k : 0)) * 128 + (pl & 7) * 16,
                     k < n ? 16 : 0);
        }
        cp_async_commit();
        if (q >= LAG) {
          cp_async_wait<LAG>();
          publish(q - LAG);
        }
        ++q;
        b += n;
      }
    }
    cp_async_wait<0>();                         // also on the way out after giving up: nothing stays in flight
    if (ok)
      for (int stage = q >= LAG ? q - LAG : 0; stage < q; ++stage) publish(stage);
  } else if (NP == 0 && warp == 4) {
    // ---- producer: one tiled copy per block, one bulk copy for the tiles of a stage ------------
    const int64_t stream_end = ptrs.at(R);
    int64_t win = ptrs.at(0);
    int idx_cur = (win + lane < stream_end) ? indices[win + lane] : 0;
    int idx_nxt = (win + 32 + lane < stream_end) ? indices[win + 32 + lane] : 0;
    int q = 0;      // stages armed so far: stage q uses slot q % D for the (q / D)-th time
    bool ok = true;
    for (int r = 0; r < R && ok; ++r) {
      int64_t b = ptrs.at(r);
      const int64_t be = ptrs.at(r + 1);
      while (b < be) {
        const int n = (int)min((int64_t)SB, be - b);
        const int n_pad = (n + 1) & ~1;   // an odd last block is paired with a zero tile and its own B rows again
        const int slot = q % D;
        const uint32_t round = (uint32_t)(q / D);
        if (round > 0) {
          ok = mbar_wait(bar_empty + 8 * slot, (round - 1) & 1u, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        const uint32_t full = bar_full + 8 * slot;
        const uint32_t dstA = base_u32 + Cfg::kOffA + slot * Cfg::kStageA;
        if (n_pad != n) {   // zero tile: 128 bytes written by 8 lanes, then made visible to the tensor core
          if (lane < 8) *reinterpret_cast<uint4*>(base + Cfg::kOffA + slot * Cfg::kStageA + n * 128 + lane * 16) = make_uint4(0u, 0u, 0u, 0u);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
        }
        if (lane == 0) mbar_expect_tx(full, (uint32_t)n_pad * Cfg::kBlockB + (uint32_t)n * 128);   // the one arrival + bytes
        ++q;
        const uint32_t dstB = base_u32 + slot * Cfg::kStageB;
        for (int k = 0; k < n_pad; ++k) {
          const int64_t bk = b + (k < n ? k : n - 1);
          if (bk >= win + 32) {
            win += 32;
            idx_cur = idx_nxt;
            idx_nxt = (win + 32 + lane < stream_end) ? indices[win + 32 + lane] : 0;
          }
          const int J = __shfl_sync(0xffffffffu, idx_cur, (int)(bk - win));
          if (lane == 0) {
            if (boxes_per_block == 1) {
              tma_load_3d(dstB + k * Cfg::kBlockB, &mapB, 0, J * 8, tile * NS, full);
            } else {
#pragma unroll
              for (int s = 0; s < NS; ++s)
                tma_load_2d(dstB + k * Cfg::kBlockB + s * 1024, &mapB, (tile * NS + s) * 64, J * 8, full);
            }
          }
        }
        if (lane == 0) bulk_load(dstA, blocks + b * 128, (uint32_t)n * 128, full);
        b += n;
      }
    }
    if (!ok) {   // giving up: let the copies already issued land (bounded) before the shared memory goes away
      for (int p = q - 1; p >= 0 && p >= q - D; --p) {
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_full + 8 * (p % D), (uint32_t)(p / D) & 1u) && clock64() - t0 < kWaitCycles) {}
      }
    }
  } else if (warp == kMmaWarp) {
    // ---- MMA issuer -------------------------------------------------------------------------------
    constexpr uint32_t idesc = instr_desc(BF16, 64, 8);
    int q = 0;      // stages consumed so far
    int u = 0;      // block rows with blocks seen so far: row u uses accumulator stage u % AS
    bool ok = true;
    for (int r = 0; r < R && ok; ++r) {
      int64_t b = ptrs.at(r);
      const int64_t be = ptrs.at(r + 1);
      if (b == be) continue;
      const int as = u % AS;
      const uint32_t around = (uint32_t)(u / AS);
      if (around > 0) {   // the epilogue must have read this accumulator stage back
        ok = mbar_wait(bar_acc_empty + 8 * as, (around - 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      uint32_t accumulate = 0;
      while (b < be) {
        const int n = (int)min((int64_t)SB, be - b);
        const int slot = q % D;
        ok = mbar_wait(bar_full + 8 * slot, (uint32_t)(q / D) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t sB = base_u32 + slot * Cfg::kStageB;
          const uint32_t sA = base_u32 + Cfg::kOffA + slot * Cfg::kStageA;
          for (int k = 0; k < n; k += 2) {
            // B operand: two 8x8 tiles = two core matrices along K, 128 bytes apart
            const uint64_t b_desc = smem_desc(sA + k * 128, 128, 128, 0);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
              // A operand: box of block k (k-rows 0..7) and of block k + 1 (k-rows 8..15), 64 features each
              const uint64_t a_desc = smem_desc(sB + k * Cfg::kBlockB + s * 1024, 1024, Cfg::kBlockB, 2);
              umma_f16(tmem_base + (uint32_t)((as * NS + s) * 8), a_desc, b_desc, idesc, accumulate);
            }
            accumulate = 1;
          }
          umma_commit(bar_empty + 8 * slot);   // the stage returns to the producer when these MMAs are done
        }
        __syncwarp();
        ++q;
        b += n;
      }
      if (!ok) break;
      if (lane == 0) umma_commit(bar_acc_full + 8 * as);
      __syncwarp();
      ++u;
    }
  } else {
    // ---- epilogue: warp w reads the lanes 32 w .. 32 w + 31 of tensor memory -----------------------
    // a 64-row accumulator keeps row i in lane (i % 16) + 32 (i / 16): lanes 0..15 of every warp hold
    // features 16 w + lane of each 64-feature slice
    int u = 0;
    bool ok = true;
    const int F0 = tile * NS * 64 + 16 * warp + (lane & 15);
    for (int r = 0; r < R && ok; ++r) {
      const bool empty_row = ptrs.at(r) == ptrs.at(r + 1);
      float* c_row = C + (I0 + r - block_row_begin) * 8 * ldc;
      uint32_t v[NS][8];
      if (!empty_row) {
        const int as = u % AS;
        ok = mbar_wait(bar_acc_full + 8 * as, (uint32_t)(u / AS) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int s = 0; s < NS; ++s)
          tmem_ld8(tmem_base + ((uint32_t)(32 * warp) << 16) + (uint32_t)((as * NS + s) * 8), v[s]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * as);
        ++u;
      } else {
#pragma unroll
        for (int s = 0; s < NS; ++s)
#pragma unroll
          for (int i = 0; i < 8; ++i) v[s][i] = 0u;
      }
      if (lane < 16) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          const int f = F0 + s * 64;
          if (f < N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) __stcs(c_row + i * ldc + f, __uint_as_float(v[s][i]));
          }
        }
      }
    }
  }

  // every warp arrives here, also after giving up: tensor memory is freed before the block exits
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) {
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
    if (*abort_flag && lane == 0) atomicAdd(&g_umma_timeouts, 1);
  }
}

template <bool BF16, int NS, int SB, int D, int AS, int MINB, int NP>
int launch(const CUtensorMap& map, int boxes, const int64_t* indptr, const int32_t* indices, const void* blocks,
           const uint16_t* B, int64_t ldb, int64_t r0, int64_t r1, float* C, int64_t ldc, int N, int rows_per_cta,
           cudaStream_t st) {
  using Cfg = UmmaCfg<NS, SB, D, AS>;
  const int tiles = (N + NS * 64 - 1) / (NS * 64);
  const int64_t grid = ceil_div64(r1 - r0, rows_per_cta) * tiles;
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  auto k = bsr8_spmm_umma_kernel<BF16, NS, SB, D, AS, MINB, NP>;
  LF_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  k<<<(unsigned)grid, (5 + (NP > 0 ? NP : 1)) * 32, Cfg::kSmem, st>>>(map, indptr, indices, (const uint8_t*)blocks, B, (int)ldb,
                                                                     r0, r1, C, ldc, N, tiles, rows_per_cta, boxes);
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

}  // namespace

// shape: blocks per stage * 10 + stages (44 default, 83, 46, 86); producer: 0 tiled bulk copies, 2 or 4 = that many
// warps issuing cp.async
int bsr8_16bit_umma_launch(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks, int64_t r0,
                           int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int N, int shape,
                           int rows_per_cta, bool allow_3d, int producer, cudaStream_t st) {
  CUtensorMap map = {};
  int boxes = 0;
  const int ns = N > 128 ? 4 : 2;   // 256 features per thread block when there are that many, else 128
  if (producer == 0)
    if (int s = bsr8_make_b_map(&map, &boxes, B, ldb, N, 2, ns, allow_3d)) return s;
  const int rpc = rows_per_cta >= 1 && rows_per_cta <= 31 ? rows_per_cta : 31;
#define LF_UMMA(NS_, SB_, D_, AS_, M_, NP_)                                                                              \
  (bf16 ? launch<true, NS_, SB_, D_, AS_, M_, NP_>(map, boxes, indptr, indices, blocks, B, ldb, r0, r1, C, ldc, N, rpc, st)    \
        : launch<false, NS_, SB_, D_, AS_, M_, NP_>(map, boxes, indptr, indices, blocks, B, ldb, r0, r1, C, ldc, N, rpc, st))
#define LF_UMMA_P(NS_, SB_, D_, AS_, M_) \
  (producer == 0 ? LF_UMMA(NS_, SB_, D_, AS_, M_, 0) : producer == 4 ? LF_UMMA(NS_, SB_, D_, AS_, M_, 4) : LF_UMMA(NS_, SB_, D_, AS_, M_, 2))
  if (ns == 4) {
    switch (shape) {
      case 83: return LF_UMMA_P(4, 8, 4, 2, 1);
      case 46: return LF_UMMA_P(4, 4, 6, 2, 2);
      case 24: return LF_UMMA_P(4, 2, 4, 2, 3);
      default: return LF_UMMA_P(4, 4, 4, 2, 3);
    }
  }
  switch (shape) {
    case 83: return LF_UMMA_P(2, 8, 4, 4, 3);
    case 46: return LF_UMMA_P(2, 4, 6, 4, 4);
    case 86: return LF_UMMA_P(2, 8, 6, 4, 2);
    case 24: return LF_UMMA_P(2, 2, 4, 4, 6);
    default: return LF_UMMA_P(2, 4, 4, 4, 6);
  }
#undef LF_UMMA_P
#undef LF_UMMA
}

int bsr8_umma_timeouts(cudaStream_t st, int* count) {
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  int n = 0;
  LF_CUDA_CHECK(cudaMemcpyFromSymbol(&n, g_umma_timeouts, sizeof(int)));
  if (n) {
    const int zero = 0;
    LF_CUDA_CHECK(cudaMemcpyToSymbol(g_umma_timeouts, &zero, sizeof(int)));
  }
  *count = n;
  return LF_OK;
}

}  // namespace lf
