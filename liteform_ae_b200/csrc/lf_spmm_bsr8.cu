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
//     m16n8k8 tf32 MMAs (hi*hi + lo*hi + hi*lo) reproduce the fp32 product to ~2^-22 relative.
//   * 16-bit path (bf16 or fp16 inputs): m16n8k16 over a pair of blocks, fp32 accumulate.
//
// Because M and K of an MMA are only summation/placement indices, both are permuted so that every
// global access is a full-width vector: a lane's four (float32) or eight (16-bit) consecutive
// features of one B row feed four / eight different MMA tiles, and the k-slots of a lane map to
// adjacent block columns so that its two A values are one 64-bit (32-bit) load.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "lf_common.cuh"

namespace lf {
namespace {

constexpr int kWarps = 8;
constexpr int kThreadsBsr = kWarps * 32;

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool BF16>
__device__ __forceinline__ void mma_16bit(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// ---------------------------------------------------------------------------------------------
// float32 in / float32 out, 3xTF32.  One warp = one block row x one tile of 64*T features.
// Lane (g = lane / 4, t = lane % 4).  MMA index maps (see the file header):
//   k-slot t   <-> block column 2t      k-slot t+4 <-> block column 2t+1
//   MMA tile j of unit q: m = g   <-> feature F + 64q + 4g + j
//                         m = g+8 <-> feature F + 64q + 32 + 4g + j
//   n <-> row of the block; a lane ends with C[row 2t / 2t+1][4 consecutive features] as float4.
// The loop over the blocks of the row is software-pipelined: the B rows and A values of block
// b+1 are requested before the MMAs of block b are issued (two register buffers, ping-pong).
// ---------------------------------------------------------------------------------------------
template <int T>
struct FragF32 {
  float4 x0[T], x1[T], y0[T], y1[T];
  float2 av;
};

template <int T, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_f32_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                     const float* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                     const float* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                     int tiles) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // tile index runs fastest so that the tiles of one block row are resident together and the
  // A blocks they share are fetched from HBM once
  const int64_t work = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t I = block_row_begin + work / tiles;
  if (I >= block_row_end) return;
  const int F = (int)(work % tiles) * (64 * T);

  float acc[T][4][4];
#pragma unroll
  for (int q = 0; q < T; ++q)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[q][j][i] = 0.f;

  bool lo_ok[T], hi_ok[T];  // feature ranges of m = g and m = g+8 inside N?
#pragma unroll
  for (int q = 0; q < T; ++q) {
    lo_ok[q] = F + 64 * q + 4 * g < N;
    hi_ok[q] = F + 64 * q + 32 + 4 * g < N;
  }

  const int64_t bs = indptr[I];
  const int nblk = (int)(indptr[I + 1] - bs);
  const float* Bl = B + F + 4 * g + (int64_t)(2 * t) * ldb;
  const float* Al = blocks + g * 8 + 2 * t;
  int my_idx = 0;

  auto load = [&](FragF32<T>& f, int b) {
    if ((b & 31) == 0) my_idx = (b + lane < nblk) ? indices[bs + b + lane] : 0;
    const int J = __shfl_sync(0xffffffffu, my_idx, b & 31);
    f.av = __ldcs(reinterpret_cast<const float2*>(Al + (bs + b) * 64));
    const float* r0 = Bl + (int64_t)J * 8 * ldb;
    const float* r1 = r0 + ldb;
#pragma unroll
    for (int q = 0; q < T; ++q) {
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      f.x0[q] = lo_ok[q] ? __ldg(reinterpret_cast<const float4*>(r0 + 64 * q)) : z;
      f.y0[q] = lo_ok[q] ? __ldg(reinterpret_cast<const float4*>(r1 + 64 * q)) : z;
      f.x1[q] = hi_ok[q] ? __ldg(reinterpret_cast<const float4*>(r0 + 64 * q + 32)) : z;
      f.y1[q] = hi_ok[q] ? __ldg(reinterpret_cast<const float4*>(r1 + 64 * q + 32)) : z;
    }
  };

  auto compute = [&](const FragF32<T>& f) {
    const uint32_t b0h = to_tf32(f.av.x), b1h = to_tf32(f.av.y);
    const uint32_t b0l = to_tf32(f.av.x - __uint_as_float(b0h)), b1l = to_tf32(f.av.y - __uint_as_float(b1h));
#pragma unroll
    for (int q = 0; q < T; ++q) {
      const float a_f[4][4] = {{f.x0[q].x, f.x1[q].x, f.y0[q].x, f.y1[q].x},
                               {f.x0[q].y, f.x1[q].y, f.y0[q].y, f.y1[q].y},
                               {f.x0[q].z, f.x1[q].z, f.y0[q].z, f.y1[q].z},
                               {f.x0[q].w, f.x1[q].w, f.y0[q].w, f.y1[q].w}};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t ah[4], al[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ah[i] = to_tf32(a_f[j][i]);
          al[i] = to_tf32(a_f[j][i] - __uint_as_float(ah[i]));
        }
        mma_tf32(acc[q][j], al, b0h, b1h);
        mma_tf32(acc[q][j], ah, b0l, b1l);
        mma_tf32(acc[q][j], ah, b0h, b1h);
      }
    }
  };

  FragF32<T> fa, fb;
  if (nblk > 0) load(fa, 0);
  for (int b = 0; b < nblk; b += 2) {
    if (b + 1 < nblk) load(fb, b + 1);
    compute(fa);
    if (b + 1 < nblk) {
      if (b + 2 < nblk) load(fa, b + 2);
      compute(fb);
    }
  }

  float* c0 = C + ((I - block_row_begin) * 8 + 2 * t) * ldc + F + 4 * g;
  float* c1 = c0 + ldc;
#pragma unroll
  for (int q = 0; q < T; ++q) {
    if (lo_ok[q]) {
      __stcs(reinterpret_cast<float4*>(c0 + 64 * q), make_float4(acc[q][0][0], acc[q][1][0], acc[q][2][0], acc[q][3][0]));
      __stcs(reinterpret_cast<float4*>(c1 + 64 * q), make_float4(acc[q][0][1], acc[q][1][1], acc[q][2][1], acc[q][3][1]));
    }
    if (hi_ok[q]) {
      __stcs(reinterpret_cast<float4*>(c0 + 64 * q + 32), make_float4(acc[q][0][2], acc[q][1][2], acc[q][2][2], acc[q][3][2]));
      __stcs(reinterpret_cast<float4*>(c1 + 64 * q + 32), make_float4(acc[q][0][3], acc[q][1][3], acc[q][2][3], acc[q][3][3]));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// 16-bit in (bf16 or fp16) / float32 out.  One warp = one block row x one tile of 128 features;
// two blocks per m16n8k16 MMA.  Index maps:
//   k-slots 2t, 2t+1   <-> block 0, columns 2t, 2t+1      k-slots 2t+8, 2t+9 <-> block 1, same columns
//   MMA tile j: m = g   <-> feature F + 8g + j
//               m = g+8 <-> feature F + 64 + 8g + j
// A lane loads 8 consecutive 16-bit features (one 128-bit load) from each of its four B rows and
// interleaves rows pairwise with byte permutes to form the packed k-pairs the MMA wants.  Same
// two-buffer software pipeline as the float32 kernel, over pairs of blocks.
// ---------------------------------------------------------------------------------------------
struct Frag16 {
  uint4 v[4][2];   // [row][half]: rows = (blk0 col 2t), (blk0 col 2t+1), (blk1 col 2t), (blk1 col 2t+1)
  uint32_t b0, b1;
};

template <bool BF16, int MINB>
__global__ void __launch_bounds__(kThreadsBsr, MINB)
bsr8_spmm_16bit_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                       const uint16_t* __restrict__ blocks, int64_t block_row_begin, int64_t block_row_end,
                       const uint16_t* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                       int tiles) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t work = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int64_t I = block_row_begin + work / tiles;
  if (I >= block_row_end) return;
  const int F = (int)(work % tiles) * 128;

  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  const bool lo_ok = F + 8 * g < N, hi_ok = F + 64 + 8 * g < N;

  const int64_t bs = indptr[I];
  const int nblk = (int)(indptr[I + 1] - bs);
  const int npair = (nblk + 1) >> 1;
  const uint16_t* Bl = B + F + 8 * g + (int64_t)(2 * t) * ldb;
  const uint16_t* Al = blocks + g * 8 + 2 * t;
  int my_idx = 0;

  auto load = [&](Frag16& f, int p) {
    const int b = 2 * p;
    if ((b & 31) == 0) my_idx = (b + lane < nblk) ? indices[bs + b + lane] : 0;
    const bool two = b + 1 < nblk;
    const int J0 = __shfl_sync(0xffffffffu, my_idx, b & 31);
    const int J1 = __shfl_sync(0xffffffffu, my_idx, (b + 1) & 31);
    f.b0 = __ldcs(reinterpret_cast<const uint32_t*>(Al + (bs + b) * 64));
    f.b1 = two ? __ldcs(reinterpret_cast<const uint32_t*>(Al + (bs + b + 1) * 64)) : 0u;
    const uint16_t* p0 = Bl + (int64_t)J0 * 8 * ldb;
    const uint16_t* p2 = Bl + (int64_t)J1 * 8 * ldb;
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    f.v[0][0] = lo_ok ? __ldg(reinterpret_cast<const uint4*>(p0)) : z;
    f.v[1][0] = lo_ok ? __ldg(reinterpret_cast<const uint4*>(p0 + ldb)) : z;
    f.v[2][0] = (lo_ok && two) ? __ldg(reinterpret_cast<const uint4*>(p2)) : z;
    f.v[3][0] = (lo_ok && two) ? __ldg(reinterpret_cast<const uint4*>(p2 + ldb)) : z;
    f.v[0][1] = hi_ok ? __ldg(reinterpret_cast<const uint4*>(p0 + 64)) : z;
    f.v[1][1] = hi_ok ? __ldg(reinterpret_cast<const uint4*>(p0 + ldb + 64)) : z;
    f.v[2][1] = (hi_ok && two) ? __ldg(reinterpret_cast<const uint4*>(p2 + 64)) : z;
    f.v[3][1] = (hi_ok && two) ? __ldg(reinterpret_cast<const uint4*>(p2 + ldb + 64)) : z;
  };

  auto compute = [&](const Frag16& f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // feature j of the lane's 8: 32-bit word j/2, half-word j%2 of each 128-bit load
      const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;  // (hi,hi) or (lo,lo) halves of two words
      auto word = [&](const uint4& u) { return j < 2 ? u.x : (j < 4 ? u.y : (j < 6 ? u.z : u.w)); };
      uint32_t a[4];
      a[0] = __byte_perm(word(f.v[0][0]), word(f.v[1][0]), sel);  // m = g,   k = 2t, 2t+1
      a[1] = __byte_perm(word(f.v[0][1]), word(f.v[1][1]), sel);  // m = g+8, k = 2t, 2t+1
      a[2] = __byte_perm(word(f.v[2][0]), word(f.v[3][0]), sel);  // m = g,   k = 2t+8, 2t+9
      a[3] = __byte_perm(word(f.v[2][1]), word(f.v[3][1]), sel);  // m = g+8, k = 2t+8, 2t+9
      mma_16bit<BF16>(acc[j], a, f.b0, f.b1);
    }
  };

  Frag16 fa, fb;
  if (npair > 0) load(fa, 0);
  for (int p = 0; p < npair; p += 2) {
    if (p + 1 < npair) load(fb, p + 1);
    compute(fa);
    if (p + 1 < npair) {
      if (p + 2 < npair) load(fa, p + 2);
      compute(fb);
    }
  }

  float* c0 = C + ((I - block_row_begin) * 8 + 2 * t) * ldc + F + 8 * g;
  float* c1 = c0 + ldc;
#pragma unroll
  for (int h = 0; h < 2; ++h) {  // features 8g + 4h .. +3
    if (lo_ok) {
      __stcs(reinterpret_cast<float4*>(c0 + 4 * h), make_float4(acc[4 * h][0], acc[4 * h + 1][0], acc[4 * h + 2][0], acc[4 * h + 3][0]));
      __stcs(reinterpret_cast<float4*>(c1 + 4 * h), make_float4(acc[4 * h][1], acc[4 * h + 1][1], acc[4 * h + 2][1], acc[4 * h + 3][1]));
    }
    if (hi_ok) {
      __stcs(reinterpret_cast<float4*>(c0 + 64 + 4 * h), make_float4(acc[4 * h][2], acc[4 * h + 1][2], acc[4 * h + 2][2], acc[4 * h + 3][2]));
      __stcs(reinterpret_cast<float4*>(c1 + 64 + 4 * h), make_float4(acc[4 * h][3], acc[4 * h + 1][3], acc[4 * h + 2][3], acc[4 * h + 3][3]));
    }
  }
}

// tuning state of the block kernels (lf_set_option)
int g_bsr_feat_units = 0;   // 0 = automatic, 1 or 2 = features per warp / 64 of the float32 kernel
int g_bsr_min_blocks = 0;   // 0 = automatic

int check_common(const void* indptr, const void* indices, const void* blocks, int64_t r0, int64_t r1,
                 const void* B, int64_t ldb, const void* C, int64_t ldc, int N, int feat_align, int elem_b) {
  LF_REQUIRE(indptr && B && C, "null pointer argument");
  LF_REQUIRE(0 <= r0 && r0 <= r1, "bad block-row range");
  LF_REQUIRE(r0 == r1 || (indices && blocks), "block arrays missing");
  LF_REQUIRE(N >= 1 && ldb >= N && ldc >= N && ldb < (1ll << 31), "bad dense operands");
  if (N % feat_align != 0 || ldb % feat_align != 0 || ldc % 4 != 0 || (uintptr_t)B % 16 != 0 ||
      (uintptr_t)C % 16 != 0 || (uintptr_t)blocks % 8 != 0)
    return fail(LF_ERR_UNSUPPORTED,
                "the 8x8 block kernel needs N and ldb to be multiples of %d elements, ldc a multiple of 4 and "
                "16-byte aligned B and C (use the composed-format or CSR entry points otherwise)", feat_align);
  (void)elem_b;
  return LF_OK;
}

}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

int lf_bsr_set_tuning(int32_t feat_units, int32_t min_blocks) {
  LF_REQUIRE(feat_units >= 0 && feat_units <= 2 && min_blocks >= 0 && min_blocks <= 3, "bad tuning values");
  g_bsr_feat_units = feat_units;
  g_bsr_min_blocks = min_blocks;
  return LF_OK;
}

int lf_spmm_bsr8_f32(const int64_t* indptr, const int32_t* indices, const float* blocks,
                     int64_t block_row_begin, int64_t block_row_end, const float* B, int64_t ldb,
                     float* C, int64_t ldc, int32_t N, void* stream) {
  if (int s = check_common(indptr, indices, blocks, block_row_begin, block_row_end, B, ldb, C, ldc, N, 4, 4)) return s;
  if (block_row_begin == block_row_end) return LF_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows = block_row_end - block_row_begin;
  const int T = g_bsr_feat_units ? g_bsr_feat_units : (N > 64 ? 2 : 1);
  const int minb = g_bsr_min_blocks ? g_bsr_min_blocks : (T == 2 ? 1 : 2);
  const int tiles = (N + 64 * T - 1) / (64 * T);
  const int64_t grid = ceil_div64(rows * tiles, kWarps);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
#define LF_BSR(T_, M_)                                                                                          \
  bsr8_spmm_f32_kernel<T_, M_><<<(unsigned)grid, kThreadsBsr, 0, st>>>(indptr, indices, blocks, block_row_begin, \
                                                                       block_row_end, B, (int)ldb, C, ldc, N, tiles)
  if (T == 2) { if (minb == 1) LF_BSR(2, 1); else if (minb == 2) LF_BSR(2, 2); else LF_BSR(2, 3); }
  else        { if (minb == 1) LF_BSR(1, 1); else if (minb == 2) LF_BSR(1, 2); else LF_BSR(1, 3); }
#undef LF_BSR
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

static int launch_16bit(bool bf16, const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                        int64_t r0, int64_t r1, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int32_t N,
                        void* stream) {
  if (int s = check_common(indptr, indices, blocks, r0, r1, B, ldb, C, ldc, N, 8, 2)) return s;
  if (r0 == r1) return LF_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int tiles = (N + 127) / 128;
  const int64_t grid = ceil_div64((r1 - r0) * tiles, kWarps);
  LF_REQUIRE(grid < (1ll << 31), "too many thread blocks");
  const int minb = g_bsr_min_blocks ? g_bsr_min_blocks : 2;
#define LF_BSR16(B_, M_)                                                                                        \
  bsr8_spmm_16bit_kernel<B_, M_><<<(unsigned)grid, kThreadsBsr, 0, st>>>(indptr, indices, blocks, r0, r1, B,     \
                                                                         (int)ldb, C, ldc, N, tiles)
  if (bf16) { if (minb == 1) LF_BSR16(true, 1); else if (minb == 2) LF_BSR16(true, 2); else LF_BSR16(true, 3); }
  else      { if (minb == 1) LF_BSR16(false, 1); else if (minb == 2) LF_BSR16(false, 2); else LF_BSR16(false, 3); }
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
