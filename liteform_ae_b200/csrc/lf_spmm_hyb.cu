// SpMM over the composed format: C[r, :] (=|+=) sum over the ELL rows carrying row id r of
// sum_j vals[i, j] * B[cols[i, j], :].
//
// Takes over the kernel the reference generates through SparseTIR/TVM at run time
// (playground_pipline/format_algos.py:388-605; the arithmetic is format_algos.py:99-102 over the
// ELL axes of format_algos.py:55-70, the launch shape format_algos.py:503-539).  Like the
// reference, every (partition, bucket) pair runs inside ONE launch; unlike it, a thread group
// walks a contiguous run of ELL rows and keeps the running sum in registers while the row id does
// not change, so that only runs cut by a group boundary (or by column partitioning) need an
// atomic: the reference issues one atomicAdd per ELL row of every widest bucket
// (format_algos.py:508-515).
//
// Work decomposition (hand-written for sm_100a, HBM/L2-bound):
//   * G lanes (8, 16 or 32) form a group; lane l of the group owns features [f0 + 4*l, +4) of V
//     consecutive G*4-wide feature chunks, so one B-row gather is a 128-bit load per lane and a
//     fully coalesced 128..512 B segment per group;
//   * the group reads the (col, val) slots and row ids of its ELL rows G at a time, coalesced,
//     parks them in shared memory and broadcasts one pair per gather with a 64-bit shared load;
//     U gathers are issued back to back before any FMA consumes them;
//   * the kernel is specialised on min(width, 8): a row id is compared only where an ELL row can
//     start, so buckets of width >= 8 pay one check per 8 gathers;
//   * padded slots issue no gather.  Padding is recognised by its stored value 0 (the builder writes
//     exact zeros there); a stored ENTRY whose value is exactly 0 is skipped the same way, so
//     0 * Inf and 0 * NaN from B do not reach C (SciPy would produce NaN there);
//   * by default the products with 128-bit gathers run a second form of the same walk whose gathers
//     land in a per-lane shared-memory ring (cp.async, 16 rows ahead) instead of registers: see
//     spmm_hyb_ring_kernel (rows of B that fill a warp) and spmm_hyb_ring_rows_kernel (rows of 8
//     or 16 lanes, several slots per step);
//   * variants of the same code: B in bf16 (8 features per lane), and a broadcasting epilogue that
//     stores every row into several full-size C matrices (the GPUs of a group) at once.
#include <type_traits>

#include "lf_bsr8_tma.cuh"
#include "lf_common.cuh"

namespace lf {
namespace {

constexpr int kThreads = 256;

struct BucketDesc {
  int64_t row_off;        // first element of this bucket in the rows arena
  int64_t slot_off;       // first element in the cols / vals arenas
  int64_t ell_rows;       // R
  int64_t tile_begin;     // bucket-major order: first thread block of this bucket;
                          // interleaved order: first thread block of this bucket inside a segment
  int32_t wlog;           // log2(width)
  int32_t rows_per_group; // ELL rows one group walks
  int32_t force_atomic;   // every flush of this bucket must be an atomic add
  int32_t tiles_per_seg;  // interleaved order: thread blocks of this bucket per segment
};

// Order of the thread blocks.  Bucket-major (seg_tiles == 0): all thread blocks of bucket 0, then
// bucket 1, ...  Interleaved (seg_tiles > 0): every bucket is cut into the same number of
// segments (consecutive ELL rows, hence consecutive matrix rows) and the launch runs segment 0 of
// all buckets, then segment 1, ...: thread blocks that are resident together then work on the
// same stretch of matrix rows in every bucket.
template <int MAXB>
struct SpmmTable {
  int32_t n;
  int32_t seg_tiles;      // thread blocks per segment over all buckets (0 = bucket-major)
  BucketDesc b[MAXB];
};

// Destinations of a broadcasting launch: full-size C matrices (row 0 first), one per GPU of the
// group, addressed through peer mappings; the shard's rows are written into every one of them.
struct DestList {
  float* p[LF_MAX_DESTS];
  int32_t n;
  int32_t pad_;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Programmatic dependent launch: the product kernel is launched while the launch that clears
// rows is still running; everything up to this point (bucket look-up, first loads) overlaps with
// it, and nothing is written to C before the clearing launch has completed and flushed.  Without
// a programmatic dependency the instruction returns at once.
__device__ __forceinline__ void wait_for_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <int VEC> struct Chunk;
template <> struct Chunk<4> {
  float4 v;
  __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void load(const float* p) { v = __ldg(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void store_stream(float* p) const { __stcs(reinterpret_cast<float4*>(p), v); }
  __device__ __forceinline__ void fma(float a, const Chunk& x) {
    v.x = fmaf(a, x.v.x, v.x); v.y = fmaf(a, x.v.y, v.y); v.z = fmaf(a, x.v.z, v.z); v.w = fmaf(a, x.v.w, v.w);
  }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ void red(float* p) const { red_add_v4(p, v.x, v.y, v.z, v.w); }
};
template <> struct Chunk<1> {
  float v;
  __device__ __forceinline__ void zero() { v = 0.f; }
  __device__ __forceinline__ void load(const float* p) { v = __ldg(p); }
  __device__ __forceinline__ void store_stream(float* p) const { __stcs(p, v); }
  __device__ __forceinline__ void fma(float a, const Chunk& x) { v = fmaf(a, x.v, v); }
  __device__ __forceinline__ void store(float* p) const { *p = v; }
  __device__ __forceinline__ void red(float* p) const { atomicAdd(p, v); }
};

// VEC = 8 stands for "B holds bf16": a lane gathers 8 consecutive 16-bit features with one
// 128-bit load and accumulates them in 8 floats (fp32 accumulation, fp32 C).
template <> struct Chunk<8> {
  float a[8];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(a[4], a[5], a[6], a[7]);
  }
  __device__ __forceinline__ void store_stream(float* p) const {
    __stcs(reinterpret_cast<float4*>(p), make_float4(a[0], a[1], a[2], a[3]));
    __stcs(reinterpret_cast<float4*>(p + 4), make_float4(a[4], a[5], a[6], a[7]));
  }
  __device__ __forceinline__ void red(float* p) const {
    red_add_v4(p, a[0], a[1], a[2], a[3]);
    red_add_v4(p + 4, a[4], a[5], a[6], a[7]);
  }
};
struct RawBf16x8 {
  uint4 v;
  __device__ __forceinline__ void zero() { v = make_uint4(0u, 0u, 0u, 0u); }
  __device__ __forceinline__ void load(const uint16_t* p) { v = __ldg(reinterpret_cast<const uint4*>(p)); }
};
// element type of B and the register image of one gathered chunk, per VEC
template <int VEC> struct BTraits { using elem = float; using raw = Chunk<VEC>; };
template <> struct BTraits<8> { using elem = uint16_t; using raw = RawBf16x8; };

__device__ __forceinline__ void chunk_fma(Chunk<4>& acc, float a, const Chunk<4>& x) { acc.fma(a, x); }
__device__ __forceinline__ void chunk_fma(Chunk<1>& acc, float a, const Chunk<1>& x) { acc.fma(a, x); }
__device__ __forceinline__ void chunk_fma(Chunk<8>& acc, float a, const RawBf16x8& x) {
  const uint32_t w[4] = {x.v.x, x.v.y, x.v.z, x.v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // a bf16 is the upper half of the float with the same value
    acc.a[2 * i] = fmaf(a, __uint_as_float(w[i] << 16), acc.a[2 * i]);
    acc.a[2 * i + 1] = fmaf(a, __uint_as_float(w[i] & 0xffff0000u), acc.a[2 * i + 1]);
  }
}

// One thread group walks the slots [s0, s1) of whole ELL rows of one bucket.
//   G lanes per group, V chunks of VEC floats per lane: one pass covers G*V*VEC features.
//   WC = min(bucket width, 8): ELL rows start every WC slots at the earliest, so the row id has to
//        be looked at only there (once per batch of 8 gathers when the bucket is 8 or wider).
//   POL selects cache behaviour: 0 = default loads/stores; 1 = slots, row ids and C use streaming
//        (evict-first) accesses, so that B rows -- the only data with reuse -- keep the L2.
// The group stages G (column, value) pairs and row ids in shared memory with one coalesced load
// each, then broadcasts a pair per gather with a single 64-bit shared load.
template <int G, int V, int VEC, int WC, int POL, bool MD>
__device__ __forceinline__ void walk_slots(const int32_t* __restrict__ rows, const int32_t* __restrict__ cols,
                                           const float* __restrict__ vals, int wlog, int64_t e0, int64_t e1,
                                           int64_t ell_rows, bool all_open,
                                           const typename BTraits<VEC>::elem* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N,
                                           int64_t row_base, int lane, unsigned gmask, int2* cv, int* rd,
                                           const DestList& dl) {
  constexpr int U = V == 1 ? 8 : (V == 2 ? 4 : 2);  // gathers in flight per lane (x V chunks)
  static_assert(G % U == 0 && 8 % U == 0, "unroll must divide the group size and the batch");
  const int first_row = rows[e0], last_row = rows[e1 - 1];
  // does the first / last run of equal row ids continue in a neighbouring group?
  const bool head_open = e0 > 0 && rows[e0 - 1] == first_row;
  const bool tail_open = e1 < ell_rows && rows[e1] == last_row;

  const int f0 = blockIdx.y * (G * V * VEC) + lane * VEC;
  bool active[V];
  Chunk<VEC> acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    active[v] = f0 + v * G * VEC < N;
    acc[v].zero();
  }
  int cur = first_row;
  wait_for_prior_grid();   // no store or atomic to C before the row-clearing launch is complete

  auto flush = [&](int row) {
    const bool open = all_open || (row == first_row && head_open) || (row == last_row && tail_open);
    const int64_t off = (int64_t)(row - row_base) * ldc + f0;
    if (MD) {   // the same row goes to every destination (peer stores / peer atomics over NVLink)
      for (int k = 0; k < dl.n; ++k) {
        float* dst = dl.p[k] + off;
#pragma unroll
        for (int v = 0; v < V; ++v) {
          if (active[v]) {
            if (open) acc[v].red(dst + v * G * VEC); else acc[v].store(dst + v * G * VEC);
          }
        }
      }
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v].zero();
      return;
    }
    float* dst = C + off;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (active[v]) {
        if (open) acc[v].red(dst + v * G * VEC);
        else if (POL >= 1) acc[v].store_stream(dst + v * G * VEC);
        else acc[v].store(dst + v * G * VEC);
      }
      acc[v].zero();
    }
  };

  const typename BTraits<VEC>::elem* __restrict__ Bf = B + f0;
  const int64_t s0 = e0 << wlog, s1 = e1 << wlog;
  for (int64_t s = s0; s < s1; s += G) {
    const int64_t idx = s + lane;
    const bool in = idx < s1;
    const int64_t cidx = in ? idx : s1 - 1;
    const int my_col = POL >= 1 ? __ldcs(cols + cidx) : cols[cidx];
    const float my_val = in ? (POL >= 1 ? __ldcs(vals + cidx) : vals[cidx]) : 0.f;
    const int my_rid = rows[cidx >> wlog];
    __syncwarp(gmask);  // the previous strip has been consumed by every lane of the group
    cv[lane] = make_int2(my_col, __float_as_int(my_val));
    rd[lane] = my_rid;
    __syncwarp(gmask);
    const int nstrip = (int)min((int64_t)G, s1 - s);
    for (int t = 0; t < nstrip; t += U) {
      float val[U];
      typename BTraits<VEC>::raw b[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int2 p = cv[t + u];
        val[u] = __int_as_float(p.y);
        const typename BTraits<VEC>::elem* src = Bf + (int64_t)p.x * ldb;
#pragma unroll
        for (int v = 0; v < V; ++v) {
          if (val[u] != 0.f && active[v]) b[u][v].load(src + v * G * VEC);
          else b[u][v].zero();
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u % WC == 0) {  // an ELL row can only start here
          const int r = rd[t + u];
          if (r != cur) {
            flush(cur);
            cur = r;
          }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) chunk_fma(acc[v], val[u], b[u][v]);
      }
    }
  }
  flush(cur);
}

// All buckets of all partitions in one launch: a thread block looks up its bucket in the table
// passed as kernel parameter and each of its groups takes a contiguous run of that bucket's ELL rows.
template <int G, int V, int VEC, int MAXB, int POL, int MINB, bool MD>
__global__ void __launch_bounds__(kThreads, MINB)
spmm_hyb_kernel(const __grid_constant__ SpmmTable<MAXB> tbl, const int32_t* __restrict__ rows_arena,
                const int32_t* __restrict__ cols_arena, const float* __restrict__ vals_arena,
                const typename BTraits<VEC>::elem* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc,
                int N, int64_t row_base, const __grid_constant__ DestList dests) {
  constexpr int GPC = kThreads / G;  // groups per thread block
  __shared__ int2 s_cv[kThreads];
  __shared__ int s_rd[kThreads];

  int64_t tile = blockIdx.x;   // position of this thread block inside its bucket, once found
  int64_t key = tile;
  uint32_t seg = 0;
  if (tbl.seg_tiles > 0) {
    seg = (uint32_t)blockIdx.x / (uint32_t)tbl.seg_tiles;
    key = (uint32_t)blockIdx.x - seg * (uint32_t)tbl.seg_tiles;
  }
  int lo = 0, hi = tbl.n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tbl.b[mid].tile_begin <= key) lo = mid; else hi = mid;
  }
  const BucketDesc& d = tbl.b[lo];
  tile = tbl.seg_tiles > 0 ? (int64_t)seg * d.tiles_per_seg + (key - d.tile_begin) : key - d.tile_begin;
  const int wlog = d.wlog;
  const int g = threadIdx.x / G, lane = threadIdx.x % G;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) / G * G));
  const int64_t e0 = (tile * GPC + g) * (int64_t)d.rows_per_group;
  if (e0 >= d.ell_rows) return;
  const int64_t e1 = min(e0 + d.rows_per_group, d.ell_rows);
  const int32_t* __restrict__ rows = rows_arena + d.row_off;
  const int32_t* __restrict__ cols = cols_arena + d.slot_off;
  const float* __restrict__ vals = vals_arena + d.slot_off;
  const bool all_open = d.force_atomic != 0;
  int2* cv = s_cv + g * G;
  int* rd = s_rd + g * G;
#define LF_WALK(WC_)                                                                                     \
  walk_slots<G, V, VEC, WC_, POL, MD>(rows, cols, vals, wlog, e0, e1, d.ell_rows, all_open, B, ldb, C, ldc, \
                                  N, row_base, lane, gmask, cv, rd, dests)
  switch (wlog) {
    case 0: LF_WALK(1); break;
    case 1: LF_WALK(2); break;
    case 2: LF_WALK(4); break;
    default: LF_WALK(8); break;
  }
#undef LF_WALK
}

// ---- gathers staged through a per-lane ring in shared memory --------------------------------
// The register kernel above keeps at most 8 gathered rows of B per warp in flight (32 registers per
// lane), 192 per SM at three thread blocks, and its warps spend their time waiting for them (on
// the power-law benchmark matrix: 11 stall cycles on the long scoreboard per issued instruction,
// time down by a quarter from two to three resident blocks).  This variant moves the landing zone
// of the gathers from registers to shared memory: every lane owns D slots of 16 bytes, fills
// them with cp.async up to D rows ahead of the row it is adding up, and reads back only bytes it
// copied itself, so no lane ever waits for another one.  D = 16 at three thread blocks doubles
// the rows in flight per SM; the wait for B leaves the stall profile and the kernel runs into the
// DRAM instead (98 % of the copy bandwidth on that matrix).  What it pays is a second pass of
// every gathered byte through the load/store unit, so the loop over the slots is written to issue
// as few instructions as possible: what is the same for all lanes is computed once per slot while
// a strip is staged, columns and values are read back four at a time, ring slots are compile-time
// constants and the address of a row is one multiply-add.  A warp covers 128 float32 (256 bf16)
// features, one 16-byte chunk per lane; wider feature matrices use further thread blocks along
// y.  Rows are added up in the same order as in the register kernel.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// address of row `col` of a matrix whose rows are `pitch_bytes` apart: one 32 x 32 + 64 bit multiply-add
__device__ __forceinline__ const void* row_of_b(const void* base, uint32_t col, uint32_t pitch_bytes) {
  uint64_t a;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(a) : "r"(col), "r"(pitch_bytes), "l"(reinterpret_cast<uint64_t>(base)));
  return reinterpret_cast<const void*>(a);
}

constexpr int kRingFeatures = 128;   // features one warp of the ring kernel covers

constexpr uint32_t kNoGather = 0xffffffffu;   // column of a slot that gathers nothing (padding, stored zero)

// Everything that is the same for all lanes of a warp is computed once per slot by ONE lane while
// a strip of 32 slots is staged ("gathers nothing" folded into the column index, "an ELL row with
// another row id starts here" as one bit of a warp vote), so that the loop over the slots, which
// every lane executes for every slot, is left with one address computation, one copy, one
// shared-memory load and the multiply-adds.
// VEC = 4: B in float32, a lane owns 4 features; VEC = 8: B in bf16, a lane owns 8 features -- 16 bytes
// per lane and row either way, so the ring is the same.
template <int D, int WC, int POL, bool MD, int VEC>
__device__ __forceinline__ void walk_slots_ring(const int32_t* __restrict__ rows, const int32_t* __restrict__ cols,
                                                const float* __restrict__ vals, int wlog, int64_t e0, int64_t e1,
                                                int64_t ell_rows, bool all_open,
                                                const typename BTraits<VEC>::elem* __restrict__ B, int ldb,
                                                float* __restrict__ C, int64_t ldc, int N, int64_t row_base, int lane,
                                                uint32_t* so, float* sv, int* rd, float4* ring, const DestList& dl) {
  constexpr int U = 8;   // rows per commit group; row ids can change every WC <= 8 slots
  static_assert(D % U == 0 && D >= 2 * U && D <= 32, "ring depth: 16, 24 or 32 rows (two to four groups)");
  const int first_row = rows[e0], last_row = rows[e1 - 1];
  const bool head_open = e0 > 0 && rows[e0 - 1] == first_row;
  const bool tail_open = e1 < ell_rows && rows[e1] == last_row;
  const int f0 = blockIdx.y * (32 * VEC) + lane * VEC;
  const bool active = f0 < N;
  Chunk<VEC> acc;
  acc.zero();
  int cur = first_row;

  auto flush = [&](int row) {
    const bool open = all_open || (row == first_row && head_open) || (row == last_row && tail_open);
    const int64_t off = (int64_t)(row - row_base) * ldc + f0;
    if (MD) {   // the same row goes to every destination (peer stores / peer atomics over NVLink)
      if (active) {
        for (int k = 0; k < dl.n; ++k) {
          if (open) acc.red(dl.p[k] + off); else acc.store(dl.p[k] + off);
        }
      }
    } else if (active) {
      float* dst = C + off;
      if (open) acc.red(dst);
      else if (POL >= 1) acc.store_stream(dst);
      else acc.store(dst);
    }
    acc.zero();
  };

  const typename BTraits<VEC>::elem* __restrict__ Bf = B + f0;
  const int64_t s0 = e0 << wlog, s1 = e1 << wlog;
  const int n = (int)(s1 - s0);            // a group walks a few hundred slots (one ELL row at the most if wider)
  const int nstrips = (n + 31) >> 5;
  // Offsets, values and row ids of two strips of 32 slots live in shared memory; the strip after
  // those is already on its way in registers.
  int pc = 0, pr = 0;
  float pv = 0.f;
  auto load_strip = [&](int k) {
    const int64_t idx = s0 + (int64_t)k * 32 + lane;
    const bool in = idx < s1;
    const int64_t cidx = in ? idx : s1 - 1;
    pc = POL >= 1 ? __ldcs(cols + cidx) : cols[cidx];
    pv = in ? (POL >= 1 ? __ldcs(vals + cidx) : vals[cidx]) : 0.f;
    pr = rows[cidx >> wlog];
  };
  uint32_t chg0 = 0, chg1 = 0;   // bit i: slot i of the even / odd strip carries another row id than the slot before
  int carry = first_row;         // row id of the last slot of the strip staged before
  auto store_strip = [&](int k) {
    const int h = (k & 1) * 32 + lane;
    so[h] = pv != 0.f ? (uint32_t)pc : kNoGather;
    sv[h] = pv;
    rd[h] = pr;
    int before = __shfl_up_sync(0xffffffffu, pr, 1);
    if (lane == 0) before = carry;
    const uint32_t m = __ballot_sync(0xffffffffu, pr != before);
    carry = __shfl_sync(0xffffffffu, pr, 31);
    if (k & 1) chg1 = m; else chg0 = m;
  };
  load_strip(0);
  store_strip(0);
  __syncwarp();
  if (nstrips > 1) load_strip(1);

  const float4* ring_lane = ring + lane;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring_lane);
  const uint32_t pitch = (uint32_t)ldb * (uint32_t)sizeof(typename BTraits<VEC>::elem);   // ldb < 2^30 is checked by the launch
  const uint4* so4 = reinterpret_cast<const uint4*>(so);
  const float4* sv4 = reinterpret_cast<const float4*>(sv);
  // start the copies of rows j0 .. j0+7 (j0 a multiple of 8) into ring slots SLOT .. SLOT+7 and close
  // them as one group; past the end of the range the group is empty, which keeps the number of
  // groups per iteration constant
  auto issue_batch = [&](int j0, auto slot_tag) {
    constexpr int SLOT = decltype(slot_tag)::value;
    if (j0 < nstrips * 32) {
      if ((j0 & 31) == 0 && j0 > 0) {   // first rows of strip k: its slots move from registers to shared memory
        const int k = j0 >> 5;          // (the half they overwrite held strip k-2, consumed D <= 32 rows ago)
        __syncwarp();
        store_strip(k);
        __syncwarp();
        if (k + 1 < nstrips) load_strip(k + 1);
      }
      const uint4 oa = so4[(j0 & 63) >> 2], ob = so4[((j0 & 63) >> 2) + 1];
      const uint32_t o[U] = {oa.x, oa.y, oa.z, oa.w, ob.x, ob.y, ob.z, ob.w};
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (o[u] != kNoGather && active) cp_async_16(ring_s + (uint32_t)(SLOT + u) * 512u, row_of_b(Bf, o[u], pitch));
    }
    cp_async_commit();
  };

  // compile-time loop over the D/U batches of the ring
  auto for_each_batch = [&](auto&& body) {
    body(std::integral_constant<int, 0>{});
    body(std::integral_constant<int, U>{});
    if constexpr (D > 2 * U) body(std::integral_constant<int, 2 * U>{});
    if constexpr (D > 3 * U) body(std::integral_constant<int, 3 * U>{});
  };

  for_each_batch([&](auto slot_tag) { issue_batch(decltype(slot_tag)::value, slot_tag); });
  wait_for_prior_grid();   // no store or atomic to C before the row-clearing launch is complete
  for (int jc0 = 0; jc0 < n; jc0 += D) {
    for_each_batch([&](auto slot_tag) {
      constexpr int SLOT = decltype(slot_tag)::value;
      const int jc = jc0 + SLOT;
      if (jc >= n) return;
      const float4 va = sv4[(jc & 63) >> 2], vb = sv4[((jc & 63) >> 2) + 1];
      const float val[U] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      const uint32_t starts = (((jc >> 5) & 1) ? chg1 : chg0) >> (jc & 31);   // bit u: slot jc+u starts another row
      cp_async_wait<D / U - 1>();   // all but the newest D/U - 1 groups have landed: rows jc .. jc+7 are here
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u % WC == 0 && ((starts >> u) & 1u)) {  // an ELL row can only start at a multiple of WC
          flush(cur);
          cur = rd[(jc + u) & 63];
        }
        if (val[u] != 0.f && active) {
          typename BTraits<VEC>::raw x;
          const float4 raw = ring_lane[(SLOT + u) * 32];
          if constexpr (VEC == 8) x.v = make_uint4(__float_as_uint(raw.x), __float_as_uint(raw.y), __float_as_uint(raw.z), __float_as_uint(raw.w));
          else x.v = raw;
          chunk_fma(acc, val[u], x);
        }
      }
      issue_batch(jc + D, slot_tag);   // refills exactly the ring slots read above
    });
  }
  flush(cur);
}

template <int D, int MAXB, int POL, int MINB, bool MD, int VEC>
__global__ void __launch_bounds__(kThreads, MINB)
spmm_hyb_ring_kernel(const __grid_constant__ SpmmTable<MAXB> tbl, const int32_t* __restrict__ rows_arena,
                     const int32_t* __restrict__ cols_arena, const float* __restrict__ vals_arena,
                     const typename BTraits<VEC>::elem* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc,
                     int N, int64_t row_base, const __grid_constant__ DestList dests) {
  constexpr int GPC = kThreads / 32;
  extern __shared__ __align__(16) unsigned char ring_bytes[];
  __shared__ __align__(16) uint32_t s_off[GPC * 64];
  __shared__ __align__(16) float s_val[GPC * 64];
  __shared__ int s_rd[GPC * 64];

  int64_t tile = blockIdx.x;
  int64_t key = tile;
  uint32_t seg = 0;
  if (tbl.seg_tiles > 0) {
    seg = (uint32_t)blockIdx.x / (uint32_t)tbl.seg_tiles;
    key = (uint32_t)blockIdx.x - seg * (uint32_t)tbl.seg_tiles;
  }
  int lo = 0, hi = tbl.n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tbl.b[mid].tile_begin <= key) lo = mid; else hi = mid;
  }
  const BucketDesc& d = tbl.b[lo];
  tile = tbl.seg_tiles > 0 ? (int64_t)seg * d.tiles_per_seg + (key - d.tile_begin) : key - d.tile_begin;
  const int wlog = d.wlog;
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t e0 = (tile * GPC + g) * (int64_t)d.rows_per_group;
  if (e0 >= d.ell_rows) return;
  const int64_t e1 = min(e0 + d.rows_per_group, d.ell_rows);
  const int32_t* __restrict__ rows = rows_arena + d.row_off;
  const int32_t* __restrict__ cols = cols_arena + d.slot_off;
  const float* __restrict__ vals = vals_arena + d.slot_off;
  const bool all_open = d.force_atomic != 0;
  float4* ring = reinterpret_cast<float4*>(ring_bytes) + (size_t)g * D * 32;
#define LF_WALK(WC_)                                                                                       \
  walk_slots_ring<D, WC_, POL, MD, VEC>(rows, cols, vals, wlog, e0, e1, d.ell_rows, all_open, B, ldb, C, ldc, N, \
                                        row_base, lane, s_off + g * 64, s_val + g * 64, s_rd + g * 64, ring, dests)
  switch (wlog) {
    case 0: LF_WALK(1); break;
    case 1: LF_WALK(2); break;
    case 2: LF_WALK(4); break;
    default: LF_WALK(8); break;
  }
#undef LF_WALK
}

// ---- the same ring for rows of B that fill half or a quarter of a warp ------------------------
// Up to 64 float32 (128 bf16) features a row of B is 8 or 16 lanes wide.  A warp then takes R = 4 or
// 2 consecutive slots per step: lanes [h * 32/R, (h+1) * 32/R) copy and multiply the row of slot
// R * step + h, every lane keeps the partial sum of its own quarter / half, and a flush adds the R
// partial sums with shuffles before the first 32/R lanes write the row.  All R slots of a step lie
// in one ELL row (buckets at least R wide; narrower buckets go to the register kernel in a launch
// of their own), so row changes stay the same for all lanes.  Columns and values of a strip are
// staged per part (part h of a strip holds slots h, h + R, ...) so that a lane still reads the
// next four of its own with one 128-bit load.
__device__ __forceinline__ void chunk_add_from_lane_xor(Chunk<4>& a, int m) {
  a.v.x += __shfl_xor_sync(0xffffffffu, a.v.x, m);
  a.v.y += __shfl_xor_sync(0xffffffffu, a.v.y, m);
  a.v.z += __shfl_xor_sync(0xffffffffu, a.v.z, m);
  a.v.w += __shfl_xor_sync(0xffffffffu, a.v.w, m);
}
__device__ __forceinline__ void chunk_add_from_lane_xor(Chunk<8>& a, int m) {
#pragma unroll
  for (int i = 0; i < 8; ++i) a.a[i] += __shfl_xor_sync(0xffffffffu, a.a[i], m);
}

template <int R, int VEC, int WCS, int POL>
__device__ __forceinline__ void walk_slots_ring_rows(const int32_t* __restrict__ rows, const int32_t* __restrict__ cols,
                                                     const float* __restrict__ vals, int wlog, int64_t e0, int64_t e1,
                                                     int64_t ell_rows, bool all_open,
                                                     const typename BTraits<VEC>::elem* __restrict__ B, int ldb,
                                                     float* __restrict__ C, int64_t ldc, int N, int64_t row_base,
                                                     int lane, uint32_t* so, float* sv, int* rd, float4* ring) {
  constexpr int U = 8, D = 16;               // steps per commit group, steps in flight
  constexpr int G = 32 / R;                  // lanes per row of B
  constexpr int SPS = 32 / R;                // steps per strip of 32 slots
  constexpr int NB = (D * R + 31) / 32 + 1;  // strips held in shared memory: the one being added up and those ahead
  static_assert(R == 2 || R == 4, "two or four rows per step");
  const int sub = lane / G, gl = lane % G;
  const int first_row = rows[e0], last_row = rows[e1 - 1];
  const bool head_open = e0 > 0 && rows[e0 - 1] == first_row;
  const bool tail_open = e1 < ell_rows && rows[e1] == last_row;
  const int f0 = blockIdx.y * (G * VEC) + gl * VEC;
  const bool active = f0 < N;
  Chunk<VEC> acc;
  acc.zero();
  int cur = first_row;

  auto flush = [&](int row) {
#pragma unroll
    for (int m = 16; m >= G; m >>= 1) chunk_add_from_lane_xor(acc, m);   // sum over the R parts of the warp
    const bool open = all_open || (row == first_row && head_open) || (row == last_row && tail_open);
    if (active && sub == 0) {
      float* dst = C + (int64_t)(row - row_base) * ldc + f0;
      if (open) acc.red(dst);
      else if (POL >= 1) acc.store_stream(dst);
      else acc.store(dst);
    }
    acc.zero();
  };

  const typename BTraits<VEC>::elem* __restrict__ Bf = B + f0;
  const int64_t s0 = e0 << wlog, s1 = e1 << wlog;
  const int n = (int)(s1 - s0);
  const int nsteps = n / R;                  // the bucket is at least R wide: whole steps
  const int nstrips = (n + 31) >> 5;
  int pc = 0, pr = 0;
  float pv = 0.f;
  auto load_strip = [&](int k) {
    const int64_t idx = s0 + (int64_t)k * 32 + lane;
    const bool in = idx < s1;
    const int64_t cidx = in ? idx : s1 - 1;
    pc = POL >= 1 ? __ldcs(cols + cidx) : cols[cidx];
    pv = in ? (POL >= 1 ? __ldcs(vals + cidx) : vals[cidx]) : 0.f;
    pr = rows[cidx >> wlog];
  };
  uint32_t chg0 = 0, chg1 = 0, chg2 = 0;   // per resident strip: bit i = slot i carries another row id than the slot before
  int carry = first_row;
  auto store_strip = [&](int k) {
    const int hb = k % NB;
    const int at = hb * 32 + (lane % R) * SPS + lane / R;   // part (slot % R), position slot / R
    so[at] = pv != 0.f ? (uint32_t)pc : kNoGather;
    sv[at] = pv;
    rd[hb * 32 + lane] = pr;
    int before = __shfl_up_sync(0xffffffffu, pr, 1);
    if (lane == 0) before = carry;
    const uint32_t m = __ballot_sync(0xffffffffu, pr != before);
    carry = __shfl_sync(0xffffffffu, pr, 31);
    if (hb == 0) chg0 = m; else if (hb == 1) chg1 = m; else chg2 = m;
  };
  load_strip(0);
  store_strip(0);
  __syncwarp();
  if (nstrips > 1) load_strip(1);

  const float4* ring_lane = ring + lane;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring_lane);
  const uint32_t pitch = (uint32_t)ldb * (uint32_t)sizeof(typename BTraits<VEC>::elem);
  const uint4* so4 = reinterpret_cast<const uint4*>(so);
  const float4* sv4 = reinterpret_cast<const float4*>(sv);
  // steps j0 .. j0+7 (j0 a multiple of 8) into ring slots SLOT .. SLOT+7, closed as one group
  auto issue_batch = [&](int j0, auto slot_tag) {
    constexpr int SLOT = decltype(slot_tag)::value;
    if (j0 < nstrips * SPS) {
      const int k = j0 / SPS, q0 = j0 % SPS;
      if (q0 == 0 && j0 > 0) {   // first steps of strip k: its slots move from registers to shared memory
        __syncwarp();
        store_strip(k);
        __syncwarp();
        if (k + 1 < nstrips) load_strip(k + 1);
      }
      const int at = (k % NB) * 32 + sub * SPS + q0;
      const uint4 oa = so4[at >> 2], ob = so4[(at >> 2) + 1];
      const uint32_t o[U] = {oa.x, oa.y, oa.z, oa.w, ob.x, ob.y, ob.z, ob.w};
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (o[u] != kNoGather && active) cp_async_16(ring_s + (uint32_t)(SLOT + u) * 512u, row_of_b(Bf, o[u], pitch));
    }
    cp_async_commit();
  };
  auto for_each_batch = [&](auto&& body) {
    body(std::integral_constant<int, 0>{});
    body(std::integral_constant<int, U>{});
  };

  for_each_batch([&](auto slot_tag) { issue_batch(decltype(slot_tag)::value, slot_tag); });
  wait_for_prior_grid();   // no store or atomic to C before the row-clearing launch is complete
  for (int jc0 = 0; jc0 < nsteps; jc0 += D) {
    for_each_batch([&](auto slot_tag) {
      constexpr int SLOT = decltype(slot_tag)::value;
      const int jc = jc0 + SLOT;
      if (jc >= nsteps) return;
      const int k = jc / SPS, q0 = jc % SPS, hb = k % NB;
      const int at = hb * 32 + sub * SPS + q0;
      const float4 va = sv4[at >> 2], vb = sv4[(at >> 2) + 1];
      const float val[U] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      const uint32_t starts = (hb == 0 ? chg0 : (hb == 1 ? chg1 : chg2)) >> (q0 * R);   // bit u*R: step jc+u starts another row
      cp_async_wait<D / U - 1>();
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (u % WCS == 0 && ((starts >> (u * R)) & 1u)) {  // an ELL row can only start at a multiple of width / R steps
          flush(cur);
          cur = rd[hb * 32 + (q0 + u) * R];
        }
        if (val[u] != 0.f && active) {
          typename BTraits<VEC>::raw x;
          const float4 raw = ring_lane[(SLOT + u) * 32];
          if constexpr (VEC == 8) x.v = make_uint4(__float_as_uint(raw.x), __float_as_uint(raw.y), __float_as_uint(raw.z), __float_as_uint(raw.w));
          else x.v = raw;
          chunk_fma(acc, val[u], x);
        }
      }
      issue_batch(jc + D, slot_tag);
    });
  }
  flush(cur);
}

template <int R, int VEC, int MAXB, int POL>
__global__ void __launch_bounds__(kThreads, 3)
spmm_hyb_ring_rows_kernel(const __grid_constant__ SpmmTable<MAXB> tbl, const int32_t* __restrict__ rows_arena,
                          const int32_t* __restrict__ cols_arena, const float* __restrict__ vals_arena,
                          const typename BTraits<VEC>::elem* __restrict__ B, int ldb, float* __restrict__ C,
                          int64_t ldc, int N, int64_t row_base) {
  constexpr int GPC = kThreads / 32;
  constexpr int NB = (16 * R + 31) / 32 + 1;
  constexpr int LR = R == 2 ? 1 : 2;
  extern __shared__ __align__(16) unsigned char ring_bytes[];
  __shared__ __align__(16) uint32_t s_off[GPC * NB * 32];
  __shared__ __align__(16) float s_val[GPC * NB * 32];
  __shared__ int s_rd[GPC * NB * 32];

  int64_t tile = blockIdx.x;
  int64_t key = tile;
  uint32_t seg = 0;
  if (tbl.seg_tiles > 0) {
    seg = (uint32_t)blockIdx.x / (uint32_t)tbl.seg_tiles;
    key = (uint32_t)blockIdx.x - seg * (uint32_t)tbl.seg_tiles;
  }
  int lo = 0, hi = tbl.n;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tbl.b[mid].tile_begin <= key) lo = mid; else hi = mid;
  }
  const BucketDesc& d = tbl.b[lo];
  tile = tbl.seg_tiles > 0 ? (int64_t)seg * d.tiles_per_seg + (key - d.tile_begin) : key - d.tile_begin;
  const int wlog = d.wlog;
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t e0 = (tile * GPC + g) * (int64_t)d.rows_per_group;
  if (e0 >= d.ell_rows) return;
  const int64_t e1 = min(e0 + d.rows_per_group, d.ell_rows);
  const int32_t* __restrict__ rows = rows_arena + d.row_off;
  const int32_t* __restrict__ cols = cols_arena + d.slot_off;
  const float* __restrict__ vals = vals_arena + d.slot_off;
  const bool all_open = d.force_atomic != 0;
  float4* ring = reinterpret_cast<float4*>(ring_bytes) + (size_t)g * 16 * 32;
#define LF_WALK(WCS_)                                                                                            \
  walk_slots_ring_rows<R, VEC, WCS_, POL>(rows, cols, vals, wlog, e0, e1, d.ell_rows, all_open, B, ldb, C, ldc, N, \
                                          row_base, lane, s_off + g * NB * 32, s_val + g * NB * 32,               \
                                          s_rd + g * NB * 32, ring)
  switch (wlog - LR) {   // width / R steps per ELL row
    case 0: LF_WALK(1); break;
    case 1: LF_WALK(2); break;
    case 2: LF_WALK(4); break;
    default: LF_WALK(8); break;
  }
#undef LF_WALK
}

// Rows that no single ELL row owns are cleared before the accumulating launch.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
zero_rows_kernel(const int32_t* __restrict__ zero_rows, int64_t n, float* __restrict__ C, int64_t ldc,
                 int N, int64_t row_base) {
  let_dependents_launch();   // the product kernel may become resident; it waits before touching C
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t i = warp; i < n; i += n_warps) {
    float* dst = C + (int64_t)(zero_rows[i] - row_base) * ldc;
    if (VEC == 4) {
      for (int f = lane * 4; f < N; f += 128) *reinterpret_cast<float4*>(dst + f) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int f = lane; f < N; f += 32) dst[f] = 0.f;
    }
  }
}

// Same for a broadcasting launch: the rows are cleared in every destination.
__global__ void __launch_bounds__(kThreads)
zero_rows_multi_kernel(const int32_t* __restrict__ zero_rows, int64_t n, const __grid_constant__ DestList dests,
                       int64_t ldc, int N) {
  let_dependents_launch();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t i = warp; i < n; i += n_warps) {
    const int64_t off = (int64_t)zero_rows[i] * ldc;
    for (int k = 0; k < dests.n; ++k)
      for (int f = lane * 4; f < N; f += 128)
        *reinterpret_cast<float4*>(dests.p[k] + off + f) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// CSR SpMM (the kernel behind bench_naive, format_algos.py:1660-1755), balanced over entries
// instead of rows: every thread group takes `spg` consecutive stored entries, whatever rows they
// belong to, so a 100 000-entry row is shared by hundreds of groups and short rows are packed
// together.  A row that lies inside one group's range is written with a plain store; a row cut
// by a range boundary is accumulated with vector atomics after csr_prepare_kernel cleared it.
// ---------------------------------------------------------------------------------------------
// One warp per candidate: lane 0 decides which rows (at most two) have to be cleared, the warp
// clears them with coalesced (128-bit when VEC == 4) stores.
template <int VEC>
__global__ void __launch_bounds__(256)
csr_prepare_kernel(const int64_t* __restrict__ indptr, int64_t row_begin, int64_t row_end, int64_t spg,
                   float* __restrict__ C, int64_t ldc, int N) {
  let_dependents_launch();
  const int lane = threadIdx.x & 31;
  const int64_t rows = row_end - row_begin;
  const int64_t base = indptr[row_begin];
  const int64_t total = indptr[row_end] - base;
  const int64_t groups = (total + spg - 1) / spg;
  const int64_t n = rows > groups ? rows : groups;
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  auto clear = [&](int64_t row) {
    float* dst = C + row * ldc;
    if (VEC == 4) {
      for (int f = lane * 4; f < N; f += 128) *reinterpret_cast<float4*>(dst + f) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int f = lane; f < N; f += 32) dst[f] = 0.f;
    }
  };
  for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += n_warps) {
    int64_t empty_row = -1, cut_row = -1;
    if (lane == 0) {
      if (i < rows && indptr[row_begin + i] == indptr[row_begin + i + 1]) empty_row = i;
      if (i >= 1 && i < groups) {   // the row that contains the first entry of group i, if it started earlier
        const int64_t x = base + i * spg;
        int64_t lo = row_begin, hi = row_end;   // indptr[lo] <= x, answer in [lo, hi)
        while (hi - lo > 1) {
          const int64_t mid = (lo + hi) >> 1;
          if (indptr[mid] <= x) lo = mid; else hi = mid;
        }
        if (indptr[lo] < x) cut_row = lo - row_begin;
      }
    }
    empty_row = __shfl_sync(0xffffffffu, empty_row, 0);
    cut_row = __shfl_sync(0xffffffffu, cut_row, 0);
    if (empty_row >= 0) clear(empty_row);
    if (cut_row >= 0) clear(cut_row);
  }
}

template <int G, int V, int VEC>
__global__ void __launch_bounds__(kThreads, 3)
spmm_csr_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                const float* __restrict__ data, int64_t row_begin, int64_t row_end,
                const float* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N, int spg) {
  constexpr int GPC = kThreads / G;
  constexpr int U = V == 1 ? 8 : (V == 2 ? 4 : 2);
  __shared__ int2 s_cv[kThreads];
  __shared__ int64_t s_bd[kThreads];
  const int g = threadIdx.x / G, lane = threadIdx.x % G;
  const int shift = (threadIdx.x & 31) / G * G;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << shift);
  const int64_t base = indptr[row_begin];
  const int64_t total = indptr[row_end] - base;
  const int64_t s0 = ((int64_t)blockIdx.x * GPC + g) * (int64_t)spg;
  if (s0 >= total) return;
  const int64_t s1 = min(s0 + spg, total);
  int2* cv = s_cv + g * G;
  int64_t* bd = s_bd + g * G;

  // (G+1)-ary search, one probe per lane: the row that holds entry s0
  int64_t lo = row_begin, hi = row_end;   // indptr[lo] - base <= s0, answer in [lo, hi)
  while (hi - lo > 1) {
    const int64_t span = hi - lo;
    int64_t q = lo + ((int64_t)(lane + 1) * span) / (G + 1);
    if (q <= lo) q = lo + 1;
    const bool le = indptr[q] - base <= s0;
    const int cnt = __popc((__ballot_sync(gmask, le) & gmask) >> shift);   // probes are monotone
    const int64_t qlo = __shfl_sync(gmask, q, cnt > 0 ? cnt - 1 : 0, G);
    const int64_t qhi = __shfl_sync(gmask, q, cnt < G ? cnt : G - 1, G);
    if (cnt > 0) lo = qlo;
    if (cnt < G) hi = qhi;
  }
  int64_t cur = lo;
  const int64_t first_row = cur;
  const bool head_open = indptr[cur] - base < s0;

  // boundaries of the next G rows, refilled when used up
  int kb = 0;
  auto refill = [&]() {
    __syncwarp(gmask);
    const int64_t r = cur + 1 + lane;
    bd[lane] = indptr[r < row_end ? r : row_end] - base;
    __syncwarp(gmask);
    kb = 0;
  };
  refill();
  int64_t nb = bd[0];   // first entry of the next row

  const int f0 = blockIdx.y * (G * V * VEC) + lane * VEC;
  bool active[V];
  Chunk<VEC> acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) { active[v] = f0 + v * G * VEC < N; acc[v].zero(); }

  auto flush = [&](int64_t row, bool open) {
    float* dst = C + (row - row_begin) * ldc + f0;
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (active[v]) {
        if (open) acc[v].red(dst + v * G * VEC); else acc[v].store_stream(dst + v * G * VEC);
      }
      acc[v].zero();
    }
  };

  const float* __restrict__ Bf = B + f0;
  wait_for_prior_grid();   // csr_prepare_kernel has cleared the rows that receive atomics
  for (int64_t s = s0; s < s1; s += G) {
    const int64_t idx = s + lane;
    const bool in = idx < s1;
    const int my_col = in ? __ldcs(indices + base + idx) : 0;
    const float my_val = in ? (data ? __ldcs(data + base + idx) : 1.f) : 0.f;
    __syncwarp(gmask);
    cv[lane] = make_int2(my_col, __float_as_int(my_val));
    __syncwarp(gmask);
    const int nstrip = (int)min((int64_t)G, s1 - s);
    for (int t = 0; t < nstrip; t += U) {
      float val[U];
      Chunk<VEC> b[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int2 p = cv[t + u];
        val[u] = __int_as_float(p.y);
        const float* src = Bf + (int64_t)p.x * ldb;
#pragma unroll
        for (int v = 0; v < V; ++v) {
          if (val[u] != 0.f && active[v]) b[u][v].load(src + v * G * VEC); else b[u][v].zero();
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t pos = s + t + u;
        if (pos < s1) {
          while (pos == nb) {   // the current row ended here (and empty rows may follow)
            flush(cur, cur == first_row && head_open);
            ++cur;
            if (++kb == G) refill();
            nb = bd[kb];
          }
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v].fma(val[u], b[u][v]);
        }
      }
    }
  }
  flush(cur, (cur == first_row && head_open) || s1 < nb);
}

// The CSR product with the gathers staged through the same per-lane shared-memory ring as
// spmm_hyb_ring_kernel: a warp takes `spg` consecutive entries and 128 features, copies rows of B
// 16 entries ahead of the one it is adding up, and follows the row boundaries exactly like the
// register kernel above (same order of additions, same flush rules).
template <int D>
__global__ void __launch_bounds__(kThreads, 3)
spmm_csr_ring_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                     const float* __restrict__ data, int64_t row_begin, int64_t row_end,
                     const float* __restrict__ B, int ldb, float* __restrict__ C, int64_t ldc, int N, int spg) {
  constexpr int GPC = kThreads / 32, U = 8;
  static_assert(D == 2 * U, "two commit groups of eight rows");
  extern __shared__ __align__(16) unsigned char ring_bytes[];
  __shared__ __align__(16) uint32_t s_off[GPC * 64];
  __shared__ __align__(16) float s_val[GPC * 64];
  __shared__ int64_t s_bd[kThreads];
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = indptr[row_begin];
  const int64_t total = indptr[row_end] - base;
  const int64_t s0 = ((int64_t)blockIdx.x * GPC + g) * (int64_t)spg;
  if (s0 >= total) return;
  const int64_t s1 = min(s0 + spg, total);
  uint32_t* so = s_off + g * 64;
  float* sv = s_val + g * 64;
  int64_t* bd = s_bd + g * 32;

  // 33-ary search, one probe per lane: the row that holds entry s0
  int64_t lo = row_begin, hi = row_end;   // indptr[lo] - base <= s0, answer in [lo, hi)
  while (hi - lo > 1) {
    const int64_t span = hi - lo;
    int64_t q = lo + ((int64_t)(lane + 1) * span) / 33;
    if (q <= lo) q = lo + 1;
    const bool le = indptr[q] - base <= s0;
    const int cnt = __popc(__ballot_sync(0xffffffffu, le));   // probes are monotone
    const int64_t qlo = __shfl_sync(0xffffffffu, q, cnt > 0 ? cnt - 1 : 0);
    const int64_t qhi = __shfl_sync(0xffffffffu, q, cnt < 32 ? cnt : 31);
    if (cnt > 0) lo = qlo;
    if (cnt < 32) hi = qhi;
  }
  int64_t cur = lo;
  const int64_t first_row = cur;
  const bool head_open = indptr[cur] - base < s0;

  int kb = 0;   // boundaries of the next 32 rows, refilled when used up
  auto refill = [&]() {
    __syncwarp();
    const int64_t r = cur + 1 + lane;
    bd[lane] = indptr[r < row_end ? r : row_end] - base;
    __syncwarp();
    kb = 0;
  };
  refill();
  int64_t nb = bd[0];   // first entry of the next row

  const int f0 = blockIdx.y * kRingFeatures + lane * 4;
  const bool active = f0 < N;
  Chunk<4> acc;
  acc.zero();
  auto flush = [&](int64_t row, bool open) {
    float* dst = C + (row - row_begin) * ldc + f0;
    if (active) {
      if (open) acc.red(dst); else acc.store_stream(dst);
    }
    acc.zero();
  };

  const float* __restrict__ Bf = B + f0;
  const int n = (int)(s1 - s0);
  const int nstrips = (n + 31) >> 5;
  int pc = 0;
  float pv = 0.f;
  auto load_strip = [&](int k) {
    const int64_t idx = s0 + (int64_t)k * 32 + lane;
    const bool in = idx < s1;
    pc = in ? __ldcs(indices + base + idx) : 0;
    pv = in ? (data ? __ldcs(data + base + idx) : 1.f) : 0.f;
  };
  auto store_strip = [&](int k) {
    const int h = (k & 1) * 32 + lane;
    so[h] = pv != 0.f ? (uint32_t)pc : kNoGather;
    sv[h] = pv;
  };
  load_strip(0);
  store_strip(0);
  __syncwarp();
  if (nstrips > 1) load_strip(1);

  const float4* ring_lane = reinterpret_cast<const float4*>(ring_bytes) + (size_t)g * D * 32 + lane;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring_lane);
  const uint32_t pitch = (uint32_t)ldb * 4u;
  const uint4* so4 = reinterpret_cast<const uint4*>(so);
  const float4* sv4 = reinterpret_cast<const float4*>(sv);
  auto issue_batch = [&](int j0, auto slot_tag) {
    constexpr int SLOT = decltype(slot_tag)::value;
    if (j0 < nstrips * 32) {
      if ((j0 & 31) == 0 && j0 > 0) {
        const int k = j0 >> 5;
        __syncwarp();
        store_strip(k);
        __syncwarp();
        if (k + 1 < nstrips) load_strip(k + 1);
      }
      const uint4 oa = so4[(j0 & 63) >> 2], ob = so4[((j0 & 63) >> 2) + 1];
      const uint32_t o[U] = {oa.x, oa.y, oa.z, oa.w, ob.x, ob.y, ob.z, ob.w};
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (o[u] != kNoGather && active) cp_async_16(ring_s + (uint32_t)(SLOT + u) * 512u, row_of_b(Bf, o[u], pitch));
    }
    cp_async_commit();
  };
  auto for_each_batch = [&](auto&& body) {
    body(std::integral_constant<int, 0>{});
    body(std::integral_constant<int, U>{});
  };

  for_each_batch([&](auto slot_tag) { issue_batch(decltype(slot_tag)::value, slot_tag); });
  wait_for_prior_grid();   // csr_prepare_kernel has cleared the rows that receive atomics
  for (int jc0 = 0; jc0 < n; jc0 += D) {
    for_each_batch([&](auto slot_tag) {
      constexpr int SLOT = decltype(slot_tag)::value;
      const int jc = jc0 + SLOT;
      if (jc >= n) return;
      const float4 va = sv4[(jc & 63) >> 2], vb = sv4[((jc & 63) >> 2) + 1];
      const float val[U] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      const int64_t pos0 = s0 + jc;
      cp_async_wait<D / U - 1>();
      if (nb >= pos0 + U) {   // no row ends inside these eight entries
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (val[u] != 0.f && active) {
            Chunk<4> x;
            x.v = ring_lane[(SLOT + u) * 32];
            acc.fma(val[u], x);
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t pos = pos0 + u;
          if (pos < s1) {
            while (pos == nb) {   // the current row ended here (and empty rows may follow)
              flush(cur, cur == first_row && head_open);
              ++cur;
              if (++kb == 32) refill();
              nb = bd[kb];
            }
            if (val[u] != 0.f && active) {
              Chunk<4> x;
              x.v = ring_lane[(SLOT + u) * 32];
              acc.fma(val[u], x);
            }
          }
        }
      }
      issue_batch(jc + D, slot_tag);
    });
  }
  flush(cur, (cur == first_row && head_open) || s1 < nb);
}

// Ragged all-gather of C over peer mappings: the rows of this rank's block are read once and
// stored into the same rows of every destination (plain 128-bit peer stores over NVLink).
template <int VEC>
__global__ void __launch_bounds__(256)
allgather_rows_kernel(const float* __restrict__ src, int64_t ld_src, int64_t rows, int N, int64_t row_begin,
                      const __grid_constant__ DestList dests, int64_t ldc) {
  const int per_row = (N + VEC - 1) / VEC;
  const int64_t total = rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / per_row;
    const int f = (int)(i - r * per_row) * VEC;
    const int64_t off = (row_begin + r) * ldc + f;
    if (VEC == 4) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * ld_src + f));
      for (int k = 0; k < dests.n; ++k) *reinterpret_cast<float4*>(dests.p[k] + off) = v;
    } else {
      const float v = __ldcs(src + r * ld_src + f);
      for (int k = 0; k < dests.n; ++k) dests.p[k][off] = v;
    }
  }
}

struct FeatCfg { int G, V, VEC, pass; };

// Kernel launch with, optionally, a programmatic dependency on the previous kernel of the stream
// (the row-clearing launch): the product kernel may start before that kernel has finished and
// orders itself with griddepcontrol.wait.
template <typename... Params, typename... Args>
cudaError_t launch_dep_smem(void (*kernel)(Params...), dim3 grid, int threads, size_t smem, cudaStream_t st,
                            bool dependent, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}
template <typename... Params, typename... Args>
cudaError_t launch_dep(void (*kernel)(Params...), dim3 grid, int threads, cudaStream_t st, bool dependent, Args... args) {
  return launch_dep_smem(kernel, grid, threads, 0, st, dependent, args...);
}

FeatCfg pick_cfg(const void* B, int64_t ldb, const void* C, int64_t ldc, int N) {
  const bool vec = (N % 4 == 0) && (ldb % 4 == 0) && (ldc % 4 == 0) && ((uintptr_t)B % 16 == 0) &&
                   ((uintptr_t)C % 16 == 0);
  FeatCfg c;
  if (vec) {
    c.VEC = 4;
    if (N <= 32) { c.G = 8; c.V = 1; }
    else if (N <= 64) { c.G = 16; c.V = 1; }
    else if (N <= 128) { c.G = 32; c.V = 1; }
    else if (N <= 256) { c.G = 32; c.V = 2; }
    else { c.G = 32; c.V = 4; }
  } else {
    c.VEC = 1;
    c.G = 32;
    c.V = N <= 32 ? 1 : (N <= 64 ? 2 : 4);
  }
  c.pass = c.G * c.V * c.VEC;
  return c;
}

// bf16 B: 8 features per lane and chunk; needs N, ldb multiples of 8 and 16-byte aligned bases
FeatCfg pick_cfg_bf16(int N) {
  FeatCfg c;
  c.VEC = 8;
  if (N <= 64) { c.G = 8; c.V = 1; }
  else if (N <= 128) { c.G = 16; c.V = 1; }
  else if (N <= 256) { c.G = 32; c.V = 1; }
  else { c.G = 32; c.V = 2; }
  c.pass = c.G * c.V * c.VEC;
  return c;
}

// Process-wide tuning knobs (lf_set_option); the environment gives the initial values.
constexpr int kDefaultGatherRing = 16;
// stored slots from which rows of B narrower than a warp take the two-launch ring path (LF_OPT_SPMM_RING_MIN_SLOTS)
int g_ring_rows_min_slots = 1 << 20;
int g_slots_per_group = 0;
int g_cache_policy = -1;

// 0 = automatic: 256 slots per group, halved (down to 32) while the launch would have fewer than
// eight waves of thread blocks, so that small shards do not lose a third of the time in the tail.
int slots_per_group() {
  static bool env_read = false;
  if (!env_read) {
    env_read = true;
    const char* e = getenv("LF_SPMM_SLOTS_PER_GROUP");
    const int v = e ? atoi(e) : 0;
    if (!g_slots_per_group && v >= 8 && v <= (1 << 20)) g_slots_per_group = v;
  }
  return g_slots_per_group;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int g_tile_segments = -1;   // 0 = bucket-major order, S > 0 = interleaved over S segments
int tile_segments() {
  if (g_tile_segments < 0) {
    const char* e = getenv("LF_SPMM_TILE_SEGMENTS");
    const int v = e ? atoi(e) : 0;
    g_tile_segments = (v >= 0 && v <= 4096) ? v : 0;
  }
  return g_tile_segments;
}

int g_min_blocks = 0;
int min_blocks() {
  if (!g_min_blocks) {
    const char* e = getenv("LF_SPMM_MIN_BLOCKS");
    const int v = e ? atoi(e) : 0;
    g_min_blocks = (v >= 2 && v <= 4) ? v : 3;
  }
  return g_min_blocks;
}

// Depth of the shared-memory gather ring (rows in flight per warp): 0 = gathers land in registers.
int g_gather_ring = -1;
int gather_ring() {
  if (g_gather_ring < 0) {
    const char* e = getenv("LF_SPMM_GATHER_RING");
    const int v = e ? atoi(e) : kDefaultGatherRing;
    g_gather_ring = (v == 0 || v == 16) ? v : kDefaultGatherRing;
  }
  return g_gather_ring;
}

int cache_policy() {
  if (g_cache_policy < 0) {
    const char* e = getenv("LF_SPMM_POLICY");
    const int v = e ? atoi(e) : 1;
    g_cache_policy = (v >= 0 && v <= 1) ? v : 1;
  }
  return g_cache_policy;
}

template <int MAXB>
int launch_hyb_bf16(const SpmmTable<MAXB>& tbl, int64_t tiles, const lf_hyb* A, const uint16_t* B, int64_t ldb,
                    float* C, int64_t ldc, int N, FeatCfg cfg, cudaStream_t st, const DestList& dests, bool dep) {
  // (rows of 8 or 16 lanes -- up to 128 features -- reach spmm_hyb_ring_rows_kernel from the bucket
  // loop of the caller; what arrives here with such rows is the register-kernel share)
  if (gather_ring() > 0 && cfg.G == 32 && ldb < (1ll << 30) && dests.n == 0) {
    // more than 128 bf16 features: full warps, one thread block along y per 256 features
    dim3 rgrid((unsigned)tiles, (unsigned)((N + 255) / 256));
    const size_t smem = (size_t)(kThreads / 32) * 16 * 32 * sizeof(float4);
    auto kern = spmm_hyb_ring_kernel<16, MAXB, 1, 3, false, 8>;
    LF_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LF_CUDA_CHECK(launch_dep_smem(kern, rgrid, kThreads, smem, st, dep, tbl, A->rows, A->cols, A->vals, B, (int)ldb, C,
                                  ldc, N, A->row_begin, dests));
    return LF_OK;
  }
  dim3 grid((unsigned)tiles, (unsigned)((N + cfg.pass - 1) / cfg.pass));
#define LF_LAUNCH(G_, V_)                                                                                   \
  LF_CUDA_CHECK(launch_dep(spmm_hyb_kernel<G_, V_, 8, MAXB, 1, 3, false>, grid, kThreads, st, dep, tbl, A->rows, \
                           A->cols, A->vals, B, (int)ldb, C, ldc, N, A->row_begin, dests))
  if (cfg.G == 8) LF_LAUNCH(8, 1);
  else if (cfg.G == 16) LF_LAUNCH(16, 1);
  else if (cfg.V == 1) LF_LAUNCH(32, 1);
  else LF_LAUNCH(32, 2);
#undef LF_LAUNCH
  return LF_OK;
}

template <int MAXB, int POL, int MINB, bool MD>
int launch_hyb_pol(const SpmmTable<MAXB>& tbl, int64_t tiles, const lf_hyb* A, const float* B, int64_t ldb,
                   float* C, int64_t ldc, int N, FeatCfg cfg, cudaStream_t st, const DestList& dests, bool dep) {
  const int64_t row_base = MD ? 0 : A->row_begin;
  dim3 grid((unsigned)tiles, (unsigned)((N + cfg.pass - 1) / cfg.pass));
#define LF_LAUNCH(G_, V_, VEC_)                                                                               \
  LF_CUDA_CHECK(launch_dep(spmm_hyb_kernel<G_, V_, VEC_, MAXB, POL, MINB, MD>, grid, kThreads, st, dep, tbl,   \
                           A->rows, A->cols, A->vals, B, (int)ldb, C, ldc, N, row_base, dests))
  if (cfg.VEC == 4) {
    if (cfg.G == 8) LF_LAUNCH(8, 1, 4);
    else if (cfg.G == 16) LF_LAUNCH(16, 1, 4);
    else if (cfg.V == 1) LF_LAUNCH(32, 1, 4);
    else if (cfg.V == 2) LF_LAUNCH(32, 2, 4);
    else LF_LAUNCH(32, 4, 4);
  } else {
    if (cfg.V == 1) LF_LAUNCH(32, 1, 1);
    else if (cfg.V == 2) LF_LAUNCH(32, 2, 1);
    else LF_LAUNCH(32, 4, 1);
  }
#undef LF_LAUNCH
  return LF_OK;
}

// Rows of B that are 8 or 16 lanes wide: the ring kernel that takes several slots per step.
template <int MAXB>
int launch_hyb_ring_rows(const SpmmTable<MAXB>& tbl, int64_t tiles, const lf_hyb* A, const void* B, bool bf16,
                         int64_t ldb, float* C, int64_t ldc, int N, int lanes_per_row, cudaStream_t st, bool dep) {
  const int vec = bf16 ? 8 : 4;
  dim3 grid((unsigned)tiles, (unsigned)((N + lanes_per_row * vec - 1) / (lanes_per_row * vec)));
  const size_t smem = (size_t)(kThreads / 32) * 16 * 32 * sizeof(float4);
#define LF_ROWS(R_, VEC_, T_)                                                                                   \
  do {                                                                                                          \
    auto kern = spmm_hyb_ring_rows_kernel<R_, VEC_, MAXB, 1>;                                                   \
    LF_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));          \
    LF_CUDA_CHECK(launch_dep_smem(kern, grid, kThreads, smem, st, dep, tbl, A->rows, A->cols, A->vals,          \
                                  (const T_*)B, (int)ldb, C, ldc, N, A->row_begin));                            \
    return LF_OK;                                                                                               \
  } while (0)
  if (bf16) { if (lanes_per_row == 16) LF_ROWS(2, 8, uint16_t); else LF_ROWS(4, 8, uint16_t); }
  else      { if (lanes_per_row == 16) LF_ROWS(2, 4, float); else LF_ROWS(4, 4, float); }
#undef LF_ROWS
}

// The ring kernels exist for 128-bit gathers over full warps; they multiply the column by a 32-bit
// row pitch in bytes.
bool ring_applies(const FeatCfg& cfg, int64_t ldb) { return cfg.VEC == 4 && cfg.G == 32 && ldb < (1ll << 30); }

template <int MAXB>
int launch_hyb(const SpmmTable<MAXB>& tbl, int64_t tiles, const lf_hyb* A, const void* Bv, int64_t ldb,
               float* C, int64_t ldc, int N, FeatCfg cfg, cudaStream_t st, const DestList& dests, bool dep) {
  if (cfg.VEC == 8)   // bf16 B: one compiled variant per feature layout
    return launch_hyb_bf16<MAXB>(tbl, tiles, A, (const uint16_t*)Bv, ldb, C, ldc, N, cfg, st, dests, dep);
  const float* B = (const float*)Bv;
  const int pol = cache_policy(), minb = min_blocks();
  const int ring = gather_ring();
  if (ring > 0 && ring_applies(cfg, ldb)) {
    // one warp per 128 features; the ring of a thread block takes depth * 4 KiB of shared memory
    dim3 grid((unsigned)tiles, (unsigned)((N + kRingFeatures - 1) / kRingFeatures));
    const size_t smem = (size_t)(kThreads / 32) * ring * 32 * sizeof(float4);
#define LF_RING(D_, P_, M_, MD_)                                                                                \
  do {                                                                                                          \
    auto kern = spmm_hyb_ring_kernel<D_, MAXB, P_, M_, MD_, 4>;                                                 \
    LF_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));          \
    LF_CUDA_CHECK(launch_dep_smem(kern, grid, kThreads, smem, st, dep, tbl, A->rows, A->cols, A->vals, B,       \
                                  (int)ldb, C, ldc, N, MD_ ? (int64_t)0 : A->row_begin, dests));                \
    return LF_OK;                                                                                               \
  } while (0)
    if (dests.n > 0) LF_RING(16, 1, 3, true);   // broadcasting launch: one compiled variant
    else if (pol == 0) LF_RING(16, 0, 3, false);
    else LF_RING(16, 1, 3, false);
#undef LF_RING
  }
  if (dests.n > 0)   // broadcasting launch: one compiled variant
    return launch_hyb_pol<MAXB, 1, 3, true>(tbl, tiles, A, B, ldb, C, ldc, N, cfg, st, dests, dep);
#define LF_CASE(P_, M_) if (pol == P_ && minb == M_) return launch_hyb_pol<MAXB, P_, M_, false>(tbl, tiles, A, B, ldb, C, ldc, N, cfg, st, dests, dep)
  LF_CASE(0, 2); LF_CASE(0, 3); LF_CASE(0, 4);
  LF_CASE(1, 2); LF_CASE(1, 3); LF_CASE(1, 4);
#undef LF_CASE
  return fail(LF_ERR_INVALID_ARGUMENT, "bad tuning state");
}

int check_hyb(const lf_hyb* A) {
  LF_REQUIRE(A, "null format descriptor");
  LF_REQUIRE(A->num_parts >= 1 && A->num_buckets >= 0, "bad partition / bucket count");
  LF_REQUIRE(A->part_bucket_off && A->ell_rows && A->row_off && A->slot_off, "format host arrays missing");
  LF_REQUIRE(A->num_buckets == 0 || A->widths, "widths missing");
  LF_REQUIRE(0 <= A->row_begin && A->row_begin <= A->row_end && A->row_end <= A->num_rows, "bad row range");
  LF_REQUIRE(A->part_bucket_off[A->num_parts] == A->num_buckets, "num_buckets does not match part_bucket_off");
  for (int i = 0; i < A->num_buckets; ++i) {
    const int w = A->widths[i];
    LF_REQUIRE(w >= 1 && (w & (w - 1)) == 0, "bucket width %d is not a power of two", w);
    LF_REQUIRE(A->ell_rows[i] >= 0, "negative ELL row count");
  }
  return LF_OK;
}

}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

int lf_set_option(int32_t option, int32_t value) {
  switch (option) {
    case LF_OPT_SPMM_SLOTS_PER_GROUP:
      LF_REQUIRE(value == 0 || (value >= 8 && value <= (1 << 20)), "slots per group %d out of range", value);
      g_slots_per_group = value;
      return LF_OK;
    case LF_OPT_SPMM_CACHE_POLICY:
      LF_REQUIRE(value >= 0 && value <= 1, "cache policy %d out of range", value);
      g_cache_policy = value;
      return LF_OK;
    case LF_OPT_SPMM_MIN_BLOCKS:
      LF_REQUIRE(value >= 2 && value <= 4, "min blocks %d out of range", value);
      g_min_blocks = value;
      return LF_OK;
    case LF_OPT_SPMM_GATHER_RING:
      LF_REQUIRE(value == 0 || value == 16, "gather ring depth %d is not 0 or 16", value);
      g_gather_ring = value;
      return LF_OK;
    case LF_OPT_SPMM_RING_MIN_SLOTS:
      LF_REQUIRE(value >= 0, "slot threshold %d out of range", value);
      g_ring_rows_min_slots = value;
      return LF_OK;
    case LF_OPT_SPMM_TILE_SEGMENTS:
      LF_REQUIRE(value >= 0 && value <= 4096, "segment count %d out of range", value);
      g_tile_segments = value;
      return LF_OK;
    case LF_OPT_BSR_COPY_ENGINE:
      LF_REQUIRE(value >= 0 && value <= 5, "copy engine %d out of range", value);
      g_bsr_copy_engine = value;
      return LF_OK;
    case LF_OPT_BSR_BLOCK_WARPS:
      LF_REQUIRE(value == 0 || (value >= 1 && value <= 8), "warps per thread block %d out of range", value);
      g_bsr_block_warps = value;
      return LF_OK;
    case LF_OPT_BSR_PIPE_SHAPE:
      LF_REQUIRE(value >= 0 && value <= 99, "pipeline shape %d out of range", value);
      g_bsr_pipe_shape = value;
      return LF_OK;
    case LF_OPT_BSR_UMMA_PRODUCER:
      LF_REQUIRE(value == 0 || value == 2 || value == 4, "producer %d is not one of 0, 2, 4", value);
      g_bsr_umma_producer = value;
      return LF_OK;
    case LF_OPT_BSR_PIPE_3D:
      LF_REQUIRE(value == 0 || value == 1, "pipeline copy form %d out of range", value);
      g_bsr_pipe_3d = value;
      return LF_OK;
    case LF_OPT_BSR_TILE_ORDER:
      LF_REQUIRE(value >= 0 && value <= 2, "tile order %d out of range", value);
      g_bsr_tile_order = value;
      return LF_OK;
    default:
      return fail(LF_ERR_INVALID_ARGUMENT, "unknown option %d", option);
  }
}

static int spmm_hyb_impl(const lf_hyb* A, const void* B, bool b_is_bf16, int64_t ldb, float* C, int64_t ldc,
                         int32_t N, int32_t flags, void* stream, const DestList& dests);

int lf_spmm_hyb_f32(const lf_hyb* A, const float* B, int64_t ldb, float* C, int64_t ldc, int32_t N,
                    int32_t flags, void* stream) {
  DestList none;
  none.n = 0;
  none.pad_ = 0;
  return spmm_hyb_impl(A, B, false, ldb, C, ldc, N, flags, stream, none);
}

const char* lf_spmm_hyb_f32_kernel_name(const lf_hyb* A, const float* B, int64_t ldb, const float* C, int64_t ldc,
                                        int32_t N) {
  if (!A || N < 1) return "";
  const FeatCfg cfg = pick_cfg(B, ldb, C, ldc, N);
  if (gather_ring() > 0 && cfg.VEC == 4 && cfg.G < 32 && ldb < (1ll << 30) && cache_policy() == 1 &&
      A->slot_off && A->slot_off[A->num_buckets] >= g_ring_rows_min_slots)
    return "spmm_hyb_ring_rows_kernel";   // buckets narrower than 32 / lanes-per-row slots: spmm_hyb_kernel
  return gather_ring() > 0 && ring_applies(cfg, ldb) ? "spmm_hyb_ring_kernel" : "spmm_hyb_kernel";
}

int lf_spmm_hyb_bf16(const lf_hyb* A, const uint16_t* B, int64_t ldb, float* C, int64_t ldc, int32_t N,
                     int32_t flags, void* stream) {
  DestList none;
  none.n = 0;
  none.pad_ = 0;
  if (N % 8 != 0 || ldb % 8 != 0 || ldc % 4 != 0 || (uintptr_t)B % 16 != 0 || (uintptr_t)C % 16 != 0)
    return fail(LF_ERR_UNSUPPORTED, "the bf16 SpMM needs N and ldb multiples of 8, ldc a multiple of 4 and 16-byte aligned B and C");
  return spmm_hyb_impl(A, B, true, ldb, C, ldc, N, flags, stream, none);
}

int lf_spmm_hyb_f32_bcast(const lf_hyb* A, const float* B, int64_t ldb, float* const* C_full, int32_t num_dests,
                          int64_t ldc, int32_t N, void* stream) {
  LF_REQUIRE(C_full && num_dests >= 1 && num_dests <= LF_MAX_DESTS, "1..%d destinations are supported", LF_MAX_DESTS);
  DestList d;
  d.n = num_dests;
  d.pad_ = 0;
  for (int k = 0; k < LF_MAX_DESTS; ++k) d.p[k] = k < num_dests ? C_full[k] : nullptr;
  for (int k = 0; k < num_dests; ++k)
    LF_REQUIRE(d.p[k] && (uintptr_t)d.p[k] % 16 == 0, "destination %d is null or not 16-byte aligned", k);
  LF_REQUIRE(N % 4 == 0 && ldc % 4 == 0 && ldb % 4 == 0 && (uintptr_t)B % 16 == 0,
             "the broadcasting SpMM needs N, ldb, ldc multiples of 4 and 16-byte aligned operands");
  return spmm_hyb_impl(A, B, false, ldb, d.p[0], ldc, N, LF_SPMM_OVERWRITE, stream, d);
}

static int spmm_hyb_impl(const lf_hyb* A, const void* B, bool b_is_bf16, int64_t ldb, float* C, int64_t ldc,
                         int32_t N, int32_t flags, void* stream, const DestList& dests) {
  if (int s = check_hyb(A)) return s;
  LF_REQUIRE(N >= 1, "N must be >= 1");
  LF_REQUIRE(ldb >= N && ldc >= N && ldb < (1ll << 31), "bad leading dimensions");
  if (A->row_end == A->row_begin) return LF_OK;   // empty shard: nothing to write, C may be NULL
  LF_REQUIRE(B && C, "bad dense operands");
  LF_REQUIRE(flags == LF_SPMM_OVERWRITE || flags == LF_SPMM_ACCUMULATE, "unknown flags %d", flags);
  const int64_t total_rows = A->row_off[A->num_buckets];
  LF_REQUIRE(total_rows == 0 || (A->rows && A->cols && A->vals), "format device arrays missing");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t shard_rows = A->row_end - A->row_begin;
  if (shard_rows == 0) return LF_OK;
  const FeatCfg cfg = b_is_bf16 ? pick_cfg_bf16(N) : pick_cfg(B, ldb, C, ldc, N);
  const bool accumulate = flags == LF_SPMM_ACCUMULATE;
  const bool all_atomic = accumulate || A->num_parts > 1;
  bool cleared_by_kernel = false;   // a row-clearing launch precedes: the product depends on it programmatically

  if (dests.n > 0) {
    if (A->num_parts > 1) {
      for (int k = 0; k < dests.n; ++k)
        LF_CUDA_CHECK(cudaMemset2DAsync(dests.p[k] + A->row_begin * ldc, sizeof(float) * ldc, 0, sizeof(float) * N,
                                        shard_rows, st));
    } else if (A->num_zero_rows > 0) {
      LF_REQUIRE(A->zero_rows, "zero_rows missing");
      const int64_t want = ceil_div64(A->num_zero_rows, kThreads / 32);
      const int grid = (int)(want > 148 * 16 ? 148 * 16 : want);
      zero_rows_multi_kernel<<<grid, kThreads, 0, st>>>(A->zero_rows, A->num_zero_rows, dests, ldc, N);
      LF_CUDA_CHECK(cudaGetLastError());
      cleared_by_kernel = true;
    }
  } else if (!accumulate) {
    if (A->num_parts > 1) {
      LF_CUDA_CHECK(cudaMemset2DAsync(C, sizeof(float) * ldc, 0, sizeof(float) * N, shard_rows, st));
    } else if (A->num_zero_rows > 0) {
      LF_REQUIRE(A->zero_rows, "zero_rows missing");
      const int64_t want = ceil_div64(A->num_zero_rows, kThreads / 32);
      const int grid = (int)(want > 148 * 16 ? 148 * 16 : want);
      if (cfg.VEC != 1)
        zero_rows_kernel<4><<<grid, kThreads, 0, st>>>(A->zero_rows, A->num_zero_rows, C, ldc, N, A->row_begin);
      else
        zero_rows_kernel<1><<<grid, kThreads, 0, st>>>(A->zero_rows, A->num_zero_rows, C, ldc, N, A->row_begin);
      LF_CUDA_CHECK(cudaGetLastError());
      cleared_by_kernel = true;
    }
  }

  // Rows of B narrower than a warp (8 or 16 lanes): buckets at least as wide as the slots of a step
  // go to the ring kernel that takes several slots per step, the narrower ones to the register
  // kernel in a launch of their own.
  // Small products stay with the one launch of the register kernel (a 16384-row matrix: 0.013 ms
  // against 0.023 ms for the two launches).
  const int rows_per_step = 32 / cfg.G;
  const bool split = gather_ring() > 0 && cfg.VEC != 1 && rows_per_step > 1 && dests.n == 0 && ldb < (1ll << 30) &&
                     cache_policy() == 1 && A->slot_off[A->num_buckets] >= g_ring_rows_min_slots;
  const int segs = tile_segments();
  for (int pass = 0; pass < (split ? 2 : 1); ++pass) {
    const bool ring_rows = split && pass == 0;
    // one launch per LF_MAX_BUCKETS_PER_LAUNCH non-empty buckets (one launch in every practical case)
    const int gpc = ring_rows ? kThreads / 32 : kThreads / cfg.G;
    auto in_pass = [&](int k) {
      if (A->ell_rows[k] == 0) return false;
      if (!split) return true;
      return (A->widths[k] >= rows_per_step) == ring_rows;
    };
    int spg = slots_per_group();
    if (!spg) {
      const int64_t want_tiles = (int64_t)sm_count() * min_blocks() * 8;
      for (spg = 256; spg > 32; spg >>= 1) {
        int64_t t = 0;
        for (int k = 0; k < A->num_buckets; ++k) {
          if (!in_pass(k)) continue;
          const int w = A->widths[k];
          const int rpg = spg / w > 0 ? spg / w : 1;
          t += ceil_div64(A->ell_rows[k], (int64_t)rpg * gpc);
        }
        if (t >= want_tiles) break;
      }
    }
    int i = 0;
    while (i < A->num_buckets) {
      static thread_local SpmmTable<LF_MAX_BUCKETS_PER_LAUNCH> big;
      int n = 0;
      int64_t tiles = 0, seg_tiles = 0;
      for (; i < A->num_buckets && n < LF_MAX_BUCKETS_PER_LAUNCH; ++i) {
        if (!in_pass(i)) continue;
        BucketDesc d;
        int wlog = 0;
        while ((1 << wlog) < A->widths[i]) ++wlog;
        d.row_off = A->row_off[i];
        d.slot_off = A->slot_off[i];
        d.ell_rows = A->ell_rows[i];
        d.wlog = wlog;
        d.rows_per_group = (spg >> wlog) > 0 ? (spg >> wlog) : 1;
        d.force_atomic = all_atomic ? 1 : 0;
        const int64_t my_tiles = ceil_div64(d.ell_rows, (int64_t)d.rows_per_group * gpc);
        const int64_t per_seg = segs > 0 ? ceil_div64(my_tiles, segs) : 0;
        d.tile_begin = segs > 0 ? seg_tiles : tiles;
        d.tiles_per_seg = (int32_t)per_seg;
        tiles += my_tiles;
        seg_tiles += per_seg;
        big.b[n] = d;
        ++n;
      }
      if (n == 0) break;
      const int64_t grid_tiles = segs > 0 ? seg_tiles * segs : tiles;   // interleaved: a few idle thread blocks at bucket ends
      LF_REQUIRE(grid_tiles < (1ll << 31) && seg_tiles < (1ll << 31), "too many thread blocks for one launch");
      int s;
      if (n <= 16) {
        SpmmTable<16> small;
        small.n = n;
        small.seg_tiles = (int32_t)(segs > 0 ? seg_tiles : 0);
        for (int k = 0; k < n; ++k) small.b[k] = big.b[k];
        s = ring_rows ? launch_hyb_ring_rows<16>(small, grid_tiles, A, B, b_is_bf16, ldb, C, ldc, N, cfg.G, st, cleared_by_kernel)
                      : launch_hyb<16>(small, grid_tiles, A, B, ldb, C, ldc, N, cfg, st, dests, cleared_by_kernel);
      } else {
        big.n = n;
        big.seg_tiles = (int32_t)(segs > 0 ? seg_tiles : 0);
        s = ring_rows ? launch_hyb_ring_rows<LF_MAX_BUCKETS_PER_LAUNCH>(big, grid_tiles, A, B, b_is_bf16, ldb, C, ldc, N, cfg.G, st, cleared_by_kernel)
                      : launch_hyb<LF_MAX_BUCKETS_PER_LAUNCH>(big, grid_tiles, A, B, ldb, C, ldc, N, cfg, st, dests, cleared_by_kernel);
      }
      if (s) return s;
      cleared_by_kernel = false;   // a further launch follows a product kernel, not the clearing one
    }
  }
  return LF_OK;
}

int lf_allgather_rows(const float* C_rows, int64_t ld_rows, int64_t row_begin, int64_t rows, int32_t N,
                      float* const* C_full, int32_t num_dests, int64_t ldc, void* stream) {
  LF_REQUIRE(C_full && num_dests >= 1 && num_dests <= LF_MAX_DESTS, "1..%d destinations are supported", LF_MAX_DESTS);
  LF_REQUIRE(rows >= 0 && row_begin >= 0 && N >= 1 && ld_rows >= N && ldc >= N, "bad shape");
  if (rows == 0) return LF_OK;
  LF_REQUIRE(C_rows, "source rows missing");
  DestList d;
  d.n = num_dests;
  d.pad_ = 0;
  bool vec = N % 4 == 0 && ld_rows % 4 == 0 && ldc % 4 == 0 && (uintptr_t)C_rows % 16 == 0;
  for (int k = 0; k < LF_MAX_DESTS; ++k) d.p[k] = k < num_dests ? C_full[k] : nullptr;
  for (int k = 0; k < num_dests; ++k) {
    LF_REQUIRE(d.p[k], "destination %d is null", k);
    vec = vec && (uintptr_t)d.p[k] % 16 == 0;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t items = rows * (vec ? N / 4 : N);
  const int64_t want = ceil_div64(items, 256 * 4);
  const unsigned grid = (unsigned)(want < 1 ? 1 : (want > (int64_t)sm_count() * 16 ? (int64_t)sm_count() * 16 : want));
  if (vec) allgather_rows_kernel<4><<<grid, 256, 0, st>>>(C_rows, ld_rows, rows, N, row_begin, d, ldc);
  else allgather_rows_kernel<1><<<grid, 256, 0, st>>>(C_rows, ld_rows, rows, N, row_begin, d, ldc);
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

static size_t host_ws_layout(const lf_hyb* A, int32_t N, size_t off[7]) {
  const int nb = A->num_buckets;
  const size_t n_rows = (size_t)A->row_off[nb], n_slots = (size_t)A->slot_off[nb];
  size_t o = 0;
  auto take = [&](size_t bytes) { size_t r = o; o = align_up(o + (bytes ? bytes : 1), 256); return r; };
  off[0] = take(n_rows * 4);                                      // rows
  off[1] = take(n_slots * 4);                                     // cols
  off[2] = take(n_slots * 4);                                     // vals
  off[3] = take((size_t)A->num_zero_rows * 4);                    // zero_rows
  off[4] = take((size_t)A->num_cols * N * 4);                     // B
  off[5] = take((size_t)(A->row_end - A->row_begin) * N * 4);     // C
  off[6] = o;
  return o;
}

size_t lf_spmm_hyb_f32_host_workspace_bytes(const lf_hyb* A_host, int32_t N) {
  if (!A_host || !A_host->row_off || !A_host->slot_off || N < 1) return 0;
  size_t off[7];
  return host_ws_layout(A_host, N, off);
}

int lf_spmm_hyb_f32_host(const lf_hyb* A, const float* B, float* C, int32_t N, int32_t flags,
                         void* device_workspace, size_t workspace_bytes, void* stream) {
  if (int s = check_hyb(A)) return s;
  LF_REQUIRE(B && C && N >= 1 && device_workspace, "bad arguments");
  LF_REQUIRE((flags & ~(LF_SPMM_ACCUMULATE | LF_SPMM_NO_SYNC | LF_SPMM_FORMAT_RESIDENT)) == 0, "unknown flags %d", flags);
  const bool accumulate = (flags & LF_SPMM_ACCUMULATE) != 0;
  const bool upload_format = (flags & LF_SPMM_FORMAT_RESIDENT) == 0;
  size_t off[7];
  if (workspace_bytes < host_ws_layout(A, N, off)) return fail(LF_ERR_WORKSPACE_TOO_SMALL, "host-call workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)device_workspace;
  const int nb = A->num_buckets;
  const size_t n_rows = (size_t)A->row_off[nb], n_slots = (size_t)A->slot_off[nb];
  const size_t c_bytes = (size_t)(A->row_end - A->row_begin) * N * 4;
  if (upload_format) {   // otherwise the workspace still holds this format from an earlier call
    if (n_rows) LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[0], A->rows, n_rows * 4, cudaMemcpyHostToDevice, st));
    if (n_slots) {
      LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[1], A->cols, n_slots * 4, cudaMemcpyHostToDevice, st));
      LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[2], A->vals, n_slots * 4, cudaMemcpyHostToDevice, st));
    }
    if (A->num_zero_rows) LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[3], A->zero_rows, (size_t)A->num_zero_rows * 4, cudaMemcpyHostToDevice, st));
  }
  LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[4], B, (size_t)A->num_cols * N * 4, cudaMemcpyHostToDevice, st));
  if (accumulate && c_bytes) LF_CUDA_CHECK(cudaMemcpyAsync(ws + off[5], C, c_bytes, cudaMemcpyHostToDevice, st));
  lf_hyb dev = *A;
  dev.rows = (const int32_t*)(ws + off[0]);
  dev.cols = (const int32_t*)(ws + off[1]);
  dev.vals = (const float*)(ws + off[2]);
  dev.mask = nullptr;
  dev.zero_rows = (const int32_t*)(ws + off[3]);
  if (int s = lf_spmm_hyb_f32(&dev, (const float*)(ws + off[4]), N, (float*)(ws + off[5]), N, N,
                              accumulate ? LF_SPMM_ACCUMULATE : LF_SPMM_OVERWRITE, st))
    return s;
  if (c_bytes) LF_CUDA_CHECK(cudaMemcpyAsync(C, ws + off[5], c_bytes, cudaMemcpyDeviceToHost, st));
  if (!(flags & LF_SPMM_NO_SYNC)) LF_CUDA_CHECK(cudaStreamSynchronize(st));
  return LF_OK;
}

int lf_spmm_csr_f32(const int64_t* indptr, const int32_t* indices, const float* data, int64_t row_begin,
                    int64_t row_end, int64_t nnz, const float* B, int64_t ldb, float* C, int64_t ldc, int32_t N,
                    void* stream) {
  LF_REQUIRE(N >= 1 && ldb >= N && ldc >= N && ldb < (1ll << 31), "bad arguments");
  LF_REQUIRE(0 <= row_begin && row_begin <= row_end, "bad row range");
  if (row_begin == row_end) return LF_OK;
  LF_REQUIRE(indptr && B && C, "null pointer argument");
  cudaStream_t st = (cudaStream_t)stream;
  if (nnz < 0) {   // the launch shape depends on the number of entries: read it back
    int64_t ends[2] = {0, 0};
    LF_CUDA_CHECK(cudaMemcpyAsync(&ends[0], indptr + row_begin, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    LF_CUDA_CHECK(cudaMemcpyAsync(&ends[1], indptr + row_end, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    LF_CUDA_CHECK(cudaStreamSynchronize(st));
    nnz = ends[1] - ends[0];
  }
  LF_REQUIRE(nnz == 0 || indices, "indices missing");
  const FeatCfg cfg = pick_cfg(B, ldb, C, ldc, N);
  const int gpc = kThreads / cfg.G;
  int spg = 256;   // entries per group; smaller for small matrices so that the grid has several waves
  while (spg > 32 && ceil_div64(nnz, (int64_t)spg * gpc) < (int64_t)sm_count() * 3 * 8) spg >>= 1;
  {
    const int64_t rows = row_end - row_begin, groups = ceil_div64(nnz, spg);
    const int64_t n = rows > groups ? rows : groups;
    const int64_t want = ceil_div64(n, 256 / 32);
    const unsigned pgrid = (unsigned)(want > 148 * 32 ? 148 * 32 : want);
    if (cfg.VEC == 4) csr_prepare_kernel<4><<<pgrid, 256, 0, st>>>(indptr, row_begin, row_end, spg, C, ldc, N);
    else csr_prepare_kernel<1><<<pgrid, 256, 0, st>>>(indptr, row_begin, row_end, spg, C, ldc, N);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  if (nnz == 0) return LF_OK;
  const int64_t blocks = ceil_div64(nnz, (int64_t)spg * gpc);
  LF_REQUIRE(blocks < (1ll << 31), "too many thread blocks");
  if (gather_ring() > 0 && ring_applies(cfg, ldb)) {
    dim3 rgrid((unsigned)blocks, (unsigned)((N + kRingFeatures - 1) / kRingFeatures));
    const size_t smem = (size_t)(kThreads / 32) * 16 * 32 * sizeof(float4);
    auto kern = spmm_csr_ring_kernel<16>;
    LF_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LF_CUDA_CHECK(launch_dep_smem(kern, rgrid, kThreads, smem, st, true, indptr, indices, data, row_begin, row_end, B,
                                  (int)ldb, C, ldc, N, spg));
    return LF_OK;
  }
  dim3 grid((unsigned)blocks, (unsigned)((N + cfg.pass - 1) / cfg.pass));
#define LF_LAUNCH(G_, V_, VEC_)                                                                              \
  LF_CUDA_CHECK(launch_dep(spmm_csr_kernel<G_, V_, VEC_>, grid, kThreads, st, true, indptr, indices, data, row_begin, \
                           row_end, B, (int)ldb, C, ldc, N, spg))
  if (cfg.VEC == 4) {
    if (cfg.G == 8) LF_LAUNCH(8, 1, 4);
    else if (cfg.G == 16) LF_LAUNCH(16, 1, 4);
    else if (cfg.V == 1) LF_LAUNCH(32, 1, 4);
    else if (cfg.V == 2) LF_LAUNCH(32, 2, 4);
    else LF_LAUNCH(32, 4, 4);
  } else {
    if (cfg.V == 1) LF_LAUNCH(32, 1, 1);
    else if (cfg.V == 2) LF_LAUNCH(32, 2, 1);
    else LF_LAUNCH(32, 4, 1);
  }
#undef LF_LAUNCH
  return LF_OK;
}

}  // extern "C"
