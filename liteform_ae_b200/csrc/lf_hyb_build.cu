// Device-side construction of LiteForm's composed format (column partitions x power-of-two ELL
// buckets) from CSR: statistics for the width search, then count -> scan -> scatter.
//
// What the reference does on the host, one Python iteration per nonzero:
//   get_init_buckets   playground_pipline/format_algos.py:819-900   -> lf_hyb_stats
//   build_hyb_format   playground_pipline/format_algos.py:226-385   -> lf_hyb_plan + lf_hyb_fill
//
// None of the kernels below waits on another thread block: offsets across blocks come from a
// separate scan launch, never from a look-back spin.
#include <mutex>

#include "lf_common.cuh"

namespace lf {

static thread_local char g_err[512] = "";
char* error_buffer() { return g_err; }
int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

namespace {

constexpr int kRowsPerBlock = 256;   // one thread per matrix row in the count / fill kernels
constexpr int kClasses = LF_NUM_WIDTH_CLASSES;
constexpr int kLongRowChunks = 32;   // rows with more ELL rows than this are written by the whole block

// First position in [pos, end) whose column is >= bound (columns ascend inside a row).
__device__ __forceinline__ int64_t segment_end(const int32_t* __restrict__ indices, int64_t pos,
                                               int64_t end, int64_t bound) {
  if (pos >= end || indices[pos] >= bound) return pos;
  int64_t lo = pos + 1, hi = end;  // indices[lo-1] < bound
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if (indices[mid] < bound) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// ------------------------------------------------------------------------------------------
// statistics
// ------------------------------------------------------------------------------------------
// A (row, partition) segment of at least kLongSegMin entries is not marked by the warp that
// found it (a 100 000-entry row would keep one warp busy for thousands of iterations while the
// rest of the grid has long finished; even 8 000 entries are 250 dependent steps, as long as the
// whole rest of the pass on a million-row graph): the warp appends it to a list, and stats_long_kernel
// spreads the listed segments over the whole grid in chunks.  Such a segment is always in the
// widest class.  A full list is not an error: further segments are marked in place.
struct LongSeg {
  long long pos, end;
};
constexpr int kLongSegMin = 2048;
constexpr int kLongSegCap = 8192;
constexpr int kLongChunk = 2048;
constexpr size_t kLongListBytes = 256 + sizeof(LongSeg) * kLongSegCap;   // counter slot + list
static_assert(kLongSegMin > (1 << (kClasses - 1)), "a deferred segment must belong to the widest class");

// A warp marks the columns of entries [lo, hi) with `bit`: four strided entries per lane and
// step, their columns and masks loaded before the first atomic, so that the loads overlap.
// Columns outside [0, num_cols) are skipped everywhere below (never used as an index): a
// malformed matrix gives wrong statistics, not a stray access; lf_csr_validate reports it.
__device__ __forceinline__ void warp_mark(const int32_t* __restrict__ indices, uint32_t* __restrict__ colmask,
                                          int64_t lo, int64_t hi, int lane, uint32_t bit, uint32_t num_cols) {
  for (int64_t i = lo + lane; i < hi; i += 128) {
    int32_t c[4];
    uint32_t m[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      c[u] = i + 32 * u < hi ? indices[i + 32 * u] : -1;
      if ((uint32_t)c[u] >= num_cols) c[u] = -1;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) m[u] = c[u] >= 0 ? colmask[c[u]] : bit;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (!(m[u] & bit)) atomicOr(colmask + c[u], bit);
  }
}

// Several partitions: one warp per matrix row.  For each column partition the row touches:
// degree -> width class, three counters per (partition, class), and the class bit OR-ed into
// every touched column.
__global__ void __launch_bounds__(256)
stats_rows_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                  int64_t num_rows, uint32_t num_cols, int64_t psz, int num_parts,
                  unsigned long long* __restrict__ class_stats, uint32_t* __restrict__ colmask,
                  int use_smem, unsigned int* __restrict__ long_count, LongSeg* __restrict__ long_list) {
  extern __shared__ unsigned long long s_stats[];
  const int n_stat = num_parts * kClasses * 3;
  if (use_smem) {
    for (int i = threadIdx.x; i < n_stat; i += blockDim.x) s_stats[i] = 0ull;
    __syncthreads();
  }
  unsigned long long* acc = use_smem ? s_stats : class_stats;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  // The chain row pointer -> column -> class mask of the column is three dependent loads; the
  // row pointer and the first 32 columns of the warp's NEXT row are fetched before the current
  // row is worked on, so that two chains are in flight per warp.
  int64_t r = warp, s = 0, e = 0;
  int32_t c_first = 0;
  if (r < num_rows) {
    s = indptr[r];
    e = indptr[r + 1];
    c_first = s + lane < e ? indices[s + lane] : 0;
  }
  while (r < num_rows) {
    const int64_t r_next = r + n_warps;
    int64_t s_next = 0, e_next = 0;
    int32_t c_next = 0;
    if (r_next < num_rows) {
      s_next = indptr[r_next];
      e_next = indptr[r_next + 1];
      c_next = s_next + lane < e_next ? indices[s_next + lane] : 0;
    }
    int64_t pos = s;
    if (num_parts > 1 && e - s <= 32) {
      // short row, several partitions: one entry per lane.  A lane whose partition differs from
      // its left neighbour's heads a segment; segment lengths come from the ballot of heads, so
      // all segments of the row are counted and marked at once instead of one after the other.
      const int n = (int)(e - s);
      const bool on = lane < n && (uint32_t)c_first < num_cols;
      const int32_t c = on ? c_first : 0;
      const int p = on ? (int)((uint32_t)c / (uint32_t)psz) : -1;
      const int left = __shfl_up_sync(0xffffffffu, p, 1);
      const bool head = on && (lane == 0 || p != left);
      const unsigned heads = __ballot_sync(0xffffffffu, head);
      int kc = 0;
      if (head) {
        const unsigned later = lane == 31 ? 0u : heads >> (lane + 1);
        const uint32_t deg = later ? (uint32_t)__ffs(later) : (uint32_t)min(n - lane, 32);
        kc = ceil_log2_u32(deg);   // deg <= 32: never beyond the widest class
        unsigned long long* a = acc + (p * kClasses + kc) * 3;
        atomicAdd(a + 0, 1ull);
        atomicAdd(a + 1, (unsigned long long)deg);
        atomicAdd(a + 2, 1ull);
      }
      const unsigned upto = heads & (0xffffffffu >> (31 - lane));   // heads at or before this lane
      const int my_head = on ? 31 - __clz(upto) : 0;
      const uint32_t bit = 1u << __shfl_sync(0xffffffffu, kc, my_head);
      if (on && !(colmask[c] & bit)) atomicOr(colmask + c, bit);
      pos = e;
    }
    while (pos < e) {
      int64_t nxt;
      int p;
      if (num_parts == 1) {
        p = 0;
        nxt = e;
      } else {
        const int32_t c0 = indices[pos];
        if ((uint32_t)c0 >= num_cols) { ++pos; continue; }   // malformed entry: skipped
        p = (int)(c0 / psz);
        nxt = segment_end(indices, pos, e, (int64_t)(p + 1) * psz);
      }
      const uint32_t deg = (uint32_t)(nxt - pos);
      const int k = ceil_log2_u32(deg);
      const int kc = k > kClasses - 1 ? kClasses - 1 : k;
      if (lane == 0) {
        const unsigned long long reps = k > kClasses - 1 ? (1ull << (k - (kClasses - 1))) : 1ull;
        unsigned long long* a = acc + (p * kClasses + kc) * 3;
        atomicAdd(a + 0, reps);
        atomicAdd(a + 1, (unsigned long long)deg);
        atomicAdd(a + 2, 1ull);
      }
      const uint32_t bit = 1u << kc;
      bool deferred = false;
      if (deg >= (uint32_t)kLongSegMin) {
        unsigned int slot = 0;
        if (lane == 0) slot = atomicAdd(long_count, 1u);
        slot = __shfl_sync(0xffffffffu, slot, 0);
        if (slot < (unsigned int)kLongSegCap) {
          if (lane == 0) long_list[slot] = LongSeg{(long long)pos, (long long)nxt};
          deferred = true;
        }
      }
      if (!deferred) warp_mark(indices, colmask, pos, nxt, lane, bit, num_cols);
      pos = nxt;
    }
    r = r_next;
    s = s_next;
    e = e_next;
    c_first = c_next;
  }
  if (use_smem) {
    __syncthreads();
    for (int i = threadIdx.x; i < n_stat; i += blockDim.x)
      if (s_stats[i]) atomicAdd(class_stats + i, s_stats[i]);
  }
}

// One partition: a warp takes 32 consecutive rows, one row pointer per lane.  Counters are added
// by the lane that holds the row.  The entries of the 32 rows are one contiguous range of the
// CSR arrays: the warp walks it with coalesced loads, 128 entries per step, and every entry finds
// its row (hence its class bit) by a five-step bisection over the row ends held in the lanes'
// registers.  Short and medium rows cost the same per entry and there is no per-row chain of
// dependent loads; a warp per row spent its time waiting on exactly that chain.  Rows of
// kLongSegMin entries or more go to the list; a batch that holds one (rare) marks its other rows
// one after the other instead, so that the walk does not have to step over the long row.
// Measured against a warp per row (with the next row prefetched): 0.55 against 0.62 ms on 134 M
// entries at 32 per row, 0.12 against 0.15 ms on a power-law graph of 14 entries per row.
__global__ void __launch_bounds__(256)
stats_rows_p1_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices, int64_t num_rows,
                     uint32_t num_cols, unsigned long long* __restrict__ class_stats, uint32_t* __restrict__ colmask,
                     unsigned int* __restrict__ long_count, LongSeg* __restrict__ long_list) {
  __shared__ unsigned long long s_stats[kClasses * 3];
  for (int i = threadIdx.x; i < kClasses * 3; i += blockDim.x) s_stats[i] = 0ull;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t base = warp * 32; base < num_rows; base += n_warps * 32) {
    const int64_t r = base + lane;
    // lanes past the last row hold an empty row at the end of the arrays: row ends stay monotone
    const int64_t s = indptr[r < num_rows ? r : num_rows];
    const int64_t e = indptr[r + 1 < num_rows ? r + 1 : num_rows];
    const int64_t len = e - s;
    const int k = len > 0 ? ceil_log2_u32((uint32_t)len) : 0;
    const int kc = k > kClasses - 1 ? kClasses - 1 : k;
    // counters: the rows of a batch mostly share a few classes, and 32 lanes adding to the same
    // shared-memory words one after the other cost more than the marking; one lane per class
    // present adds the batch's totals instead
    for (unsigned pending = __ballot_sync(0xffffffffu, len > 0); pending;) {
      const int leader = __ffs(pending) - 1;
      const int k_lead = __shfl_sync(0xffffffffu, kc, leader);
      const bool mine = len > 0 && kc == k_lead;
      const unsigned group = __ballot_sync(0xffffffffu, mine);
      unsigned long long sum_len = mine ? (unsigned long long)len : 0ull;
      unsigned long long sum_rows = mine ? (k > kClasses - 1 ? (1ull << (k - (kClasses - 1))) : 1ull) : 0ull;
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        sum_len += __shfl_xor_sync(0xffffffffu, sum_len, o);
        sum_rows += __shfl_xor_sync(0xffffffffu, sum_rows, o);
      }
      if (lane == leader) {
        unsigned long long* a = s_stats + k_lead * 3;
        atomicAdd(a + 0, sum_rows);
        atomicAdd(a + 1, sum_len);
        atomicAdd(a + 2, (unsigned long long)__popc(group));
      }
      pending &= ~group;
    }
    bool deferred = false;
    if (len >= kLongSegMin) {
      const unsigned int slot = atomicAdd(long_count, 1u);
      if (slot < (unsigned int)kLongSegCap) {
        long_list[slot] = LongSeg{(long long)s, (long long)e};
        deferred = true;
      }
    }
    const bool has_long = __any_sync(0xffffffffu, len >= kLongSegMin);
    const int64_t first = __shfl_sync(0xffffffffu, s, 0);
    const int64_t batch_entries = __shfl_sync(0xffffffffu, e, 31) - first;
    if (!has_long) {   // fewer than 32 * kLongSegMin entries
      const uint32_t total = (uint32_t)batch_entries;
      const uint32_t my_end = (uint32_t)(e - first);
      for (uint32_t step = 0; step < total; step += 128) {
        int32_t c[4];
        uint32_t bit[4], m[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t i = step + 32 * u + lane;
          int lo = 0, hi = 31;   // smallest lane whose row ends after entry i
#pragma unroll
          for (int it = 0; it < 5; ++it) {
            const int mid = (lo + hi) >> 1;
            const uint32_t end_mid = __shfl_sync(0xffffffffu, my_end, mid);
            if (end_mid > i) hi = mid; else lo = mid + 1;
          }
          bit[u] = 1u << __shfl_sync(0xffffffffu, kc, lo);
          c[u] = i < total ? indices[first + i] : -1;
          if ((uint32_t)c[u] >= num_cols) c[u] = -1;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) m[u] = c[u] >= 0 ? colmask[c[u]] : 0xffffffffu;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (!(m[u] & bit[u])) atomicOr(colmask + c[u], bit[u]);
      }
    } else {
      // a batch around a listed row: one row after the other, the next row's first 32 columns
      // requested before the current row is marked
      unsigned todo = __ballot_sync(0xffffffffu, len > 0 && !deferred);
      int src = 0;
      int64_t s_cur = 0, e_cur = 0;
      int32_t c_cur = 0;
      if (todo) {
        src = __ffs(todo) - 1;
        s_cur = __shfl_sync(0xffffffffu, s, src);
        e_cur = __shfl_sync(0xffffffffu, e, src);
        c_cur = s_cur + lane < e_cur ? indices[s_cur + lane] : -1;
      }
      while (todo) {
        todo &= todo - 1;
        int src_nxt = 0;
        int64_t s_nxt = 0, e_nxt = 0;
        int32_t c_nxt = 0;
        if (todo) {
          src_nxt = __ffs(todo) - 1;
          s_nxt = __shfl_sync(0xffffffffu, s, src_nxt);
          e_nxt = __shfl_sync(0xffffffffu, e, src_nxt);
          c_nxt = s_nxt + lane < e_nxt ? indices[s_nxt + lane] : -1;
        }
        const uint32_t bit = 1u << __shfl_sync(0xffffffffu, kc, src);
        if (e_cur - s_cur <= 32) {
          if ((uint32_t)c_cur < num_cols && !(colmask[c_cur] & bit)) atomicOr(colmask + c_cur, bit);
        } else {
          warp_mark(indices, colmask, s_cur, e_cur, lane, bit, num_cols);
        }
        src = src_nxt;
        s_cur = s_nxt;
        e_cur = e_nxt;
        c_cur = c_nxt;
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kClasses * 3; i += blockDim.x)
    if (s_stats[i]) atomicAdd(class_stats + i, s_stats[i]);
}

// Marks the columns of the listed long segments.  The list is taken in tiles of 256 segments: the
// block scans their chunk counts in shared memory, and chunk number c of the running count goes
// to thread block c mod gridDim.x, which finds its segment by bisection -- a handful of very long
// rows occupies the whole grid, and thousands of listed segments cost no serial walk.
__global__ void __launch_bounds__(256)
stats_long_kernel(const int32_t* __restrict__ indices, const unsigned int* __restrict__ long_count,
                  const LongSeg* __restrict__ long_list, uint32_t* __restrict__ colmask, uint32_t num_cols) {
  __shared__ long long s_pos[256], s_end[256];
  __shared__ int s_pre[257];
  __shared__ int s_scan[256 / 32 + 1];
  const unsigned int listed = *long_count;
  const int n = (int)(listed < (unsigned int)kLongSegCap ? listed : (unsigned int)kLongSegCap);
  const uint32_t bit = 1u << (kClasses - 1);
  long long dealt = 0;   // chunks of the tiles before this one
  for (int t0 = 0; t0 < n; t0 += 256) {
    const int i = t0 + threadIdx.x;
    LongSeg seg = {0, 0};
    if (i < n) seg = long_list[i];
    const int chunks = (int)((seg.end - seg.pos + kLongChunk - 1) / kLongChunk);
    int total;
    const int before = block_exclusive_scan<256>(chunks, s_scan, &total);
    s_pos[threadIdx.x] = seg.pos;
    s_end[threadIdx.x] = seg.end;
    s_pre[threadIdx.x] = before;
    if (threadIdx.x == 0) s_pre[256] = total;
    __syncthreads();
    long long first = ((long long)blockIdx.x - dealt) % (long long)gridDim.x;
    if (first < 0) first += gridDim.x;
    for (long long c = first; c < total; c += gridDim.x) {
      int lo = 0, hi = 256;   // last segment of the tile whose first chunk is <= c
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_pre[mid] <= c) lo = mid; else hi = mid;
      }
      const long long from = s_pos[lo] + (c - s_pre[lo]) * kLongChunk;
      const long long to = from + kLongChunk < s_end[lo] ? from + kLongChunk : s_end[lo];
      constexpr int kPer = kLongChunk / 256;
      int32_t col[kPer];
      uint32_t m[kPer];
#pragma unroll
      for (int u = 0; u < kPer; ++u) {
        const long long e = from + threadIdx.x + 256 * u;
        col[u] = e < to ? indices[e] : -1;
        if ((uint32_t)col[u] >= num_cols) col[u] = -1;
      }
#pragma unroll
      for (int u = 0; u < kPer; ++u) m[u] = col[u] >= 0 ? colmask[col[u]] : bit;
#pragma unroll
      for (int u = 0; u < kPer; ++u)
        if (!(m[u] & bit)) atomicOr(colmask + col[u], bit);
    }
    dealt += total;
    __syncthreads();
  }
}

// blockIdx.y = partition; histogram of the 11-bit class masks of that partition's columns.
__global__ void __launch_bounds__(256)
colmask_hist_kernel(const uint32_t* __restrict__ colmask, int64_t num_cols, int64_t psz,
                    unsigned long long* __restrict__ hist) {
  __shared__ uint32_t s_hist[LF_COLMASK_BINS];
  for (int i = threadIdx.x; i < LF_COLMASK_BINS; i += blockDim.x) s_hist[i] = 0u;
  __syncthreads();
  const int p = blockIdx.y;
  const int64_t lo = (int64_t)p * psz;
  int64_t hi = lo + psz;
  if (hi > num_cols) hi = num_cols;
  for (int64_t c = lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < hi;
       c += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t m = colmask[c];
    if (m) atomicAdd(&s_hist[m & (LF_COLMASK_BINS - 1)], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < LF_COLMASK_BINS; i += blockDim.x)
    if (s_hist[i]) atomicAdd(hist + (size_t)p * LF_COLMASK_BINS + i, (unsigned long long)s_hist[i]);
}

// ------------------------------------------------------------------------------------------
// plan / fill
// ------------------------------------------------------------------------------------------
struct BuildMeta {            // device copy of the per-call tables, at the head of the workspace
  const int32_t* pbo;         // [P+1]
  const int32_t* widths;      // [nb]
  const int64_t* row_off;     // [nb+1]   (valid after lf_hyb_fill uploaded them)
  const int64_t* slot_off;    // [nb+1]
  const int64_t* ell_rows;    // [nb]
};

// bucket of a row of `deg` entries inside partition with widths w[0..n): bisect_left clamped.
__device__ __forceinline__ int pick_bucket(const int32_t* __restrict__ w, int n, int deg) {
  int b = 0;
  while (b < n - 1 && w[b] < deg) ++b;
  return b;
}

// One thread per matrix row: ELL rows it contributes to every (partition, bucket).
__global__ void __launch_bounds__(kRowsPerBlock)
hyb_count_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                 int64_t row_begin, int64_t row_end, uint32_t num_cols, int64_t psz, int num_parts,
                 const int32_t* __restrict__ pbo, const int32_t* __restrict__ widths, int ncat,
                 int32_t* __restrict__ block_counts, int32_t* __restrict__ err) {
  extern __shared__ int32_t s_cnt[];
  for (int i = threadIdx.x; i < ncat; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  const int64_t r = row_begin + (int64_t)blockIdx.x * kRowsPerBlock + threadIdx.x;
  if (r < row_end) {
    const int64_t s = indptr[r], e = indptr[r + 1];
    int64_t pos = s;
    int64_t total = 0;
    while (pos < e) {
      int p = 0;
      int64_t nxt = e;
      if (num_parts > 1) {
        const int32_t c0 = indices[pos];
        if ((uint32_t)c0 >= num_cols) {   // malformed matrix: report, touch nothing
          atomicExch(err, -1);
          break;
        }
        p = (int)(c0 / psz);
        nxt = segment_end(indices, pos, e, (int64_t)(p + 1) * psz);
      }
      const int deg = (int)(nxt - pos);
      const int nb = pbo[p + 1] - pbo[p];
      if (nb == 0) {
        atomicExch(err, p + 1);  // entries in a partition that was given no bucket width
      } else {
        const int b = pick_bucket(widths + pbo[p], nb, deg);
        const int w = widths[pbo[p] + b];
        const int n = (deg + w - 1) / w;
        atomicAdd(&s_cnt[pbo[p] + b], n);
        total += n;
      }
      pos = nxt;
    }
    if (total != 1) atomicAdd(&s_cnt[ncat - 1], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ncat; i += blockDim.x)
    block_counts[(size_t)blockIdx.x * ncat + i] = s_cnt[i];
}

// blockIdx.x = category; exclusive scan of that category's per-block counts over all blocks.
__global__ void __launch_bounds__(256)
scan_blocks_kernel(const int32_t* __restrict__ block_counts, int64_t num_blocks, int ncat,
                   int64_t* __restrict__ block_offsets, int64_t* __restrict__ totals) {
  __shared__ int s_scan[256 / 32 + 1];
  const int cat = blockIdx.x;
  int64_t running = 0;
  for (int64_t base = 0; base < num_blocks; base += 256) {
    const int64_t i = base + threadIdx.x;
    const int v = i < num_blocks ? block_counts[(size_t)i * ncat + cat] : 0;
    int tot;
    const int ex = block_exclusive_scan<256>(v, s_scan, &tot);
    if (i < num_blocks) block_offsets[(size_t)i * ncat + cat] = running + ex;
    running += tot;
  }
  if (threadIdx.x == 0) totals[cat] = running;
}

// One thread per matrix row.  Writes, for every ELL row the matrix row produces: the row id, and
// in scratch where its entries start in the CSR arrays and how many it holds.
__global__ void __launch_bounds__(kRowsPerBlock)
hyb_fill_rows_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices,
                     int64_t row_begin, int64_t row_end, int64_t psz, int num_parts,
                     BuildMeta meta, int ncat, const int32_t* __restrict__ block_counts,
                     const int64_t* __restrict__ block_offsets, int32_t* __restrict__ ell_rows,
                     int32_t* __restrict__ src_start, int32_t* __restrict__ src_len,
                     int32_t* __restrict__ zero_rows) {
  __shared__ int s_scan[kRowsPerBlock / 32 + 1];
  __shared__ int s_nlong;
  __shared__ int64_t s_long_dst[kRowsPerBlock];
  __shared__ int64_t s_long_src[kRowsPerBlock];
  __shared__ int32_t s_long_deg[kRowsPerBlock];
  __shared__ int32_t s_long_row[kRowsPerBlock];

  const int64_t r = row_begin + (int64_t)blockIdx.x * kRowsPerBlock + threadIdx.x;
  const bool live = r < row_end;
  const int64_t e = live ? indptr[r + 1] : 0;
  int64_t pos = live ? indptr[r] : 0;
  int64_t total = 0;
  const int32_t* bc = block_counts + (size_t)blockIdx.x * ncat;
  const int64_t* bo = block_offsets + (size_t)blockIdx.x * ncat;

  for (int p = 0; p < num_parts; ++p) {
    const int64_t seg = pos;
    const int64_t nxt = num_parts == 1 ? e : segment_end(indices, pos, e, (int64_t)(p + 1) * psz);
    pos = nxt;
    const int deg = (int)(nxt - seg);
    const int cat0 = meta.pbo[p];
    const int nb = meta.pbo[p + 1] - cat0;
    int my_b = -1, my_w = 1, my_n = 0;
    if (deg > 0 && nb > 0) {
      my_b = pick_bucket(meta.widths + cat0, nb, deg);
      my_w = meta.widths[cat0 + my_b];
      my_n = (deg + my_w - 1) / my_w;
      total += my_n;
    }
    for (int b = 0; b < nb; ++b) {
      if (bc[cat0 + b] == 0) continue;  // uniform: nobody in this block lands in the bucket
      if (threadIdx.x == 0) s_nlong = 0;
      int tot;
      const int x = (my_b == b) ? my_n : 0;
      const int ex = block_exclusive_scan<kRowsPerBlock>(x, s_scan, &tot);
      if (x > 0) {
        const int64_t dst = meta.row_off[cat0 + b] + bo[cat0 + b] + ex;
        if (x <= kLongRowChunks) {
          for (int c = 0; c < x; ++c) {
            ell_rows[dst + c] = (int32_t)r;
            src_start[dst + c] = (int32_t)(seg + (int64_t)c * my_w);
            const int left = deg - c * my_w;
            src_len[dst + c] = left < my_w ? left : my_w;
          }
        } else {
          const int q = atomicAdd(&s_nlong, 1);
          s_long_dst[q] = dst;
          s_long_src[q] = seg;
          s_long_deg[q] = deg;
          s_long_row[q] = (int32_t)r;
        }
      }
      __syncthreads();
      const int nlong = s_nlong;
      const int w = meta.widths[cat0 + b];
      for (int q = 0; q < nlong; ++q) {
        const int64_t dst = s_long_dst[q];
        const int64_t src = s_long_src[q];
        const int d = s_long_deg[q];
        const int n = (d + w - 1) / w;
        for (int c = threadIdx.x; c < n; c += kRowsPerBlock) {
          ell_rows[dst + c] = s_long_row[q];
          src_start[dst + c] = (int32_t)(src + (int64_t)c * w);
          const int left = d - c * w;
          src_len[dst + c] = left < w ? left : w;
        }
      }
      __syncthreads();
    }
  }
  if (bc[ncat - 1] != 0) {
    int tot;
    const int flag = (live && total != 1) ? 1 : 0;
    const int ex = block_exclusive_scan<kRowsPerBlock>(flag, s_scan, &tot);
    if (flag) zero_rows[bo[ncat - 1] + ex] = (int32_t)r;
  }
}

// One thread per group of four consecutive slots of the cols/vals/mask arenas (alignment gaps
// included, they get zeros; bucket starts are multiples of 64 slots, so a group never straddles
// two buckets).  A slot costs three dependent rounds of loads (bucket tables, the ELL row's
// source range, the entry itself); the four slots of a group go through the rounds together and
// leave as one 128-bit store per array (32 bits for the mask).
__global__ void __launch_bounds__(256)
hyb_fill_slots_kernel(const int32_t* __restrict__ indices, const float* __restrict__ data,
                      BuildMeta meta, int nb, const int32_t* __restrict__ src_start,
                      const int32_t* __restrict__ src_len, int32_t* __restrict__ cols,
                      float* __restrict__ vals, uint8_t* __restrict__ mask, int64_t total_slots) {
  const int64_t groups = total_slots >> 2;   // total_slots is a multiple of 64
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < groups; q += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = q << 2;
    int lo = 0, hi = nb;  // last bucket i with slot_off[i] <= t
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (meta.slot_off[mid] <= t) lo = mid; else hi = mid;
    }
    const int w = meta.widths[lo];
    const int shift = 31 - __clz(w);   // widths are powers of two
    const int64_t local = t - meta.slot_off[lo];
    const int64_t live = meta.ell_rows[lo] << shift;
    const int64_t row0 = meta.row_off[lo];
    int64_t src[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      src[u] = -1;
      if (local + u < live) {
        const int64_t er = row0 + ((local + u) >> shift);
        const int j = (int)((local + u) & (w - 1));
        if (j < src_len[er]) src[u] = (int64_t)src_start[er] + j;
      }
    }
    int32_t c[4];
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      c[u] = src[u] >= 0 ? indices[src[u]] : 0;
      v[u] = src[u] >= 0 ? (data ? data[src[u]] : 1.f) : 0.f;
    }
    *reinterpret_cast<int4*>(cols + t) = make_int4(c[0], c[1], c[2], c[3]);
    *reinterpret_cast<float4*>(vals + t) = make_float4(v[0], v[1], v[2], v[3]);
    if (mask)
      *reinterpret_cast<uint32_t*>(mask + t) = (src[0] >= 0 ? 1u : 0u) | (src[1] >= 0 ? 0x100u : 0u) |
                                               (src[2] >= 0 ? 0x10000u : 0u) | (src[3] >= 0 ? 0x1000000u : 0u);
  }
}

__global__ void shard_rows_kernel(const int64_t* __restrict__ indptr, int64_t num_rows, int shards,
                                  int64_t* __restrict__ splits) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g > shards) return;
  if (g == shards) { splits[g] = num_rows; return; }
  const int64_t nnz = indptr[num_rows] - indptr[0];
  const int64_t target = indptr[0] + (int64_t)(((__int128)nnz * g) / shards);
  int64_t lo = 0, hi = num_rows;  // first r with indptr[r] >= target
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (indptr[mid] < target) lo = mid + 1; else hi = mid;
  }
  splits[g] = lo;
}

// Row-length statistics for MTX.matrix_features (format_matrix_market.py:153-202): per block of
// 256 rows the sum, the sum of squares, the minimum and the maximum of the row lengths.  The
// partials stay exact integers; the caller folds them (in arbitrary precision) into mean / std.
__global__ void __launch_bounds__(kRowsPerBlock)
row_stats_kernel(const int64_t* __restrict__ indptr, int64_t row_begin, int64_t row_end,
                 unsigned long long* __restrict__ partials) {
  __shared__ unsigned long long s_sum[kRowsPerBlock / 32], s_sq[kRowsPerBlock / 32];
  __shared__ unsigned long long s_min[kRowsPerBlock / 32], s_max[kRowsPerBlock / 32];
  const int64_t r = row_begin + (int64_t)blockIdx.x * kRowsPerBlock + threadIdx.x;
  const bool live = r < row_end;
  const unsigned long long len = live ? (unsigned long long)(indptr[r + 1] - indptr[r]) : 0ull;
  unsigned long long sum = len, sq = len * len, mn = live ? len : ~0ull, mx = len;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const unsigned long long a = __shfl_xor_sync(0xffffffffu, mn, o), b = __shfl_xor_sync(0xffffffffu, mx, o);
    mn = a < mn ? a : mn;
    mx = b > mx ? b : mx;
  }
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { s_sum[warp] = sum; s_sq[warp] = sq; s_min[warp] = mn; s_max[warp] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kRowsPerBlock / 32; ++w) {
      sum += s_sum[w]; sq += s_sq[w];
      mn = s_min[w] < mn ? s_min[w] : mn;
      mx = s_max[w] > mx ? s_max[w] : mx;
    }
    unsigned long long* out = partials + (size_t)blockIdx.x * 4;
    out[0] = sum; out[1] = sq; out[2] = mn; out[3] = mx;
  }
}

// Structural check of a CSR matrix: row pointers non-decreasing from indptr[0] >= 0, every column in
// [0, num_cols), columns strictly ascending inside a row.  A warp takes 32 rows; rows of up to 32
// entries are checked by one lane each, longer rows by the whole warp.  Bit 0 of *flag: bad row
// pointer, bit 1: column out of range, bit 2: columns not strictly ascending.
__device__ int g_csr_flag;

__global__ void __launch_bounds__(256)
csr_validate_kernel(const int64_t* __restrict__ indptr, const int32_t* __restrict__ indices, int64_t num_rows,
                    uint32_t num_cols, int64_t nnz_bound) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  int bad = 0;
  for (int64_t base = warp * 32; base < num_rows; base += n_warps * 32) {
    const int64_t r = base + lane;
    int64_t s = 0, e = 0;
    if (r < num_rows) {
      s = indptr[r];
      e = indptr[r + 1];
      if (s < 0 || e < s || e > nnz_bound) { bad |= 1; e = s; }   // a broken row is not walked
    }
    if (e - s <= 32) {
      int32_t prev = -1;
      for (int64_t i = s; i < e; ++i) {
        const int32_t c = indices[i];
        if ((uint32_t)c >= num_cols) bad |= 2;
        else if (c <= prev) bad |= 4;
        prev = c;
      }
    }
    for (unsigned todo = __ballot_sync(0xffffffffu, e - s > 32); todo; todo &= todo - 1) {
      const int src = __ffs(todo) - 1;
      const int64_t ls = __shfl_sync(0xffffffffu, s, src), le = __shfl_sync(0xffffffffu, e, src);
      for (int64_t i = ls + lane; i < le; i += 32) {
        const int32_t c = indices[i];
        if ((uint32_t)c >= num_cols) bad |= 2;
        else if (i > ls && c <= indices[i - 1]) bad |= 4;
      }
    }
  }
  if (bad) atomicOr(&g_csr_flag, bad);
}

// ---- workspace carving ---------------------------------------------------------------------
struct BuildWs {
  int32_t* pbo; int32_t* widths; int64_t* row_off; int64_t* slot_off; int64_t* ell_rows;
  int64_t* totals; int32_t* err; int32_t* block_counts; int64_t* block_offsets;
  size_t bytes;
};

BuildWs carve_build(void* base, int64_t rows, int num_parts, int nb) {
  const int ncat = nb + 1;
  const int64_t blocks = ceil_div64(rows > 0 ? rows : 1, kRowsPerBlock);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return (char*)base + o; };
  BuildWs w;
  w.pbo = (int32_t*)take(sizeof(int32_t) * (num_parts + 1));
  w.widths = (int32_t*)take(sizeof(int32_t) * (nb > 0 ? nb : 1));
  w.row_off = (int64_t*)take(sizeof(int64_t) * (nb + 1));
  w.slot_off = (int64_t*)take(sizeof(int64_t) * (nb + 1));
  w.ell_rows = (int64_t*)take(sizeof(int64_t) * (nb > 0 ? nb : 1));
  w.totals = (int64_t*)take(sizeof(int64_t) * (ncat + 2));
  w.err = (int32_t*)take(sizeof(int32_t) * 4);
  w.block_counts = (int32_t*)take(sizeof(int32_t) * blocks * ncat);
  w.block_offsets = (int64_t*)take(sizeof(int64_t) * blocks * ncat);
  w.bytes = off;
  return w;
}

int check_widths(int32_t num_parts, const int32_t* pbo, const int32_t* widths) {
  LF_REQUIRE(num_parts >= 1, "num_parts must be >= 1 (got %d)", num_parts);
  LF_REQUIRE(pbo && pbo[0] == 0, "part_bucket_off[0] must be 0");
  for (int p = 0; p < num_parts; ++p) {
    LF_REQUIRE(pbo[p + 1] >= pbo[p], "part_bucket_off must be non-decreasing");
    for (int i = pbo[p]; i < pbo[p + 1]; ++i) {
      const int w = widths[i];
      LF_REQUIRE(w >= 1 && (w & (w - 1)) == 0, "bucket width %d (partition %d) is not a power of two", w, p);
      LF_REQUIRE(i == pbo[p] || widths[i - 1] < w, "bucket widths of partition %d are not ascending", p);
    }
  }
  return LF_OK;
}

}  // namespace
}  // namespace lf

using namespace lf;

extern "C" {

int lf_version(void) { return 100; }
const char* lf_last_error(void) { return lf::error_buffer(); }

size_t lf_hyb_stats_workspace_bytes(int64_t /*num_rows*/, int64_t num_cols, int32_t /*num_parts*/) {
  return align_up(sizeof(uint32_t) * (size_t)(num_cols > 0 ? num_cols : 1), 256) + kLongListBytes;
}

int lf_hyb_stats(const int64_t* indptr, const int32_t* indices, int64_t num_rows, int64_t num_cols,
                 int32_t num_parts, int64_t* class_stats, int64_t* colmask_hist, void* workspace,
                 size_t workspace_bytes, void* stream) {
  LF_REQUIRE(indptr && class_stats && colmask_hist && workspace, "null pointer argument");
  LF_REQUIRE(num_rows >= 0 && num_cols >= 1, "bad shape %lld x %lld", (long long)num_rows, (long long)num_cols);
  LF_REQUIRE(num_parts >= 1 && num_parts <= num_cols, "num_parts %d out of range", num_parts);
  LF_REQUIRE(num_parts <= 65535, "num_parts %d exceeds the grid limit", num_parts);
  LF_REQUIRE(num_cols < (1ll << 31), "column indices are 32-bit: %lld columns are not supported", (long long)num_cols);
  if (workspace_bytes < lf_hyb_stats_workspace_bytes(num_rows, num_cols, num_parts))
    return fail(LF_ERR_WORKSPACE_TOO_SMALL, "stats workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t psz = ceil_div64(num_cols, num_parts);
  uint32_t* colmask = (uint32_t*)workspace;
  char* long_base = (char*)workspace + align_up(sizeof(uint32_t) * (size_t)num_cols, 256);
  unsigned int* long_count = (unsigned int*)long_base;
  LongSeg* long_list = (LongSeg*)(long_base + 256);
  const size_t n_stat = (size_t)num_parts * kClasses * 3;
  LF_CUDA_CHECK(cudaMemsetAsync(colmask, 0, sizeof(uint32_t) * num_cols, st));
  LF_CUDA_CHECK(cudaMemsetAsync(long_count, 0, sizeof(unsigned int), st));
  LF_CUDA_CHECK(cudaMemsetAsync(class_stats, 0, sizeof(int64_t) * n_stat, st));
  LF_CUDA_CHECK(cudaMemsetAsync(colmask_hist, 0, sizeof(int64_t) * (size_t)num_parts * LF_COLMASK_BINS, st));
  if (num_rows > 0) {
    if (num_parts == 1) {
      const int64_t want = ceil_div64(num_rows, 8 * 32);  // 8 warps per block, 32 rows per warp and step
      const int grid = (int)(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
      stats_rows_p1_kernel<<<grid, 256, 0, st>>>(indptr, indices, num_rows, (uint32_t)num_cols,
                                                 (unsigned long long*)class_stats, colmask, long_count, long_list);
    } else {
      const size_t smem = n_stat * sizeof(unsigned long long);
      const int use_smem = smem <= 40 * 1024;
      const int64_t want = ceil_div64(num_rows, 8 * 4);  // 8 warps per block, ~4 rows per warp
      const int grid = (int)(want < 1 ? 1 : (want > 148 * 64 ? 148 * 64 : want));
      stats_rows_kernel<<<grid, 256, use_smem ? smem : 0, st>>>(
          indptr, indices, num_rows, (uint32_t)num_cols, psz, num_parts, (unsigned long long*)class_stats, colmask,
          use_smem, long_count, long_list);
    }
    LF_CUDA_CHECK(cudaGetLastError());
    stats_long_kernel<<<148 * 4, 256, 0, st>>>(indices, long_count, long_list, colmask, (uint32_t)num_cols);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  {
    const int64_t want = ceil_div64(psz, 256 * 8);
    dim3 grid((unsigned)(want < 1 ? 1 : (want > 1024 ? 1024 : want)), (unsigned)num_parts);
    colmask_hist_kernel<<<grid, 256, 0, st>>>(colmask, num_cols, psz, (unsigned long long*)colmask_hist);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  return LF_OK;
}

// ---- allocation-free statistics -------------------------------------------------------------
// Scratch of lf_hyb_stats_static: the per-column class-mask array, resident in every device
// that loads this library until the process exits.
#define LF_STATIC_STATS_MAX_COLS_IMPL (1 << 20)
constexpr size_t kStaticScratchBytes = sizeof(uint32_t) * LF_STATIC_STATS_MAX_COLS_IMPL + kLongListBytes;
static __device__ __align__(256) uint32_t g_static_colmask[kStaticScratchBytes / sizeof(uint32_t)];
static_assert(LF_STATIC_STATS_MAX_COLS_IMPL == LF_STATIC_STATS_MAX_COLS, "header and implementation disagree");

// In host code `g_static_colmask` is only a handle of the symbol, not an address a kernel can
// use; the device address is looked up once per device (with that device current) and kept.
static uint32_t* static_colmask_address(int* status) {
  constexpr int kMaxDevices = 64;
  static uint32_t* addr[kMaxDevices] = {nullptr};
  static std::mutex lock;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status = fail(LF_ERR_CUDA, "cudaGetDevice failed or device ordinal %d unsupported: %s", dev, cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(lock);
  if (!addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_colmask);
    if (e != cudaSuccess || !p) {
      *status = fail(LF_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    addr[dev] = (uint32_t*)p;
  }
  *status = LF_OK;
  return addr[dev];
}

int lf_hyb_stats_static(const int64_t* indptr, const int32_t* indices, int64_t num_rows, int64_t num_cols,
                        int32_t num_parts, int64_t* class_stats, int64_t* colmask_hist, void* stream) {
  if (num_cols > LF_STATIC_STATS_MAX_COLS)
    return fail(LF_ERR_UNSUPPORTED,
                "lf_hyb_stats_static handles at most %d columns (got %lld); use lf_hyb_stats with a caller-owned workspace",
                LF_STATIC_STATS_MAX_COLS, (long long)num_cols);
  int status = LF_OK;
  uint32_t* scratch = static_colmask_address(&status);
  if (!scratch) return status;
  // same launches as lf_hyb_stats, which clears the part of the scratch it is about to use
  return lf_hyb_stats(indptr, indices, num_rows, num_cols, num_parts, class_stats, colmask_hist, scratch,
                      kStaticScratchBytes, stream);
}

int lf_csr_validate(const int64_t* indptr, const int32_t* indices, int64_t num_rows, int64_t num_cols, int64_t nnz,
                    void* stream) {
  LF_REQUIRE(indptr && num_rows >= 0 && num_cols >= 1 && nnz >= 0, "bad arguments");
  LF_REQUIRE(num_cols < (1ll << 31) && nnz < (1ll << 31), "more than 2^31-1 columns or stored entries are not supported");
  LF_REQUIRE(nnz == 0 || indices, "indices missing");
  cudaStream_t st = (cudaStream_t)stream;
  const int zero = 0;
  LF_CUDA_CHECK(cudaMemcpyToSymbolAsync(g_csr_flag, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
  if (num_rows > 0) {
    const int64_t want = ceil_div64(num_rows, 8 * 32);
    csr_validate_kernel<<<(unsigned)(want > 148 * 16 ? 148 * 16 : want), 256, 0, st>>>(indptr, indices, num_rows,
                                                                                        (uint32_t)num_cols, nnz);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  int flag = 0;
  int64_t ends[2] = {0, 0};
  LF_CUDA_CHECK(cudaMemcpyFromSymbolAsync(&flag, g_csr_flag, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
  LF_CUDA_CHECK(cudaMemcpyAsync(&ends[0], indptr, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  LF_CUDA_CHECK(cudaMemcpyAsync(&ends[1], indptr + num_rows, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  LF_CUDA_CHECK(cudaStreamSynchronize(st));
  if (flag & 1) return fail(LF_ERR_INVALID_ARGUMENT, "row pointers are negative, decreasing or beyond the number of stored entries");
  if (ends[0] != 0 || ends[1] != nnz)
    return fail(LF_ERR_INVALID_ARGUMENT, "row pointers run from %lld to %lld, expected 0 to %lld", (long long)ends[0],
                (long long)ends[1], (long long)nnz);
  if (flag & 2) return fail(LF_ERR_INVALID_ARGUMENT, "a column index lies outside [0, %lld)", (long long)num_cols);
  if (flag & 4) return fail(LF_ERR_INVALID_ARGUMENT, "column indices are not strictly ascending inside a row (sort and merge duplicates first)");
  return LF_OK;
}

int64_t lf_row_stats_blocks(int64_t row_begin, int64_t row_end) {
  return row_end > row_begin ? ceil_div64(row_end - row_begin, kRowsPerBlock) : 0;
}

int lf_row_stats(const int64_t* indptr, int64_t row_begin, int64_t row_end, uint64_t* partials, void* stream) {
  LF_REQUIRE(indptr && partials && 0 <= row_begin && row_begin <= row_end, "bad arguments");
  const int64_t blocks = lf_row_stats_blocks(row_begin, row_end);
  if (blocks == 0) return LF_OK;
  LF_REQUIRE(blocks < (1ll << 31), "row range too large");
  row_stats_kernel<<<(unsigned)blocks, kRowsPerBlock, 0, (cudaStream_t)stream>>>(
      indptr, row_begin, row_end, (unsigned long long*)partials);
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

size_t lf_hyb_build_workspace_bytes(int64_t row_begin, int64_t row_end, int32_t num_parts,
                                    int32_t num_buckets) {
  return carve_build(nullptr, row_end - row_begin, num_parts, num_buckets).bytes;
}

size_t lf_hyb_fill_scratch_bytes(int64_t total_ell_rows) {
  return 2 * align_up(sizeof(int32_t) * (size_t)(total_ell_rows > 0 ? total_ell_rows : 1), 256);
}

int lf_hyb_plan(const int64_t* indptr, const int32_t* indices, int64_t num_rows, int64_t num_cols,
                int64_t row_begin, int64_t row_end, int32_t num_parts,
                const int32_t* part_bucket_off, const int32_t* widths, int64_t* ell_rows,
                int64_t* row_off, int64_t* slot_off, int64_t* num_zero_rows, void* workspace,
                size_t workspace_bytes, void* stream) {
  LF_REQUIRE(indptr && part_bucket_off && ell_rows && row_off && slot_off && num_zero_rows && workspace,
             "null pointer argument");
  LF_REQUIRE(num_cols >= 1 && num_cols < (1ll << 31) && 0 <= row_begin && row_begin <= row_end && row_end <= num_rows,
             "bad shape or row range");
  if (int s = check_widths(num_parts, part_bucket_off, widths)) return s;
  LF_REQUIRE(num_parts <= num_cols, "num_parts %d exceeds the number of columns", num_parts);
  const int nb = part_bucket_off[num_parts];
  const int ncat = nb + 1;
  LF_REQUIRE((size_t)ncat * sizeof(int32_t) <= 40 * 1024, "too many buckets (%d)", nb);
  const int64_t rows = row_end - row_begin;
  BuildWs ws = carve_build(workspace, rows, num_parts, nb);
  if (workspace_bytes < ws.bytes) return fail(LF_ERR_WORKSPACE_TOO_SMALL, "build workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t psz = ceil_div64(num_cols, num_parts);
  const int64_t blocks = ceil_div64(rows > 0 ? rows : 1, kRowsPerBlock);
  LF_REQUIRE(blocks < (1ll << 31), "row range too large");

  LF_CUDA_CHECK(cudaMemcpyAsync(ws.pbo, part_bucket_off, sizeof(int32_t) * (num_parts + 1), cudaMemcpyHostToDevice, st));
  if (nb) LF_CUDA_CHECK(cudaMemcpyAsync(ws.widths, widths, sizeof(int32_t) * nb, cudaMemcpyHostToDevice, st));
  LF_CUDA_CHECK(cudaMemsetAsync(ws.err, 0, sizeof(int32_t) * 4, st));
  hyb_count_kernel<<<(unsigned)blocks, kRowsPerBlock, sizeof(int32_t) * ncat, st>>>(
      indptr, indices, row_begin, row_end, (uint32_t)num_cols, psz, num_parts, ws.pbo, ws.widths, ncat,
      ws.block_counts, ws.err);
  LF_CUDA_CHECK(cudaGetLastError());
  scan_blocks_kernel<<<ncat, 256, 0, st>>>(ws.block_counts, blocks, ncat, ws.block_offsets, ws.totals);
  LF_CUDA_CHECK(cudaGetLastError());

  // host results: totals per category, the error flag and the entry range (for the int32 guard)
  int64_t h_tot_small[64];
  int64_t* h_tot = ncat <= 64 ? h_tot_small : (int64_t*)malloc(sizeof(int64_t) * ncat);
  int32_t h_err = 0;
  int64_t h_ptr[2] = {0, 0};
  cudaError_t ce = cudaMemcpyAsync(h_tot, ws.totals, sizeof(int64_t) * ncat, cudaMemcpyDeviceToHost, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(&h_err, ws.err, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(&h_ptr[0], indptr + row_begin, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(&h_ptr[1], indptr + row_end, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
  int status = LF_OK;
  if (ce != cudaSuccess) {
    status = fail(LF_ERR_CUDA, "lf_hyb_plan: %s", cudaGetErrorString(ce));
  } else if (h_err < 0) {
    status = fail(LF_ERR_INVALID_ARGUMENT, "the matrix holds a column index outside [0, %lld)", (long long)num_cols);
  } else if (h_err) {
    status = fail(LF_ERR_INVALID_ARGUMENT, "partition %d holds entries but was given no bucket width", h_err - 1);
  } else if (h_ptr[1] > 0x7fffffffll) {
    status = fail(LF_ERR_UNSUPPORTED, "more than 2^31-1 stored entries are not supported");
  } else {
    row_off[0] = slot_off[0] = 0;
    for (int i = 0; i < nb; ++i) {
      ell_rows[i] = h_tot[i];
      row_off[i + 1] = row_off[i] + (int64_t)align_up((size_t)h_tot[i], kBucketAlign);
      slot_off[i + 1] = slot_off[i] + (int64_t)align_up((size_t)h_tot[i] * widths[i], kBucketAlign);
    }
    *num_zero_rows = h_tot[nb];
  }
  if (h_tot != h_tot_small) free(h_tot);
  return status;
}

int lf_hyb_fill(const int64_t* indptr, const int32_t* indices, const float* data,
                const lf_hyb* L, void* workspace, size_t workspace_bytes, void* scratch,
                size_t scratch_bytes, void* stream) {
  LF_REQUIRE(indptr && L && workspace && scratch, "null pointer argument");
  LF_REQUIRE(L->part_bucket_off && L->ell_rows && L->row_off && L->slot_off, "layout host arrays missing");
  if (int s = check_widths(L->num_parts, L->part_bucket_off, L->widths)) return s;
  const int nb = L->num_buckets;
  LF_REQUIRE(nb == L->part_bucket_off[L->num_parts], "num_buckets does not match part_bucket_off");
  const int ncat = nb + 1;
  const int64_t rows = L->row_end - L->row_begin;
  LF_REQUIRE(rows >= 0 && L->row_end <= L->num_rows && L->num_cols >= 1, "bad row range");
  const int64_t total_rows = L->row_off[nb], total_slots = L->slot_off[nb];
  LF_REQUIRE((total_rows == 0 || L->rows) && (total_slots == 0 || (L->cols && L->vals)), "output arrays missing");
  LF_REQUIRE(L->num_zero_rows == 0 || L->zero_rows, "zero_rows array missing");
  BuildWs ws = carve_build(workspace, rows, L->num_parts, nb);
  if (workspace_bytes < ws.bytes) return fail(LF_ERR_WORKSPACE_TOO_SMALL, "build workspace too small");
  if (scratch_bytes < lf_hyb_fill_scratch_bytes(total_rows)) return fail(LF_ERR_WORKSPACE_TOO_SMALL, "fill scratch too small");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t psz = ceil_div64(L->num_cols, L->num_parts);
  const int64_t blocks = ceil_div64(rows > 0 ? rows : 1, kRowsPerBlock);
  int32_t* src_start = (int32_t*)scratch;
  int32_t* src_len = (int32_t*)((char*)scratch + lf_hyb_fill_scratch_bytes(total_rows) / 2);

  LF_CUDA_CHECK(cudaMemcpyAsync(ws.row_off, L->row_off, sizeof(int64_t) * (nb + 1), cudaMemcpyHostToDevice, st));
  LF_CUDA_CHECK(cudaMemcpyAsync(ws.slot_off, L->slot_off, sizeof(int64_t) * (nb + 1), cudaMemcpyHostToDevice, st));
  if (nb) LF_CUDA_CHECK(cudaMemcpyAsync(ws.ell_rows, L->ell_rows, sizeof(int64_t) * nb, cudaMemcpyHostToDevice, st));
  if (total_rows) LF_CUDA_CHECK(cudaMemsetAsync((void*)L->rows, 0, sizeof(int32_t) * total_rows, st));
  BuildMeta meta{ws.pbo, ws.widths, ws.row_off, ws.slot_off, ws.ell_rows};
  if (rows > 0) {
    hyb_fill_rows_kernel<<<(unsigned)blocks, kRowsPerBlock, 0, st>>>(
        indptr, indices, L->row_begin, L->row_end, psz, L->num_parts, meta, ncat, ws.block_counts,
        ws.block_offsets, (int32_t*)L->rows, src_start, src_len, (int32_t*)L->zero_rows);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  if (total_slots > 0) {
    LF_REQUIRE(total_slots % 4 == 0 && (uintptr_t)L->cols % 16 == 0 && (uintptr_t)L->vals % 16 == 0 &&
                   (uintptr_t)L->mask % 4 == 0, "cols / vals must be 16-byte aligned, mask 4-byte aligned");
    const int64_t want = ceil_div64(total_slots, 256 * 4 * 4);
    const int grid = (int)(want > 148 * 32 ? 148 * 32 : want);
    hyb_fill_slots_kernel<<<grid, 256, 0, st>>>(indices, data, meta, nb, src_start, src_len,
                                                (int32_t*)L->cols, (float*)L->vals, (uint8_t*)L->mask, total_slots);
    LF_CUDA_CHECK(cudaGetLastError());
  }
  return LF_OK;
}

int lf_shard_rows(const int64_t* indptr, int64_t num_rows, int32_t num_shards, int64_t* splits, void* stream) {
  LF_REQUIRE(indptr && splits && num_rows >= 0, "bad arguments");
  LF_REQUIRE(num_shards >= 1 && num_shards <= 1024, "num_shards %d out of range", num_shards);
  shard_rows_kernel<<<(num_shards + 1 + 63) / 64, 64, 0, (cudaStream_t)stream>>>(indptr, num_rows, num_shards, splits);
  LF_CUDA_CHECK(cudaGetLastError());
  return LF_OK;
}

}  // extern "C"
