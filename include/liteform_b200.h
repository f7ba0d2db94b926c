/*
 * liteform_b200 -- C ABI of the B200 (sm_100a) implementation of LiteForm's composed-format SpMM.
 *
 * The reference project (johnpzh/liteform_ae) is pure Python and has no native boundary of its
 * own: its format builder is interpreted Python and its kernels are generated at run time by an
 * external TVM/SparseTIR fork.  Each entry point below therefore cites the Python function (path
 * inside the reference project, file:line) whose work it takes over.  A binding for the
 * reference's pipeline is a handful of ctypes calls.
 *
 * Conventions
 *   - every function returns 0 on success or a negative lf_status; lf_last_error() returns a
 *     thread-local, human-readable message for the last failure on the calling thread;
 *   - nothing throws, nothing allocates device memory: every device buffer, including scratch
 *     ("workspace"), is owned by the caller, who obtains the required size from the matching
 *     *_workspace_bytes() query;
 *   - pointers are marked [dev] (device memory of the current CUDA device) or [host];
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); functions
 *     that return host-side results synchronise that stream before returning, all others only
 *     enqueue work;
 *   - matrices are CSR with int64 row pointers, int32 column indices sorted and distinct inside a
 *     row, float values; dense operands are row-major with an explicit leading dimension.
 */
#ifndef LITEFORM_B200_H_
#define LITEFORM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  LF_OK = 0,
  LF_ERR_INVALID_ARGUMENT = -1,
  LF_ERR_CUDA = -2,
  LF_ERR_WORKSPACE_TOO_SMALL = -3,
  LF_ERR_UNSUPPORTED = -4,
  LF_ERR_KERNEL_TIMEOUT = -5
} lf_status;

#define LF_NUM_WIDTH_CLASSES 11   /* widths 1, 2, 4 ... 1024 (format_algos.py:821) */
#define LF_COLMASK_BINS 2048      /* 2^LF_NUM_WIDTH_CLASSES */
#define LF_MAX_BUCKETS_PER_LAUNCH 256

/* flags for the SpMM entry points */
#define LF_SPMM_OVERWRITE 0       /* C = A * B   (every row of C is written)            */
#define LF_SPMM_ACCUMULATE 1      /* C += A * B  (what the generated reference kernel does,
                                     format_algos.py:508-515, 550, 595)                     */

#define LF_SPMM_FORMAT_RESIDENT 4 /* lf_spmm_hyb_f32_host only, may be OR-ed with the others: the format arrays
                                     are NOT uploaded; the workspace still holds them from an earlier call with
                                     the same A_host and N (the reference uploads them on every call,
                                     format_algos.py:568-578).  B is uploaded and C downloaded as always.   */
#define LF_SPMM_NO_SYNC 2         /* lf_spmm_hyb_f32_host only, may be OR-ed with the above: enqueue the
                                     copies and the product and return; C is valid and the workspace free
                                     again once the stream has been synchronised.  Lets a caller keep two
                                     products in flight on two streams with two workspaces, so that the
                                     copy of one result overlaps the upload of the next operands.        */

int lf_version(void);
const char* lf_last_error(void);

/* Process-wide tuning knobs of the SpMM launch (no counterpart in the reference, whose launch
 * shape is fixed by its code generator, format_algos.py:503-539).  Results do not depend on them. */
#define LF_OPT_SPMM_SLOTS_PER_GROUP 1  /* ELL slots one thread group walks (0 = automatic: 256, less for small launches) */
#define LF_OPT_SPMM_CACHE_POLICY 2     /* 0 plain loads and stores; 1 slots, row ids and C stream through (default) */
#define LF_OPT_SPMM_MIN_BLOCKS 3       /* resident thread blocks per SM the kernel is compiled for: 2..4 (default 3) */
#define LF_OPT_BSR_COPY_ENGINE 4        /* how the 8x8 block kernels fill shared memory: 0 automatic, 1 per-lane
                                          cp.async into warp-private rings, 2 tiled bulk copies through a tensor map
                                          into the same rings, 3 one bulk copy per row of B, 4 thread-block-wide
                                          pipeline: a producer warp issues one tiled bulk copy per block, consumer
                                          warps run the MMAs, 5 (16-bit inputs; float32 runs 4) the same copies feeding
                                          tcgen05.mma with accumulators in tensor memory (2 to 5 complete on mbarriers) */
#define LF_OPT_BSR_TILE_ORDER 5         /* float32 block kernel with several 128-feature tiles: 0 automatic (2 from
                                          four tiles on), 1 the tiles of a block row run together (A read once),
                                          2 one tile after the other over all rows (the B rows of one tile stay
                                          in the L2) */
#define LF_OPT_BSR_PIPE_SHAPE 7         /* copy engine 4: blocks per stage * 10 + stages of the ring (44, 43, 83, 26;
                                          0 = default 44) */
#define LF_OPT_BSR_PIPE_3D 8            /* copy engine 4: 1 (default) one 3-D tiled copy brings all feature slices of
                                          a block, 0 one 2-D tiled copy per 128-byte feature slice */
#define LF_OPT_BSR_UMMA_PRODUCER 9      /* copy engine 5: who fills shared memory: 0 (default) one warp issuing tiled bulk
                                          copies, 2 or 4 = that many warps issuing per-lane cp.async */
#define LF_OPT_BSR_BLOCK_WARPS 11       /* copy engine 1, more than 64 features: warps per thread block, 1..8 (0 = automatic:
                                          4 for 16-bit inputs up to 128 features, else 8) */
#define LF_OPT_SPMM_RING_MIN_SLOTS 12    /* products with up to 64 float32 / 128 bf16 features: stored slots from which the
                                          ring form (two launches) replaces the register kernel (default 2^20) */
#define LF_OPT_SPMM_GATHER_RING 10      /* products with 128-bit gathers: where the gathered rows of B land: 16 (default) a
                                          ring of 16 rows (or steps of 2 / 4 narrow rows) per warp in shared memory,
                                          filled by cp.async; 0 registers (8 rows in flight per warp) */
#define LF_OPT_SPMM_TILE_SEGMENTS 6     /* order of the thread blocks of the composed-format product: 0 bucket after
                                          bucket (default); S > 0: every bucket is cut into S segments of consecutive
                                          rows and the launch runs segment 0 of all buckets, then segment 1, ... */
int lf_set_option(int32_t option, int32_t value);

/* ---------------------------------------------------------------------------------------------
 * Structural check of a CSR matrix in device memory -- what every entry point below assumes and
 * what SciPy guarantees for the reference (coo.tocsr(), format_matrix_market.py:74-76): row
 * pointers run from 0 to nnz without decreasing, column indices lie in [0, num_cols) and ascend
 * strictly inside a row.  Returns LF_ERR_INVALID_ARGUMENT (with a message naming the defect)
 * otherwise.  Synchronises the stream; calls on one device must not overlap (the verdict travels
 * through one device word).  The builder kernels never use an out-of-range column as an index
 * (they skip it, lf_hyb_plan reports it), so a malformed matrix cannot make them touch memory
 * they do not own; unsorted rows give a wrong format without notice -- validate first.
 * ------------------------------------------------------------------------------------------- */
int lf_csr_validate(const int64_t* indptr /*[dev] M+1*/, const int32_t* indices /*[dev] nnz*/,
                    int64_t num_rows, int64_t num_cols, int64_t nnz, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Bucket statistics for the width search.
 * Replaces the per-nonzero Python loops of get_init_buckets (playground_pipline/
 * format_algos.py:819-900).  For every column partition p (partition size ceil(K/P),
 * format_algos.py:836) and width class k (width 2^k = 2^ceil(log2 degree) clipped to 1024,
 * format_algos.py:875-882) it produces what the cost model reads from a Bucket
 * (format_matrix_market.py:12-37):
 *   class_stats[(p*11 + k)*3 + 0] = num_rows  (a clipped row counts 2^ceil(log2 d)/1024 times)
 *   class_stats[(p*11 + k)*3 + 1] = nnz
 *   class_stats[(p*11 + k)*3 + 2] = number of rows in the class  (len(row_indices))
 * and, instead of Python sets of column ids, a histogram over per-column class bitmasks:
 *   colmask_hist[p*2048 + m] = number of columns of partition p whose set of touching classes is m
 * so that len(col_indices) of any merged bucket is a sum over the bins that intersect its classes.
 * Both outputs are device arrays that the call overwrites.
 * ------------------------------------------------------------------------------------------- */
size_t lf_hyb_stats_workspace_bytes(int64_t num_rows, int64_t num_cols, int32_t num_parts);
int lf_hyb_stats(const int64_t* indptr /*[dev] M+1*/, const int32_t* indices /*[dev] nnz*/,
                 int64_t num_rows, int64_t num_cols, int32_t num_parts,
                 int64_t* class_stats /*[dev] P*11*3*/, int64_t* colmask_hist /*[dev] P*2048*/,
                 void* workspace /*[dev]*/, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * lf_hyb_stats without any workspace argument.  It has no counterpart in the reference; it is
 * lf_hyb_stats for callers that must not allocate device memory and cannot be handed a scratch
 * buffer either: a call site inside a serving loop that promised the rest of the process a fixed
 * memory footprint, or a plugin whose host owns the allocator (a cudaMalloc there would also
 * synchronise the whole device in the middle of somebody else's work).  The per-column scratch
 * lives in a static device array inside the library instead: LF_STATIC_STATS_MAX_COLS * 4 bytes
 * plus the 128 KiB list of long row segments, 4 MiB + 128 KiB on every GPU that loads the
 * library, until the process exits.
 *   - matrices with more than LF_STATIC_STATS_MAX_COLS columns are refused (LF_ERR_UNSUPPORTED);
 *   - the first call on a device looks up the array's device address (a one-time set-up that is
 *     not stream work), so make that first call before any stream capture begins;
 *   - the array is shared by all calls and keeps whatever the last call left in it: each call
 *     clears the part it uses on `stream` first, and two calls that may overlap on the GPU
 *     (different streams, or host threads on different streams) race on it -- serialise them;
 *   - no cudaMalloc, cudaFree or other allocating routine is called; class_stats and
 *     colmask_hist are the caller's buffers exactly as for lf_hyb_stats;
 *   - the looked-up address is kept per device ordinal for the life of the process: after a
 *     cudaDeviceReset of that device it no longer names the array -- a process that resets a
 *     device must not call this entry point on it again.
 * ------------------------------------------------------------------------------------------- */
#define LF_STATIC_STATS_MAX_COLS (1 << 20)
int lf_hyb_stats_static(const int64_t* indptr /*[dev] M+1*/, const int32_t* indices /*[dev] nnz*/,
                        int64_t num_rows, int64_t num_cols, int32_t num_parts,
                        int64_t* class_stats /*[dev] P*11*3*/, int64_t* colmask_hist /*[dev] P*2048*/,
                        void* stream);

/* ---------------------------------------------------------------------------------------------
 * Description of a composed (column-partitioned, bucketed ELL) matrix in device memory.
 * This is the device form of build_hyb_format's return value (format_algos.py:226-237, 385):
 * for partition p and bucket b (global bucket index i = part_bucket_off[p] + b, width widths[i])
 *   rows + row_off[i]  : int32[ell_rows[i]]            == row_indices_nd[p][b]
 *   cols + slot_off[i] : int32[ell_rows[i]][widths[i]] == col_indices_nd[p][b]
 *   mask + slot_off[i] : uint8 [ell_rows[i]][widths[i]] == mask_nd[p][b]
 *   vals + slot_off[i] : float [ell_rows[i]][widths[i]]   the matrix values where mask is 1 and
 *                        0 in the padding (the reference stores no values: its matrices are all
 *                        ones and the mask itself is uploaded as A, format_algos.py:568-570)
 * Bucket starts are aligned to 64 elements; the gaps hold zeros.
 * zero_rows lists the matrix rows of [row_begin,row_end) that the SpMM must clear before it
 * accumulates: rows without any entry and rows held by more than one ELL row.
 * ------------------------------------------------------------------------------------------- */
typedef struct lf_hyb {
  int64_t num_rows;                 /* M of the whole matrix                               */
  int64_t num_cols;                 /* K                                                   */
  int64_t row_begin, row_end;       /* matrix rows covered by this (shard of the) format   */
  int32_t num_parts;                /* P                                                   */
  int32_t num_buckets;              /* total over partitions                               */
  const int32_t* part_bucket_off;   /* [host] P+1                                          */
  const int32_t* widths;            /* [host] num_buckets, ascending powers of two per part */
  const int64_t* ell_rows;          /* [host] num_buckets                                  */
  const int64_t* row_off;           /* [host] num_buckets+1                                */
  const int64_t* slot_off;          /* [host] num_buckets+1                                */
  const int32_t* rows;              /* [dev] row_off[num_buckets]                          */
  const int32_t* cols;              /* [dev] slot_off[num_buckets]                         */
  const float* vals;                /* [dev] slot_off[num_buckets]                         */
  const uint8_t* mask;              /* [dev] slot_off[num_buckets] or NULL                 */
  const int32_t* zero_rows;         /* [dev] num_zero_rows or NULL                         */
  int64_t num_zero_rows;
} lf_hyb;

/* ---------------------------------------------------------------------------------------------
 * Format construction, split in two calls so the caller can allocate the outputs in between.
 * Together they replace build_hyb_format (playground_pipline/format_algos.py:226-385): rows of
 * [row_begin,row_end) are placed, per partition, in the bucket bisect_left(widths, degree) clamped
 * to the widest (format_algos.py:275-278); a row longer than its bucket width becomes consecutive
 * ELL rows carrying the same row id (format_algos.py:286-305); unfinished ELL rows are padded with
 * column 0 / mask 0 (format_algos.py:297-299, 344-350).  Inside a bucket ELL rows are ordered by
 * matrix row, so a row range yields a contiguous slice of every bucket of the whole-matrix format.
 *
 * lf_hyb_plan counts: it fills ell_rows[], row_off[], slot_off[] (host) and *num_zero_rows, and
 * leaves per-block offsets in `workspace` for lf_hyb_fill, which must be given the same
 * workspace contents, the same matrix, widths and row range.  lf_hyb_fill writes four slots at a
 * time: cols and vals must be 16-byte aligned, mask (if given) 4-byte aligned.
 * ------------------------------------------------------------------------------------------- */
size_t lf_hyb_build_workspace_bytes(int64_t row_begin, int64_t row_end, int32_t num_parts,
                                    int32_t num_buckets);
/* extra scratch lf_hyb_fill needs once the plan is known (appended by the caller's allocation) */
size_t lf_hyb_fill_scratch_bytes(int64_t total_ell_rows);
int lf_hyb_plan(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/,
                int64_t num_rows, int64_t num_cols, int64_t row_begin, int64_t row_end,
                int32_t num_parts, const int32_t* part_bucket_off /*[host] P+1*/,
                const int32_t* widths /*[host]*/,
                int64_t* ell_rows /*[host] out*/, int64_t* row_off /*[host] out*/,
                int64_t* slot_off /*[host] out*/, int64_t* num_zero_rows /*[host] out*/,
                void* workspace /*[dev]*/, size_t workspace_bytes, void* stream);
int lf_hyb_fill(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/,
                const float* data /*[dev] or NULL: all ones*/,
                const lf_hyb* layout /* host arrays from lf_hyb_plan; device outputs written */,
                void* workspace /*[dev]*/, size_t workspace_bytes,
                void* scratch /*[dev]*/, size_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * SpMM on the composed format: C[row_begin:row_end, 0:N] (=|+=) A[row_begin:row_end, :] * B.
 * Replaces the kernel that bench_hyb_with_config generates, compiles and launches
 * (playground_pipline/format_algos.py:388-605; arithmetic format_algos.py:99-102; launch shape
 * format_algos.py:503-539).  All buckets of all partitions run in one launch.  C points at the
 * first row of the shard (row row_begin), ldb/ldc are in elements.
 * Padding slots are recognised by their stored value 0 and gather nothing; a stored entry whose
 * value is exactly 0 is skipped the same way, so it does not propagate an Inf or NaN of B into C.
 * ------------------------------------------------------------------------------------------- */
int lf_spmm_hyb_f32(const lf_hyb* A, const float* B /*[dev] K x N*/, int64_t ldb,
                    float* C /*[dev] (row_end-row_begin) x N*/, int64_t ldc, int32_t N,
                    int32_t flags, void* stream);

/* Name of the kernel lf_spmm_hyb_f32 launches for these operands under the current options
 * ("spmm_hyb_ring_kernel" or "spmm_hyb_kernel"); launches nothing.  For logs and benchmarks. */
const char* lf_spmm_hyb_f32_kernel_name(const lf_hyb* A, const float* B, int64_t ldb, const float* C, int64_t ldc,
                                        int32_t N);

/* The same product with B in bf16 (raw 16-bit patterns), values and accumulation in float32, C in
 * float32: halves the bytes of every gather.  N and ldb multiples of 8, ldc of 4, B and C 16-byte
 * aligned (LF_ERR_UNSUPPORTED otherwise).  Matches the float64 product of the rounded B to 1e-5 and
 * the unrounded one to 1e-2 relative. */
int lf_spmm_hyb_bf16(const lf_hyb* A, const uint16_t* B /*[dev] K x N bf16*/, int64_t ldb,
                     float* C /*[dev]*/, int64_t ldc, int32_t N, int32_t flags, void* stream);

/* The same product fused with the all-gather of C (no counterpart in the reference, which runs on
 * one device, format_algos.py:548): every output row of this shard is written by the kernel's
 * epilogue into num_dests FULL-size C matrices at once -- C_full[k] points at row 0 of a
 * num_rows x N matrix on GPU k of the group, this GPU's own buffer included, reachable from this
 * GPU through peer mappings (plain peer stores and peer vector atomics over NVLink; no
 * multicast).  Each rank calls it for its own row shard; after a barrier over the group every
 * buffer holds the whole product, without a separate collective and without re-reading C.
 * Always overwrites.  N, ldb, ldc multiples of 4, all operands 16-byte aligned. */
#define LF_MAX_DESTS 8
int lf_spmm_hyb_f32_bcast(const lf_hyb* A, const float* B /*[dev] K x N*/, int64_t ldb,
                          float* const* C_full /*[host] num_dests device pointers*/, int32_t num_dests,
                          int64_t ldc, int32_t N, void* stream);

/* Ragged all-gather of C (no counterpart in the reference, which runs on one device): this rank's
 * row block -- `rows` rows of N floats at C_rows, the rows [row_begin, row_begin + rows) of the
 * whole product -- is copied into the same rows of num_dests full-size C matrices, C_full[k]
 * pointing at row 0 of the buffer on GPU k of the group (this GPU's included), reachable through
 * peer mappings.  Row blocks may differ in size from rank to rank, which NCCL's all-gather does not
 * take; every rank calls this for its own block, a barrier over the group before (nobody still
 * reads the buffers) and after (all blocks have landed) completes the gather.  Plain peer stores,
 * each row crosses NVLink once per destination; no multicast, no staging copy. */
int lf_allgather_rows(const float* C_rows /*[dev]*/, int64_t ld_rows, int64_t row_begin, int64_t rows, int32_t N,
                      float* const* C_full /*[host] num_dests device pointers*/, int32_t num_dests, int64_t ldc,
                      void* stream);

/* Same product with every operand in HOST memory: the arrays of build_hyb_format as NumPy holds
 * them after the int32/float32 casts of format_algos.py:568-577, B and C row-major.  The call
 * copies the format and B into `device_workspace`, runs lf_spmm_hyb_f32 and copies C back, all on
 * `stream`, and synchronises (unless LF_SPMM_NO_SYNC is set; host buffers must then be pinned for
 * the copies to run asynchronously).  It is what one call of bench_hyb_with_config does between
 * format_algos.py:546 and format_algos.py:595, without the run-time code generation. */
size_t lf_spmm_hyb_f32_host_workspace_bytes(const lf_hyb* A_host, int32_t N);
int lf_spmm_hyb_f32_host(const lf_hyb* A_host /* rows/cols/vals/zero_rows are [host] here */,
                         const float* B /*[host]*/, float* C /*[host]*/, int32_t N, int32_t flags,
                         void* device_workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * CSR SpMM, C = A * B.  Replaces the kernel of bench_naive (playground_pipline/
 * format_algos.py:1660-1755); also the fallback the reference pipeline takes when the block
 * format fails (proc05.spmm.end-to-end.py:237-249).  Work is split by stored entries, not by
 * rows: a long row is shared by many thread groups (vector atomics into rows that a preparation
 * launch cleared) and short rows are packed together, so no format has to be built first.
 * ------------------------------------------------------------------------------------------- */
int lf_spmm_csr_f32(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/,
                    const float* data /*[dev] or NULL: all ones*/, int64_t row_begin, int64_t row_end,
                    int64_t nnz /* exact number of entries of rows [row_begin,row_end), or -1: the call
                                   reads it back and synchronises the stream */,
                    const float* B /*[dev]*/, int64_t ldb, float* C /*[dev]*/, int64_t ldc,
                    int32_t N, void* stream);

/* ---------------------------------------------------------------------------------------------
 * CSR -> 8x8 block-sparse rows on the device.
 * Replaces MTX.tobsr_with_padding (playground_pipline/format_matrix_market.py:116-138), which pads
 * the shape and calls scipy.sparse.bsr_matrix on the host.  The result is what SciPy builds for
 * blocksize (8, 8) after sort_indices(): bsr_indptr int64[ceil(M/8)+1], block columns ascending
 * inside a block row, tiles [nb][8][8] row-major with zeros where the matrix has no entry; rows
 * past M (padding up to a multiple of 8) are empty.  indptr/indices/data: canonical CSR (sorted
 * columns, no duplicates); data == NULL stands for all ones (what MTX gives a pattern file,
 * format_matrix_market.py:58-65).
 *   lf_bsr8_plan  counts the blocks: writes bsr_indptr, returns *num_blocks on the host
 *                 (synchronises the stream); the caller then allocates the block arrays.
 *   lf_bsr8_fill  writes bsr_indices int32[nb] and blocks[nb*64] in the dtype asked for
 *                 (values are rounded to nearest even from float32).
 * ------------------------------------------------------------------------------------------- */
#define LF_DTYPE_F32 0
#define LF_DTYPE_BF16 1
#define LF_DTYPE_F16 2
int lf_bsr8_plan(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/, int64_t M,
                 int64_t* bsr_indptr /*[dev] out*/, int64_t* num_blocks /*[host] out*/, void* stream);
int lf_bsr8_fill(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/, const float* data /*[dev]*/,
                 int64_t M, const int64_t* bsr_indptr /*[dev]*/, int32_t* bsr_indices /*[dev] out*/,
                 void* blocks /*[dev] out*/, int32_t dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Coarse blocks -> 8x8 tiles on the device.  The reference hands its block path a SciPy BSR matrix
 * with 32x32 fp16 blocks (bench_bsrmm(bsr_mat, x, block_size=32), playground_pipline/
 * format_algos.py:1562-1643, built by MTX.tobsr_with_padding, format_matrix_market.py:116-138).
 * These two calls cut R x C blocks (multiples of 8; indptr int64[block_rows+1], block columns
 * sorted inside a block row, data [num_blocks][R][C] in in_dtype) into the 8x8 tiles the product
 * kernels take and drop the tiles that hold only zeros, so the padding inside coarse blocks costs
 * nothing.  The result equals scipy.sparse.bsr_matrix(blocksize=(8, 8)) of the same matrix after
 * eliminate_zeros(): tile (a, c) of a block in block row I, block column J lands in fine block row
 * I*R/8 + a with block column J*C/8 + c.
 *   lf_bsr_split8_plan  flags and counts: writes out_indptr int64[block_rows*R/8 + 1], returns
 *                       *num_tiles on the host (synchronises the stream); `scratch` keeps one
 *                       byte per candidate tile for the fill.
 *   lf_bsr_split8_fill  writes out_indices int32[num_tiles] and out_blocks[num_tiles*64] in
 *                       out_dtype (converted through float32, round to nearest even).
 * ------------------------------------------------------------------------------------------- */
size_t lf_bsr_split8_scratch_bytes(int64_t num_blocks, int32_t R, int32_t C);
int lf_bsr_split8_plan(const int64_t* indptr /*[dev]*/, const void* data /*[dev]*/, int32_t in_dtype,
                       int64_t block_rows, int64_t num_blocks, int32_t R, int32_t C,
                       void* scratch /*[dev]*/, size_t scratch_bytes, int64_t* out_indptr /*[dev] out*/,
                       int64_t* num_tiles /*[host] out*/, void* stream);
int lf_bsr_split8_fill(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/, const void* data /*[dev]*/,
                       int32_t in_dtype, int64_t block_rows, int64_t num_blocks, int32_t R, int32_t C,
                       const void* scratch /*[dev] as left by the plan*/, const int64_t* out_indptr /*[dev]*/,
                       int32_t* out_indices /*[dev] out*/, void* out_blocks /*[dev] out*/, int32_t out_dtype,
                       void* stream);

/* ---------------------------------------------------------------------------------------------
 * Block-sparse SpMM, 8x8 blocks (BSR): C[block_row_begin*8 : block_row_end*8, 0:N] = A * B.
 * Replaces the kernel of bench_bsrmm (playground_pipline/format_algos.py:1562-1643; arithmetic
 * format_algos.py:1204-1213), which runs 32x32 fp16 blocks through wmma with fp16 accumulators
 * (format_algos.py:1226-1233).  Here: indptr int64[Mb+1], indices int32[nb] (block columns, sorted
 * inside a block row as scipy.sparse.bsr_matrix keeps them, format_matrix_market.py:137), blocks
 * [nb][8][8] row-major.  Accumulation is fp32 in every variant; the float32 variant splits each
 * operand into two tf32 halves (three tensor-core products) and matches an fp32 product to ~1e-6
 * relative.  N, ldb must be multiples of 4 (float32) or 8 (16-bit), ldc of 4, B and C 16-byte aligned.
 * C points at row block_row_begin*8.
 * ------------------------------------------------------------------------------------------- */
int lf_spmm_bsr8_f32(const int64_t* indptr /*[dev]*/, const int32_t* indices /*[dev]*/,
                     const float* blocks /*[dev]*/, int64_t block_row_begin, int64_t block_row_end,
                     const float* B /*[dev]*/, int64_t ldb, float* C /*[dev]*/, int64_t ldc, int32_t N,
                     void* stream);
/* Tuning of the block kernels (results do not depend on it): features per warp of the float32
 * kernel in units of 64 (0 = automatic, 1, 2), depth of the per-warp copy ring (0 = automatic, 3,
 * 4) and block rows one warp streams through (0 = automatic, 1..31). */
int lf_bsr_set_tuning(int32_t feat_units, int32_t stages, int32_t rows_per_warp);
/* The block kernels that copy through the tensor memory accelerator bound every wait for a copy; a
 * warp that gives up leaves its rows of C unfinished and counts itself.  This call synchronises
 * the stream and returns LF_ERR_KERNEL_TIMEOUT if any warp gave up since the last call (clearing
 * the count), LF_OK otherwise.  No counterpart in the reference. */
int lf_bsr_copy_status(void* stream);
/* bf16 blocks and bf16 B (raw 16-bit patterns), float32 C */
int lf_spmm_bsr8_bf16(const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                      int64_t block_row_begin, int64_t block_row_end, const uint16_t* B, int64_t ldb,
                      float* C, int64_t ldc, int32_t N, void* stream);
/* fp16 blocks and fp16 B (the reference's input type, format_algos.py:1629-1637), float32 C */
int lf_spmm_bsr8_f16(const int64_t* indptr, const int32_t* indices, const uint16_t* blocks,
                     int64_t block_row_begin, int64_t block_row_end, const uint16_t* B, int64_t ldb,
                     float* C, int64_t ldc, int32_t N, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Row-length statistics behind MTX.matrix_features (playground_pipline/format_matrix_market.py:
 * 153-202, a Python loop over all rows in the reference).  One record of four uint64 per block of
 * 256 rows: sum, sum of squares, minimum, maximum of the row lengths of rows [row_begin, row_end).
 * partials holds lf_row_stats_blocks() * 4 values; the caller folds the exact integers.
 * ------------------------------------------------------------------------------------------- */
int64_t lf_row_stats_blocks(int64_t row_begin, int64_t row_end);
int lf_row_stats(const int64_t* indptr /*[dev]*/, int64_t row_begin, int64_t row_end,
                 uint64_t* partials /*[dev]*/, void* stream);

/* ---------------------------------------------------------------------------------------------
 * nnz-balanced contiguous row ranges for G devices: splits[g] = first row r with
 * indptr[r] >= g*nnz/G, splits[0] = 0, splits[G] = M.  (No counterpart in the reference, which
 * runs on device 0 only, format_algos.py:548.)
 * ------------------------------------------------------------------------------------------- */
int lf_shard_rows(const int64_t* indptr /*[dev]*/, int64_t num_rows, int32_t num_shards,
                  int64_t* splits /*[dev] G+1, written asynchronously on `stream`*/, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LITEFORM_B200_H_ */
