/*
 * s24.h -- C ABI of the B200 (sm_100a) 2:4 structured-sparsity library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void*, i.e. a cudaStream_t / CUstream; NULL = the legacy default stream).  Nothing
 * on the compute path allocates device memory, synchronises the device or throws: each
 * call enqueues work on the given stream and returns S24_OK or a negative S24_ERR_* code
 * whose text is available (per calling thread) from s24_last_error().  The exceptions are
 * set-up and debug helpers and say so: s24_peer_alloc / s24_peer_free / s24_peer_open /
 * s24_peer_close (multi-GPU buffers) and s24_device_status (reads a status word back).
 *
 * Per-device state.  The library caches three things per device ordinal, each written once
 * with the same value whichever thread gets there first (so concurrent first calls are
 * benign, but the caches are not locked): the SM count, the large-shared-memory opt-in of
 * each GEMM variant, and the device addresses of two objects inside the library image (the
 * status word and the built-in scratch buffer, looked up with cudaGetSymbolAddress).  They
 * assume one CUDA context per device for the life of the process (the primary context that
 * the runtime API uses); after cudaDeviceReset the library must be reloaded.  The first GEMM
 * call on a device performs these look-ups: make it, with the device current, before any
 * stream capture.  Up to 64 devices.
 *
 * The entry points replace, one for one, the GPU work behind these functions of the
 * reference project (paths relative to its root):
 *
 *   s24_prune            compression/prune.py:57-96           prune_2_4
 *   s24_compress         compression/compress_2_4.py:32-161   compress_dense_to_sparse (fp16 / bf16)
 *   s24_compress_other   same function, its int8 / int32 / float32 branches
 *   s24_prune_compress   compression/kernels/11.1_2_kernel_baseline.py:171-203,256-279
 *                                                             ws_tma_compress_2_4_kernel
 *   s24_meta_convert     compression/compress_2_4.py:6-30     _calculate_meta_reordering_offsets
 *   s24_spmm             compression/gluon_ws_sparse.py:244-278,560-613  run_sparse_ws_matmul
 *   s24_spmm_ref_meta    same launcher, fed the reference's metadata layout directly
 *   s24_spmm_bt          same launcher, B given transposed ((N, K) row-major)
 *   s24_spmm_prune_out   compression/kernels/10.1_prune_acc.py:88-154,359-398,624-678
 *   s24_spmm_prune_in    compression/kernels/7.8.1_prune_ws.py:112-192,345-374,609-650
 *
 * Element types: S24_FP16 / S24_BF16, 16-bit storage, row-major matrices.
 *
 * Metadata layouts (all describe the same logical array meta[M][K/16] of 16-bit words,
 * group 4c+j of a row in bits 4j..4j+3 of word c, each group coded idx0 | idx1 << 2):
 *   S24_META_LOGICAL  meta[r][c], int16 (M, K/16)
 *   S24_META_REF      the reference's reordered buffer viewed (M/16, K) int16:
 *                     E[r/16][(c/4)*64 + (r%8)*8 + (c%4)*2 + (r/8)%2] = meta[r][c]
 *   S24_META_TC       records of 2048 bytes per (128-row tile t, 128-column block kb),
 *                     ordered [t][kb]; a record is 128 lanes x 4 words, lane
 *                     L = m0 + 8*k1 + 16*m2 and word j holding
 *                     meta[128t+16*m2+m0][8kb+2j+k1] | meta[128t+16*m2+8+m0][8kb+2j+k1] << 16.
 *                     This is the image tcgen05.cp (128x128b) moves into tensor memory for
 *                     four consecutive tcgen05.mma.sp instructions of K = 32.
 *                     There are ceil(M/128) x ceil(K/128) whole records; where M or K is not a
 *                     multiple of 128 the words of rows >= M and of columns >= K hold a filler
 *                     code (0x44 bytes; the values they index read as zero).  Every entry
 *                     point that writes this layout sets the filler itself, with an
 *                     asynchronous memset on the caller's stream before its kernel; a caller
 *                     that builds such a buffer on its own must do the same.
 */
#ifndef S24_H_
#define S24_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define S24_API __attribute__((visibility("default")))
#else
#define S24_API
#endif

#define S24_VERSION 1

/* status codes */
#define S24_OK 0
#define S24_ERR_INVALID_ARG (-1)   /* null pointer, bad enum, bad alignment */
#define S24_ERR_SHAPE (-2)         /* a divisibility or range rule on M, N, K, ld* failed */
#define S24_ERR_CUDA (-3)          /* a CUDA runtime / driver call failed */
#define S24_ERR_UNSUPPORTED (-4)   /* valid request this build has no kernel for */
#define S24_ERR_TIMEOUT (-5)       /* a bounded device-side wait gave up (status word set) */

/* element types */
#define S24_FP16 0
#define S24_BF16 1
/* accepted by s24_compress_other only */
#define S24_INT8 2
#define S24_INT32 3
#define S24_FP32 4

/* which keys rank the four elements of a group */
#define S24_MODE_SIGNED 0          /* the values themselves: prune.py:85 (reference default) */
#define S24_MODE_MAGNITUDE 1       /* |value| */

/* which element survives when the 2nd and 3rd largest keys are equal */
#define S24_TIE_REFERENCE 0        /* exactly what prune_2_4 does on CPU tensors: the tie order of
                                      torch.topk(k=2, largest=False) in torch 2.11.0 (CPU), measured
                                      over all 75 weak orderings of four keys; torch.topk on CUDA
                                      tensors, or another torch release, may order ties differently */
#define S24_TIE_LOWER 1            /* lower index survives (kernels/10.1_prune_acc.py:100-105) */
#define S24_TIE_HIGHER 2           /* higher index survives (kernels/11.1_2_kernel_baseline.py:95-100) */

/* metadata layouts */
#define S24_META_LOGICAL 0
#define S24_META_REF 1
#define S24_META_TC 2

/* Optional tile choice for the GEMM entry points; NULL or zeros = heuristic.
 * Mirrors the keys of the reference's manual_config (gluon_ws_sparse.py:629-636). */
typedef struct s24_tile_cfg {
    int bm;        /* rows per tile: 128 (one CTA), 256 (CTA pair) or 512 (CTA pair, two row sub-tiles), 0 = auto */
    int bn;        /* columns per tile: 128 or 256; 224 with bm = 512; 0 = auto */
    int stages;    /* reserved, ignored: every tile shape has one ring depth (512x224: 3, 256x256: 4,
                      256x128: 6, 128x128: 4 stages of K = 128) that fills the 227 KB of shared memory */
    int reserved;
} s24_tile_cfg;

S24_API int s24_version(void);

/* text of the last error on the calling thread ("" if none) */
S24_API const char* s24_last_error(void);

/*
 * prune_2_4 (compression/prune.py:57-96): for every contiguous group of four along the
 * last dimension zero the two smallest keys; survivors keep their bit patterns, dropped
 * elements become +0.0.  `numel` elements are read from A and written to out as one flat,
 * contiguous array (any leading shape); numel % 4 must be 0 (the reference's
 * ValueError, prune.py:76-77) and both pointers 8-byte aligned.  out may equal A.
 */
S24_API int s24_prune(const void* A, void* out, int64_t numel, int dtype, int mode, int tie, void* stream);

/*
 * compress_dense_to_sparse (compression/compress_2_4.py:32-161) for 16-bit types: from
 * the non-zero flags of `dense` (M, K; row stride ld elements) write the two stored
 * values of each group to vals (M, K/2 contiguous) and the metadata in the reference's
 * reordered layout to meta_ref ((M/16, K) int16) and/or in the tensor-core layout to
 * meta_tc (s24_meta_tc_bytes(M, K) bytes); either metadata pointer may be NULL.
 * Needs M % 32 == 0, K % 64 == 0 (compress_2_4.py:10,57-65), ld % 8 == 0, 16-byte aligned
 * pointers.
 */
S24_API int s24_compress(const void* dense, int64_t M, int64_t K, int64_t ld, int dtype,
                 void* vals, void* meta_ref, void* meta_tc, void* stream);

/*
 * compress_dense_to_sparse for its element types beyond fp16 / bf16
 * (compression/compress_2_4.py:41-47,73-76,144-154), which no GEMM of the reference consumes:
 *   S24_INT8   2:4, metadata int32 with eight codes per word; M % 16 == 0, K % 32 == 0
 *   S24_INT32  2:4, metadata int16 with four codes per word;  M % 32 == 0, K % 16 == 0
 *   S24_FP32   1:2 (of every pair the first element if it is non-zero, else the second; codes 0100 /
 *              1110), metadata int16; M % 32 == 0, K % 16 == 0
 * and a number of metadata words per row that is a multiple of 4 (compress_2_4.py:10).  vals is
 * (M, K/2) of the element type, meta_ref the reordered metadata buffer of M * words-per-row
 * elements (the reference returns it viewed (M/2, 2 * words-per-row)).  dense has row stride ld
 * elements (a multiple of 16 bytes); dense and vals 16-byte aligned.
 */
S24_API int s24_compress_other(const void* dense, int64_t M, int64_t K, int64_t ld, int elem_type,
                       void* vals, void* meta_ref, void* stream);

/*
 * Fused prune + compress in one pass over A (the reference's standalone kernel,
 * compression/kernels/11.1_2_kernel_baseline.py:171-203): identical results to
 * s24_prune followed by s24_compress, A read once, nothing else read.
 * Algorithmic traffic 3.125 bytes per element of A with one metadata layout.
 */
S24_API int s24_prune_compress(const void* A, int64_t M, int64_t K, int64_t ld, int dtype, int mode, int tie,
                       void* vals, void* meta_ref, void* meta_tc, void* stream);

/* bytes of a S24_META_TC buffer for an (M, K) matrix: ceil(M/128) * ceil(K/128) * 2048
 * (= M * K / 8, one bit per element, when both are multiples of 128) */
S24_API size_t s24_meta_tc_bytes(int64_t M, int64_t K);

/*
 * Convert metadata between layouts (compression/compress_2_4.py:6-30 gives
 * LOGICAL -> REF).  M % 32 == 0 and K % 64 == 0.  src and dst must not overlap.
 */
S24_API int s24_meta_convert(const void* src, int from_layout, void* dst, int to_layout,
                     int64_t M, int64_t K, void* stream);

/*
 * run_sparse_ws_matmul (compression/gluon_ws_sparse.py:560-613):
 *   C (M, N) = A24 (M, K) . B (K, N), fp32 accumulation, C in the element type of A/B.
 * A24 is given as vals (M, K/2 contiguous) + meta_tc (S24_META_TC).  B has row stride
 * ldb, C row stride ldc (elements).  M % 32 == 0, K % 64 == 0 (every shape
 * compress_dense_to_sparse accepts; tiles and k-blocks that are only partly covered read
 * zeros), N % 8 == 0, ldb % 8 == 0, ldc % 8 == 0, 16-byte aligned pointers; meta_tc must
 * span s24_meta_tc_bytes(M, K).
 */
S24_API int s24_spmm(const void* vals, const void* meta_tc, const void* B, void* C,
             int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc, int dtype,
             const s24_tile_cfg* cfg, void* stream);

/*
 * The same product with B given transposed: Bt is (N, K) row-major with row stride ldbt, i.e.
 * C = A24 . Bt^T.  This is the layout of activations stored (tokens, hidden) when the sparse
 * operand is a weight; the reference's launcher takes (K, N) row-major only
 * (compression/gluon_ws_sparse.py:522-525,563) and a caller would have to transpose first.
 * Same rules as s24_spmm with ldbt >= K, ldbt % 8 == 0.
 */
S24_API int s24_spmm_bt(const void* vals, const void* meta_tc, const void* Bt, void* C,
                int64_t M, int64_t N, int64_t K, int64_t ldbt, int64_t ldc, int dtype,
                const s24_tile_cfg* cfg, void* stream);

/*
 * Same product with the metadata in the reference's layout (the E a caller of
 * run_sparse_ws_matmul holds, gluon_ws_sparse.py:655-658).  The layout conversion runs
 * first on the same stream into `workspace`, which the caller provides:
 * workspace_bytes >= s24_meta_tc_bytes(M, K), 16-byte aligned.
 */
S24_API int s24_spmm_ref_meta(const void* vals, const void* meta_ref, const void* B, void* C,
                      int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc, int dtype,
                      const s24_tile_cfg* cfg, void* workspace, size_t workspace_bytes, void* stream);

/*
 * s24_spmm_ref_meta for callers that cannot hand the library a workspace.  This entry point
 * has no counterpart in the reference (whose launcher allocates freely through torch).
 *
 * Who needs it: code that runs with a device-memory budget fixed at start-up and may not
 * allocate afterwards -- a plugin inside a serving process whose HBM was carved up among
 * models when it started, an embedding host whose allocator must not be bypassed, a
 * latency-bound loop that cannot afford cudaMalloc's device-wide synchronisation.  Such a
 * caller owns its inputs and outputs but has nowhere to get the scratch buffer from.
 *
 * What it does: the re-laid metadata goes into a buffer of S24_STATIC_SCRATCH_BYTES that is
 * part of the library image on the device (every GPU that loads libs24 holds these bytes
 * until the process exits).  No cudaMalloc, cudaFree or allocating library routine is
 * called.  Limits and rules:
 *   - s24_meta_tc_bytes(M, K) = ceil(M/128) * ceil(K/128) * 2048 must not exceed
 *     S24_STATIC_SCRATCH_BYTES (8192 x 8192 fits exactly; for multiples of 128 the rule reads
 *     M * K <= 2^26, other shapes count whole 128 x 128 records); larger problems are
 *     rejected with S24_ERR_SHAPE and a message naming both sizes;
 *   - the first call on each device looks up the buffer's device address
 *     (cudaGetSymbolAddress) and caches it; make that first call, with the device current,
 *     before any stream capture you may use;
 *   - all calls on a device share the one buffer, which keeps whatever the previous call
 *     left in it.  Every byte the GEMM reads is rewritten by the call itself, so nothing
 *     needs clearing, but two calls whose kernels overlap on the GPU (different streams
 *     without an ordering between them) race on it: serialise them.
 * Arguments and all other rules as s24_spmm_ref_meta.
 */
#define S24_STATIC_SCRATCH_BYTES (8u << 20)
S24_API int s24_spmm_ref_meta_noalloc(const void* vals, const void* meta_ref, const void* B, void* C,
                              int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc, int dtype,
                              const s24_tile_cfg* cfg, void* stream);

/*
 * Sparse GEMM whose epilogue 2:4-prunes the accumulator along N on its way out of tensor
 * memory and stores it compressed (compression/kernels/10.1_prune_acc.py:88-154,624-678):
 * C_vals (M, N/2) in the element type and metadata of the (M, N) result in the reference
 * layout C_meta_ref ((M/16, N) int16) and/or C_meta_tc; either may be NULL.  Keys are the
 * signed accumulator values, ties keep the lower index and the codes come from the keep
 * mask, as in 10.1_prune_acc.py:100-117.  The groups are ranked after the fp32 sums have been
 * rounded to the element type: the output is, bit for bit, prune + compress (lower index on
 * ties) of the C that s24_spmm stores for the same operands and tile.  The reference's kernel
 * ranks the unrounded fp32 values and rounds the survivors (:241); the two differ only in
 * groups whose second and third largest sums round to the same 16-bit number, i.e. well inside
 * the tolerance the GEMM itself is held to.  Needs N % 128 == 0 in addition to the s24_spmm rules.
 */
S24_API int s24_spmm_prune_out(const void* vals, const void* meta_tc, const void* B,
                       void* C_vals, void* C_meta_ref, void* C_meta_tc,
                       int64_t M, int64_t N, int64_t K, int64_t ldb, int dtype,
                       const s24_tile_cfg* cfg, void* stream);

/*
 * Sparse GEMM that takes its left operand DENSE and 2:4-prunes + compresses it inside the
 * kernel, C = prune_2_4(A) . B (compression/kernels/7.8.1_prune_ws.py:609-650,
 * run_sparse_ws_matmul(A, B); in-kernel prune :112-192).  A is (M, K) with row stride lda,
 * never modified; no compressed operand or metadata is written to memory.  mode and tie as
 * for s24_prune_compress (the reference's kernel ranks signed values with a strict compare,
 * i.e. S24_MODE_SIGNED with S24_TIE_HIGHER; S24_TIE_REFERENCE gives the survivors of the torch
 * function prune_2_4 that the reference checks its kernel against).  Shape rules as for s24_spmm plus
 * lda >= K, lda % 8 == 0.  The result is bit-identical to s24_prune_compress followed by
 * s24_spmm on the 512 x 224 tile (same MMA shape).  One tile shape (256 x 480 per CTA pair, two
 * column sub-tiles sharing each pruned A stage); every k-block of A is pruned once per 480
 * columns of C, so for large N the two-kernel path is the faster one.
 */
S24_API int s24_spmm_prune_in(const void* A, int64_t lda, const void* B, void* C,
                      int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc,
                      int dtype, int mode, int tie, void* stream);

/*
 * Multi-GPU: replicated result without a separate all-gather (the reference is single-GPU; no
 * counterpart there).  s24_spmm_scatter is s24_spmm whose epilogue stores every tile of C to
 * n_dst (1..8) destinations instead of one: dsts[d] points at element (0, 0) of this call's
 * (M, N) block inside destination d, all destinations share the row stride ldc.  With C
 * (M, N_total) replicated over G GPUs and the columns of B sharded, rank r passes, for every
 * rank g, the address of column r * N/G of g's copy of C as mapped into r's address space
 * (s24_peer_open); the shard then crosses NVLink tile by tile while the GEMM runs, as whole
 * 256-byte row segments.  Only stores go to peer memory.  The caller orders the ranks (a barrier
 * or any collective on the stream) before C is read and before the next call overwrites it.
 * 256 x 256 tile; shape rules as for s24_spmm.
 */
S24_API int s24_spmm_scatter(const void* vals, const void* meta_tc, const void* B,
                     void* const* dsts, int n_dst,
                     int64_t M, int64_t N, int64_t K, int64_t ldb, int64_t ldc,
                     int dtype, void* stream);

/*
 * Buffers for the above (no counterpart in the reference).  s24_peer_alloc / s24_peer_free:
 * device memory of the current device that can be exported (plain cudaMalloc / cudaFree: they
 * synchronise; set-up code only).  s24_peer_export writes an opaque S24_PEER_HANDLE_BYTES-byte
 * handle that another process on the same box passes to s24_peer_open, with its own device
 * current, to get an address its kernels can store to; s24_peer_close unmaps it.  A buffer must
 * be closed by every opener before its owner frees it.
 */
#define S24_PEER_HANDLE_BYTES 64
S24_API int s24_peer_alloc(size_t bytes, void** ptr);
S24_API int s24_peer_free(void* ptr);
S24_API int s24_peer_export(const void* ptr, void* handle);
S24_API int s24_peer_open(const void* handle, void** ptr);
S24_API int s24_peer_close(void* ptr);

/*
 * Copy `rows` rows of `width_bytes` bytes from src (row pitch src_pitch bytes) to dst (row pitch
 * dst_pitch bytes) on `stream` with the copy engines (no counterpart in the reference).  dst may
 * be a mapping from s24_peer_open: this is how a rank pushes its column shard of C into the other
 * ranks' copies of C while its SMs keep multiplying the next row panel.  Enqueues only; the
 * caller orders the ranks afterwards as for s24_spmm_scatter.
 */
S24_API int s24_peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows, void* stream);

/*
 * Multi-GPU helper (the reference is single-GPU; no counterpart there).  When C is computed in
 * column shards, one per rank, an all-gather delivers them shard-major: stage is
 * (shards, rows, shard_cols) contiguous, 16-bit elements.  This writes the row-major matrix
 * out[r][g * shard_cols + c] = stage[g][r][c] with row stride ldo (elements).
 * shard_cols % 8 == 0, ldo % 8 == 0, ldo >= shards * shard_cols, 16-byte aligned pointers.
 */
S24_API int s24_relayout_shards(const void* stage, void* out, int64_t rows, int64_t shards, int64_t shard_cols,
                        int64_t ldo, void* stream);

/*
 * Debug / test aid (no counterpart in the reference): every device-side wait in the GEMM
 * kernels is bounded (2 s); if one gives up the kernel records a code, frees its tensor memory
 * and returns, and the launch itself still reports S24_OK with C partly written.  This call
 * synchronises `stream`, returns S24_OK if no kernel on the current device has reported a
 * failure since the last call, else S24_ERR_TIMEOUT (code in s24_last_error()), and clears
 * the record.  A caller that must not consume a partly written result polls it at its next
 * synchronisation point (the Python front end does so after every GEMM when S24_CHECK_STATUS=1).
 */
S24_API int s24_device_status(void* stream);

/*
 * Self-test of that time-out path (no counterpart in the reference).  Nothing here can hang:
 * every wait involved gives up after one millisecond.
 *   kind 0: one thread waits on a barrier that nothing will ever complete, sees the wait run
 *           out and records code 7.  The operand arguments are ignored (pass NULL / 0).
 *   kind 1: the GEMM s24_spmm would run for these operands (ldb = ldc = N), except that its
 *           producer stops loading after the first k-block, so the MMA and epilogue roles run
 *           out of data, take their time-out branches, the kernel frees its tensor memory and
 *           returns.  K must span at least two k-blocks of 128.  C is left partly written.
 * Either way the launch returns S24_OK and s24_device_status() then reports S24_ERR_TIMEOUT
 * once; the context stays usable.
 */
S24_API int s24_selftest_timeout(int kind, const void* vals, const void* meta_tc, const void* B, void* C,
                         int64_t M, int64_t N, int64_t K, int dtype, const s24_tile_cfg* cfg, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* S24_H_ */
