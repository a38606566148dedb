// prune_compress.cu -- bandwidth-bound kernels: 2:4 prune, compress, fused prune+compress
// and metadata layout conversion.
//
// Replaces the GPU work behind the reference's prune_2_4 (compression/prune.py:57-96),
// compress_dense_to_sparse (compression/compress_2_4.py:32-161) and its standalone fused
// kernel ws_tma_compress_2_4_kernel (compression/kernels/11.1_2_kernel_baseline.py:171-203).
//
// Fused kernel layout.  One warp owns a 16-row x 128-column block of A.  Lane
// (m0 = lane/4, jj = lane%4) reads rows m0 and m0+8 of the block, 32 consecutive
// elements each (64 bytes per row, two 256-bit loads), so a warp-wide load covers whole
// 128-byte lines.  All ranking happens in registers of the owning lane -- no shared memory,
// no shuffles -- and the choice of rows (r, r+8) and 32-column spans makes every output
// store a full-line store:
//   * values:   32 bytes per row per lane, 4 lanes = one 128-byte line;
//   * metadata, reference layout: the lane holds two adjacent 32-bit words of the
//     reordered buffer, the warp writes two full 128-byte lines;
//   * metadata, tensor-core layout: lane index == word index within a 128-byte line.
// Algorithmic traffic: 2 bytes read + 1 byte of values + 1/8 byte of metadata per element
// (plus another 1/8 if both metadata layouts are requested).
#include "s24_common.cuh"
#include "prune_core.cuh"

namespace s24 {

__device__ __forceinline__ void st128x2(void* p, const uint32_t (&r)[8])
{
    *reinterpret_cast<uint4*>(p) = make_uint4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<uint4*>(static_cast<char*>(p) + 16) = make_uint4(r[4], r[5], r[6], r[7]);
}

__device__ __forceinline__ void st256(void* p, const uint32_t (&r)[8])
{
    asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

struct PcParams {
    const uint16_t* A;
    int64_t lda;       // elements
    int64_t M, K;
    uint16_t* vals;    // (M, K/2)
    uint32_t* meta_ref;  // (M/16, K/2) words, may be null
    uint32_t* meta_tc;   // records, may be null
    int tie;
    int64_t col_blocks;  // ceil(K / 128)
    int64_t warp_tiles;  // (M/16) * col_blocks
};

template <int DT, int MODE, bool LD256>
__global__ void __launch_bounds__(256) prune_compress_kernel(const PcParams p)
{
    const int lane = threadIdx.x & 31;
    const int64_t wt = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wt >= p.warp_tiles) return;
    const int64_t row16 = wt / p.col_blocks;
    const int64_t cb = wt - row16 * p.col_blocks;
    const int m0 = lane >> 2, jj = lane & 3;
    const int64_t col0 = cb * 128 + jj * 32;
    if (col0 >= p.K) return;  // K % 128 == 64: the upper two lanes of each row are idle
    const int64_t rA = row16 * 16 + m0, rB = rA + 8;

    uint32_t a_lo[8], a_hi[8], b_lo[8], b_hi[8];
    const uint16_t* pa = p.A + rA * p.lda + col0;
    const uint16_t* pb = p.A + rB * p.lda + col0;
    if (LD256) {
        ld256(pa, a_lo);
        ld256(pa + 16, a_hi);
        ld256(pb, b_lo);
        ld256(pb + 16, b_hi);
    } else {
        ld128x2(pa, a_lo);
        ld128x2(pa + 16, a_hi);
        ld128x2(pb, b_lo);
        ld128x2(pb + 16, b_hi);
    }

    uint32_t va[8], vb[8];
    const uint32_t ma = row_span<DT, MODE>(a_lo, a_hi, p.tie, va);
    const uint32_t mb = row_span<DT, MODE>(b_lo, b_hi, p.tie, vb);

    const int64_t half_k = p.K >> 1;
    if (LD256) {   // 256-bit accesses need 32-byte alignment of A, its row stride and vals
        st256(p.vals + rA * half_k + (col0 >> 1), va);
        st256(p.vals + rB * half_k + (col0 >> 1), vb);
    } else {
        st128x2(p.vals + rA * half_k + (col0 >> 1), va);
        st128x2(p.vals + rB * half_k + (col0 >> 1), vb);
    }

    // metadata words: row r in the low half, row r+8 in the high half; k1 = which 16-column half
    const uint32_t w0 = __byte_perm(ma, mb, 0x5410);
    const uint32_t w1 = __byte_perm(ma, mb, 0x7632);
    if (p.meta_ref != nullptr) {
        uint32_t* e = p.meta_ref + row16 * half_k + (cb * 2 + (jj >> 1)) * 32 + m0 * 4 + 2 * (jj & 1);
        *reinterpret_cast<uint2*>(e) = make_uint2(w0, w1);
    }
    if (p.meta_tc != nullptr) {
        const int64_t tile = row16 >> 3;
        const int m2 = (int)(row16 & 7);
        uint32_t* rec = p.meta_tc + ((tile * p.col_blocks + cb) * 128 + m0 + 16 * m2) * 4 + jj;
        rec[0] = w0;       // lane L = m0 + 16*m2      (k1 = 0)
        rec[32] = w1;      // lane L = m0 + 8 + 16*m2  (k1 = 1)
    }
}

// ---------------------------------------------------------------- dense prune (prune_2_4)

template <int DT, int MODE, bool V128>
__global__ void __launch_bounds__(256) prune_dense_kernel(const uint16_t* A, uint16_t* out,   // out may alias A (in-place prune): no __restrict__
                                                          int64_t numel, int tie)
{
    const int64_t total = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i8 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i8 * 8 < numel; i8 += total) {
    const int64_t base = i8 * 8;
    uint32_t in[4] = {0, 0, 0, 0}, o[4];
    const bool full = base + 8 <= numel;  // otherwise exactly one group of 4 is left
    if (V128 && full) {
        uint4 v = *reinterpret_cast<const uint4*>(A + base);
        in[0] = v.x; in[1] = v.y; in[2] = v.z; in[3] = v.w;
    } else {
        uint2 v = *reinterpret_cast<const uint2*>(A + base);
        in[0] = v.x; in[1] = v.y;
        if (full) {
            uint2 w = *reinterpret_cast<const uint2*>(A + base + 4);
            in[2] = w.x; in[3] = w.y;
        }
    }
    prune_8<DT, MODE>(in[0], in[1], in[2], in[3], tie, o[0], o[1], o[2], o[3]);
    if (V128 && full) {
        *reinterpret_cast<uint4*>(out + base) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        *reinterpret_cast<uint2*>(out + base) = make_uint2(o[0], o[1]);
        if (full) *reinterpret_cast<uint2*>(out + base + 4) = make_uint2(o[2], o[3]);
    }
    }
}

// ---------------------------------------------------------------- metadata layouts

// index, in 16-bit units, of logical word (r, c) in each layout; ncols = K / 16
__host__ __device__ __forceinline__ int64_t meta_index(int layout, int64_t r, int64_t c, int64_t ncols)
{
    if (layout == S24_META_LOGICAL) return r * ncols + c;
    if (layout == S24_META_REF)  // compress_2_4.py:20-28
        return (r / 16) * (16 * ncols) + (c / 4) * 64 + (r % 8) * 8 + (c % 4) * 2 + (r / 8) % 2;
    const int64_t t = r / 128, m2 = (r % 128) / 16, hi = (r / 8) % 2, m0 = r % 8;
    const int64_t kb = c / 8, j = (c % 8) / 2, k1 = c % 2;
    const int64_t lane = m0 + 8 * k1 + 16 * m2;
    return 2 * (((t * ((ncols + 7) / 8) + kb) * 128 + lane) * 4 + j) + hi;   // ceil(K / 128) k-blocks per tile
}

__global__ void __launch_bounds__(256) meta_convert_kernel(const uint16_t* __restrict__ src, int from,
                                                           uint16_t* __restrict__ dst, int to, int64_t M,
                                                           int64_t ncols)
{
    // one thread per row pair (r, r+8) and column: both halves of a 32-bit word in REF and TC
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t pairs = (M / 2) * ncols;
    if (idx >= pairs) return;
    // enumerate in the order of the REF layout's words so that REF-side accesses coalesce
    const int64_t words_per_row16 = 8 * ncols;
    const int64_t row16 = idx / words_per_row16;
    const int64_t w = idx - row16 * words_per_row16;
    const int64_t c = (w / 32) * 4 + (w % 4);
    const int64_t m0 = (w / 4) % 8;
    const int64_t r = row16 * 16 + m0;
    const uint16_t lo = src[meta_index(from, r, c, ncols)];
    const uint16_t hi = src[meta_index(from, r + 8, c, ncols)];
    if (to == S24_META_LOGICAL) {
        dst[meta_index(to, r, c, ncols)] = lo;
        dst[meta_index(to, r + 8, c, ncols)] = hi;
    } else {
        *reinterpret_cast<uint32_t*>(dst + meta_index(to, r, c, ncols)) = (uint32_t)lo | ((uint32_t)hi << 16);
    }
}

// Reference layout <-> tensor-core layout, the conversion on the GEMM's path when the caller hands
// over the reference's E.  Both layouts pair row r (low half) with row r+8 (high half) in one 32-bit
// word, and the 64 words of a (16-row group, 128-column k-block) are contiguous in both: two
// adjacent 128-byte lines of E, and a 256-byte run of the k-block's 2 KB record.  Inside that run
//   E word   s = q*32 + m0*4 + cc          (q = which 64-column half, m0 = r % 8, cc = meta column % 4)
//   TC word  d = (cc%2)*32 + m0*4 + 2*q + cc/2
// so a warp moves one block with a coalesced 256-byte load, one exchange between neighbouring
// lanes and a coalesced 256-byte store (each lane 8 bytes both ways).
template <bool TO_TC>
__global__ void __launch_bounds__(256) meta_ref_tc_kernel(const uint2* __restrict__ src, uint2* __restrict__ dst,
                                                          int64_t row16s, int64_t kblocks)
{
    const int lane = threadIdx.x & 31;
    const int64_t blk = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= row16s * kblocks) return;
    const int64_t row16 = blk / kblocks, kb = blk - row16 * kblocks;
    // in units of uint2 (two words): a block is 32 of them in either layout
    const int64_t ref_off = (row16 * kblocks + kb) * 32;
    const int64_t tc_off = (((row16 >> 3) * kblocks + kb) * 8 + (row16 & 7)) * 32;
    const bool odd = lane & 1;
    if (TO_TC) {
        // lane l holds E words (2l, 2l+1): cc = 0,1 (even lane) or 2,3 (odd lane) of (q, m0) = (l/16, (l%16)/2)
        const uint2 v = src[ref_off + lane];
        const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, odd ? v.x : v.y, 1);
        // even lane: {cc=0, cc=2} -> k1 = 0; odd lane: {cc=1, cc=3} -> k1 = 1; TC word pair 2*q + {0,1}
        const uint2 o = odd ? make_uint2(other, v.y) : make_uint2(v.x, other);
        const int q = lane >> 4, m0 = (lane & 15) >> 1;
        dst[tc_off + (odd ? 16 : 0) + m0 * 2 + q] = o;
    } else {
        // the inverse: lane l holds TC words (2l, 2l+1) = (k1, m0, q) = (l/16, (l%16)/2, l%2), cc/2 = 0,1
        const uint2 v = src[tc_off + lane];
        const int k1 = lane >> 4, m0 = (lane & 15) >> 1, q = lane & 1;
        // E wants {cc = 2h, 2h+1} together: cc = 2*(cc/2) + k1, so lanes l and l^16 exchange
        const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, k1 ? v.x : v.y, 16);
        // k1 = 0 lane keeps cc/2 = 0: {cc=0 (own x), cc=1 (partner's x)}; k1 = 1 lane keeps cc/2 = 1: {cc=2 (partner's y), cc=3 (own y)}
        const uint2 o = k1 ? make_uint2(other, v.y) : make_uint2(v.x, other);
        dst[ref_off + q * 16 + m0 * 2 + k1] = o;
    }
}

// ---------------------------------------------------------------- compress, other element types

// compress_dense_to_sparse for the element types beyond fp16 / bf16 (compression/compress_2_4.py:41-47
// metadata type, :73-76 the 1:2 float branch, :144-154 eight codes per int32 word).  None of the
// reference's GEMM launchers consumes these, so this is a plain one-thread-per-metadata-word kernel:
// the thread reads the CODES groups of its word with 16-byte loads, applies the reference's flag
// logic (:113-121), stores the kept values and writes the word at its reordered place (:20-28).
//   T = int8_t : 2:4, 8 codes per int32 word (32 elements per thread)
//   T = int32_t: 2:4, 4 codes per int16 word (16 elements per thread)
//   T = float  : 1:2, a pair (e0, e1) counts as the group (e0, e0, e1, e1); 4 codes per int16 word
template <typename T, int KSPARSE, int CODES, typename META>
__global__ void __launch_bounds__(256) compress_other_kernel(const T* __restrict__ dense, int64_t ld, int64_t M, int64_t ncols,
                                                             T* __restrict__ vals, META* __restrict__ meta)
{
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * ncols) return;
    const int64_t r = idx / ncols, c = idx - r * ncols;
    constexpr int ELEMS = KSPARSE * CODES;          // elements of this thread's word
    constexpr int VEC = 16 / (int)sizeof(T);        // elements per 16-byte load
    __align__(16) T in[ELEMS];
    const T* src = dense + r * ld + c * ELEMS;
#pragma unroll
    for (int v = 0; v < ELEMS / VEC; ++v)
        *reinterpret_cast<uint4*>(in + v * VEC) = *reinterpret_cast<const uint4*>(src + v * VEC);
    __align__(16) T out[ELEMS / 2];
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < CODES; ++j) {
        const T* g = in + j * KSPARSE;
        bool m0, m1, m3;
        if (KSPARSE == 4) {
            m0 = g[0] != T(0); m1 = g[1] != T(0); m3 = g[3] != T(0);
        } else {
            m0 = m1 = g[0] != T(0);
            m3 = g[1] != T(0);
        }
        const bool expr0 = m0 && m1, expr1 = !m0 && m1, expr2 = !m0 && !m1;
        const int idx0 = (int)expr1 | ((int)expr2 << 1);
        const int idx1 = (int)(expr0 || expr2 || m3) | ((int)(expr1 || !m1) << 1);
        if (KSPARSE == 4) {
            out[2 * j] = g[idx0];
            out[2 * j + 1] = g[idx1];
        } else {
            out[j] = g[idx0 >> 1];
        }
        word |= (uint32_t)(idx0 | (idx1 << 2)) << (4 * j);
    }
    T* dst = vals + r * (ncols * (ELEMS / 2)) + c * (ELEMS / 2);
    constexpr int OUT_BYTES = (ELEMS / 2) * (int)sizeof(T);
    if (OUT_BYTES >= 16) {
#pragma unroll
        for (int v = 0; v < OUT_BYTES / 16; ++v) *reinterpret_cast<uint4*>(dst + v * VEC) = *reinterpret_cast<const uint4*>(out + v * VEC);
    } else {
#pragma unroll
        for (int v = 0; v < ELEMS / 2; ++v) dst[v] = out[v];
    }
    meta[meta_index(S24_META_REF, r, c, ncols)] = (META)word;
}

// ---------------------------------------------------------------- gathered shards -> row-major

// An all-gather of column shards arrives shard-major, (G, rows, nl); the caller wants (rows, G*nl).
// One 16-byte vector per thread, consecutive threads write consecutive output addresses and read
// whole 16-byte pieces of one shard row.
__global__ void __launch_bounds__(256) relayout_shards_kernel(const uint4* __restrict__ stage, uint4* __restrict__ out,
                                                              int64_t rows, int64_t shards, int64_t vec_per_shard_row,
                                                              int64_t out_row_vecs)
{
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_row = shards * vec_per_shard_row;
    if (idx >= rows * per_row) return;
    const int64_t r = idx / per_row;
    const int64_t c = idx - r * per_row;
    const int64_t g = c / vec_per_shard_row;
    const int64_t j = c - g * vec_per_shard_row;
    out[r * out_row_vecs + c] = stage[(g * rows + r) * vec_per_shard_row + j];
}

// ---------------------------------------------------------------- host launchers

static int launch_prune_compress(const void* A, int64_t M, int64_t K, int64_t ld, int dtype, int mode, int tie,
                                 void* vals, void* meta_ref, void* meta_tc, cudaStream_t stream)
{
    if (A == nullptr || vals == nullptr) return fail(S24_ERR_INVALID_ARG, "prune_compress: null A or vals");
    if (dtype != S24_FP16 && dtype != S24_BF16) return fail(S24_ERR_INVALID_ARG, "prune_compress: bad dtype %d", dtype);
    if (mode < 0 || mode > 2) return fail(S24_ERR_INVALID_ARG, "prune_compress: bad mode %d", mode);
    if (tie < 0 || tie > 2) return fail(S24_ERR_INVALID_ARG, "prune_compress: bad tie rule %d", tie);
    if (M < 0 || K < 0) return fail(S24_ERR_SHAPE, "prune_compress: negative shape");
    if (M % 32 != 0) return fail(S24_ERR_SHAPE, "Number of rows of dense matrix %lld must be divisible by 32", (long long)M);
    if (K % 64 != 0) return fail(S24_ERR_SHAPE, "Number of columns of dense matrix %lld must be divisible by 64", (long long)K);
    if (ld < K || ld % 8 != 0) return fail(S24_ERR_SHAPE, "prune_compress: row stride %lld must be >= K and a multiple of 8", (long long)ld);
    if (!aligned(A, 16) || !aligned(vals, 16) || !aligned(meta_ref, 16) || !aligned(meta_tc, 16))
        return fail(S24_ERR_INVALID_ARG, "prune_compress: pointers must be 16-byte aligned");
    if (M == 0 || K == 0) return S24_OK;
    if (meta_tc != nullptr && (M % 128 != 0 || K % 128 != 0)) {
        // tensor-core records are whole (128 x 128) units; the kernel writes only the words of rows
        // < M and columns < K, the rest get a valid code here (the values they index read as zero)
        int rc = check_cuda(cudaMemsetAsync(meta_tc, 0x44, s24_meta_tc_bytes(M, K), stream), "metadata prefill");
        if (rc) return rc;
    }

    PcParams p;
    p.A = static_cast<const uint16_t*>(A);
    p.lda = ld;
    p.M = M;
    p.K = K;
    p.vals = static_cast<uint16_t*>(vals);
    p.meta_ref = static_cast<uint32_t*>(meta_ref);
    p.meta_tc = static_cast<uint32_t*>(meta_tc);
    p.tie = tie;
    p.col_blocks = (K + 127) / 128;
    p.warp_tiles = (M / 16) * p.col_blocks;
    const int64_t blocks = (p.warp_tiles + 7) / 8;
    if (blocks > 0x7FFFFFFF) return fail(S24_ERR_SHAPE, "prune_compress: matrix too large for one launch");
    const bool ld256ok = aligned(A, 32) && aligned(vals, 32) && (ld % 16 == 0);
    dim3 grid((unsigned)blocks), block(256);
#define S24_LAUNCH_PC(DT, MODE)                                                              \
    do {                                                                                     \
        if (ld256ok) prune_compress_kernel<DT, MODE, true><<<grid, block, 0, stream>>>(p);   \
        else prune_compress_kernel<DT, MODE, false><<<grid, block, 0, stream>>>(p);          \
    } while (0)
#define S24_LAUNCH_PC_MODE(DT)                                        \
    do {                                                              \
        if (mode == kModeSigned) S24_LAUNCH_PC(DT, kModeSigned);      \
        else if (mode == kModeMagnitude) S24_LAUNCH_PC(DT, kModeMagnitude); \
        else S24_LAUNCH_PC(DT, kModeNone);                            \
    } while (0)
    if (dtype == S24_FP16) S24_LAUNCH_PC_MODE(kFp16);
    else S24_LAUNCH_PC_MODE(kBf16);
#undef S24_LAUNCH_PC_MODE
#undef S24_LAUNCH_PC
    return check_cuda(cudaGetLastError(), "prune_compress launch");
}

}  // namespace s24

using namespace s24;

extern "C" int s24_prune_compress(const void* A, int64_t M, int64_t K, int64_t ld, int dtype, int mode, int tie,
                                  void* vals, void* meta_ref, void* meta_tc, void* stream)
{
    if (mode != S24_MODE_SIGNED && mode != S24_MODE_MAGNITUDE)
        return fail(S24_ERR_INVALID_ARG, "prune_compress: bad mode %d", mode);
    return launch_prune_compress(A, M, K, ld, dtype, mode, tie, vals, meta_ref, meta_tc, static_cast<cudaStream_t>(stream));
}

extern "C" int s24_compress(const void* dense, int64_t M, int64_t K, int64_t ld, int dtype, void* vals,
                            void* meta_ref, void* meta_tc, void* stream)
{
    return launch_prune_compress(dense, M, K, ld, dtype, kModeNone, kTieLower, vals, meta_ref, meta_tc,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int s24_compress_other(const void* dense, int64_t M, int64_t K, int64_t ld, int elem_type, void* vals,
                                  void* meta_ref, void* stream)
{
    if (dense == nullptr || vals == nullptr || meta_ref == nullptr) return fail(S24_ERR_INVALID_ARG, "compress_other: null pointer");
    if (elem_type != S24_INT8 && elem_type != S24_INT32 && elem_type != S24_FP32)
        return fail(S24_ERR_INVALID_ARG, "compress_other: element type %d (S24_INT8, S24_INT32 or S24_FP32 expected)", elem_type);
    const int codes = elem_type == S24_INT8 ? 8 : 4;
    const int ksparse = elem_type == S24_FP32 ? 2 : 4;
    const int row_mult = elem_type == S24_INT8 ? 16 : 32;
    const int64_t esize = elem_type == S24_INT8 ? 1 : 4;
    if (M < 0 || K < 0) return fail(S24_ERR_SHAPE, "compress_other: negative shape");
    if (M % row_mult != 0) return fail(S24_ERR_SHAPE, "Number of rows of dense matrix %lld must be divisible by %d", (long long)M, row_mult);
    if (K % (4 * codes) != 0)
        return fail(S24_ERR_SHAPE, "Number of columns of dense matrix %lld must be divisible by %d", (long long)K, 4 * codes);
    const int64_t ncols = K / (ksparse * codes);
    if (ncols % 4 != 0)
        return fail(S24_ERR_SHAPE, "The number of metadata cols must be at least 4, current number: %lld", (long long)ncols);
    if (ld < K || (ld * esize) % 16 != 0) return fail(S24_ERR_SHAPE, "compress_other: row stride %lld must be >= K and a multiple of 16 bytes", (long long)ld);
    if (!aligned(dense, 16) || !aligned(vals, 16) || !aligned(meta_ref, 4))
        return fail(S24_ERR_INVALID_ARG, "compress_other: dense and vals must be 16-byte aligned");
    if (M == 0 || K == 0) return S24_OK;
    const int64_t words = M * ncols;
    const int64_t blocks = (words + 255) / 256;
    if (blocks > 0x7FFFFFFF) return fail(S24_ERR_SHAPE, "compress_other: matrix too large for one launch");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (elem_type == S24_INT8)
        compress_other_kernel<int8_t, 4, 8, int32_t><<<(unsigned)blocks, 256, 0, s>>>(
            static_cast<const int8_t*>(dense), ld, M, ncols, static_cast<int8_t*>(vals), static_cast<int32_t*>(meta_ref));
    else if (elem_type == S24_INT32)
        compress_other_kernel<int32_t, 4, 4, int16_t><<<(unsigned)blocks, 256, 0, s>>>(
            static_cast<const int32_t*>(dense), ld, M, ncols, static_cast<int32_t*>(vals), static_cast<int16_t*>(meta_ref));
    else
        compress_other_kernel<float, 2, 4, int16_t><<<(unsigned)blocks, 256, 0, s>>>(
            static_cast<const float*>(dense), ld, M, ncols, static_cast<float*>(vals), static_cast<int16_t*>(meta_ref));
    return check_cuda(cudaGetLastError(), "compress_other launch");
}

extern "C" int s24_prune(const void* A, void* out, int64_t numel, int dtype, int mode, int tie, void* stream)
{
    if (A == nullptr || out == nullptr) return fail(S24_ERR_INVALID_ARG, "prune: null pointer");
    if (dtype != S24_FP16 && dtype != S24_BF16) return fail(S24_ERR_INVALID_ARG, "prune: bad dtype %d", dtype);
    if (mode != S24_MODE_SIGNED && mode != S24_MODE_MAGNITUDE) return fail(S24_ERR_INVALID_ARG, "prune: bad mode %d", mode);
    if (tie < 0 || tie > 2) return fail(S24_ERR_INVALID_ARG, "prune: bad tie rule %d", tie);
    if (numel < 0 || numel % 4 != 0)
        return fail(S24_ERR_SHAPE, "The size of the last dimension must be divisible by 4.");
    if (!aligned(A, 8) || !aligned(out, 8)) return fail(S24_ERR_INVALID_ARG, "prune: pointers must be 8-byte aligned");
    if (numel == 0) return S24_OK;
    const int64_t threads = (numel + 7) / 8;
    const int64_t blocks = (threads + 255) / 256;
    if (blocks > 0x7FFFFFFF) return fail(S24_ERR_SHAPE, "prune: tensor too large for one launch");
    const bool v128 = aligned(A, 16) && aligned(out, 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint16_t* a = static_cast<const uint16_t*>(A);
    uint16_t* o = static_cast<uint16_t*>(out);
    // grid stride, about four vectors per thread, never fewer CTAs than the device holds at once
    int64_t nblocks = (blocks + 3) / 4;
    const int64_t resident = (int64_t)sm_count() * 8;
    if (nblocks < resident) nblocks = resident;
    if (nblocks > blocks) nblocks = blocks;
    dim3 grid((unsigned)nblocks), block(256);
#define S24_LAUNCH_PRUNE(DT, MODE)                                                          \
    do {                                                                                    \
        if (v128) prune_dense_kernel<DT, MODE, true><<<grid, block, 0, s>>>(a, o, numel, tie);  \
        else prune_dense_kernel<DT, MODE, false><<<grid, block, 0, s>>>(a, o, numel, tie);      \
    } while (0)
    if (dtype == S24_FP16) {
        if (mode == kModeMagnitude) S24_LAUNCH_PRUNE(kFp16, kModeMagnitude);
        else S24_LAUNCH_PRUNE(kFp16, kModeSigned);
    } else {
        if (mode == kModeMagnitude) S24_LAUNCH_PRUNE(kBf16, kModeMagnitude);
        else S24_LAUNCH_PRUNE(kBf16, kModeSigned);
    }
#undef S24_LAUNCH_PRUNE
    return check_cuda(cudaGetLastError(), "prune launch");
}

extern "C" size_t s24_meta_tc_bytes(int64_t M, int64_t K)
{
    if (M <= 0 || K <= 0) return 0;
    return (size_t)(((M + 127) / 128) * ((K + 127) / 128)) * 2048;   // one 2 KB record per (128-row tile, 128-column block)
}

extern "C" int s24_meta_convert(const void* src, int from_layout, void* dst, int to_layout, int64_t M, int64_t K,
                                void* stream)
{
    if (src == nullptr || dst == nullptr) return fail(S24_ERR_INVALID_ARG, "meta_convert: null pointer");
    if (from_layout < 0 || from_layout > 2 || to_layout < 0 || to_layout > 2)
        return fail(S24_ERR_INVALID_ARG, "meta_convert: bad layout");
    if (M < 0 || K < 0 || M % 32 != 0 || K % 64 != 0)
        return fail(S24_ERR_SHAPE, "meta_convert: needs M %% 32 == 0 and K %% 64 == 0 (got %lld x %lld)", (long long)M, (long long)K);
    if (!aligned(src, 4) || !aligned(dst, 4)) return fail(S24_ERR_INVALID_ARG, "meta_convert: pointers must be 4-byte aligned");
    if (M == 0 || K == 0) return S24_OK;
    if (to_layout == S24_META_TC && (M % 128 != 0 || K % 128 != 0)) {
        // words of partly covered records that lie outside the matrix: a valid code (see s24_prune_compress)
        int rc = check_cuda(cudaMemsetAsync(dst, 0x44, s24_meta_tc_bytes(M, K), static_cast<cudaStream_t>(stream)),
                            "metadata prefill");
        if (rc) return rc;
    }
    const int64_t ncols = K / 16;
    const int64_t pairs = (M / 2) * ncols;
    const int64_t blocks = (pairs + 255) / 256;
    if (blocks > 0x7FFFFFFF) return fail(S24_ERR_SHAPE, "meta_convert: matrix too large for one launch");
    const bool ref_tc = (from_layout == S24_META_REF && to_layout == S24_META_TC) ||
                        (from_layout == S24_META_TC && to_layout == S24_META_REF);
    if (ref_tc && K % 128 == 0 && aligned(src, 8) && aligned(dst, 8)) {   // whole k-blocks: two E lines per block
        // one warp per (16-row group, k-block): 64 words each
        const int64_t warps = (M / 16) * (K / 128);
        const unsigned grid = (unsigned)((warps + 7) / 8);
        if (to_layout == S24_META_TC)
            meta_ref_tc_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                static_cast<const uint2*>(src), static_cast<uint2*>(dst), M / 16, K / 128);
        else
            meta_ref_tc_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                static_cast<const uint2*>(src), static_cast<uint2*>(dst), M / 16, K / 128);
        return check_cuda(cudaGetLastError(), "meta_convert launch");
    }
    meta_convert_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(src), from_layout, static_cast<uint16_t*>(dst), to_layout, M, ncols);
    return check_cuda(cudaGetLastError(), "meta_convert launch");
}

extern "C" int s24_relayout_shards(const void* stage, void* out, int64_t rows, int64_t shards, int64_t shard_cols,
                                   int64_t ldo, void* stream)
{
    if (stage == nullptr || out == nullptr) return fail(S24_ERR_INVALID_ARG, "relayout_shards: null pointer");
    if (rows < 0 || shards <= 0 || shard_cols <= 0 || shard_cols % 8 != 0 || ldo % 8 != 0 || ldo < shards * shard_cols)
        return fail(S24_ERR_SHAPE, "relayout_shards: needs shard_cols %% 8 == 0, ldo %% 8 == 0 and ldo >= shards * shard_cols");
    if (!aligned(stage, 16) || !aligned(out, 16)) return fail(S24_ERR_INVALID_ARG, "relayout_shards: pointers must be 16-byte aligned");
    const int64_t vecs = rows * shards * (shard_cols / 8);
    if (vecs == 0) return S24_OK;
    const int64_t blocks = (vecs + 255) / 256;
    if (blocks > 0x7FFFFFFF) return fail(S24_ERR_SHAPE, "relayout_shards: too large for one launch");
    relayout_shards_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(stage), static_cast<uint4*>(out), rows, shards, shard_cols / 8, ldo / 8);
    return check_cuda(cudaGetLastError(), "relayout_shards launch");
}
