// spmm_prune_in.cu -- sparse GEMM that prunes and compresses its dense A operand on the fly:
//
//   C (M, N) = prune_2_4(A) (M, K) . B (K, N)
//
// The Blackwell counterpart of the reference's fused-input-prune experiment
// (compression/kernels/7.8.1_prune_ws.py: generate_compressed_and_meta :112-192, compute
// iteration :345-374, launcher :609-650).  On Hopper the prune sat between the shared-memory
// load and the wgmma of the same warps; here it runs in warps of its own, beside an MMA that
// is asynchronous and takes its metadata from tensor memory:
//
//   * warp 0: TMA producer for B only, a 4-stage ring of 64 k-rows x 2 x 120 columns per CTA;
//   * warps 6-21: prune warps.  Each owns 16 rows x 64 columns of this CTA's 128-row slab.  Per
//     k-block each lane reads 2 x 32 bytes of dense A straight from global memory (the next
//     k-block's loads are issued before the current one is ranked), ranks them with the same
//     packed half2 arithmetic as the standalone prune+compress kernel and stores
//       - the surviving values into the A operand stage (a 4-stage ring of its own) in the
//         128-byte-swizzled K-major form a TMA load of precompressed values would have produced,
//       - the metadata words into the 2 KB record that tcgen05.cp moves into tensor memory,
//     then fences the stores towards the asynchronous proxy and arrives on the leader CTA's
//     "A ready" barrier;
//   * warp 1: MMA issuer (leader CTA of the pair): waits for B (bytes) and A (prune warps of
//     both CTAs), copies the metadata record into tensor memory, issues four K = 32 sparse MMAs
//     per column sub-tile, commits to both CTAs' "A free" and "B empty" barriers;
//   * warps 2-5: epilogue, one warp per tensor-memory lane quadrant.
// A CTA pair computes a 256 x 480 tile as two 240-column sub-tiles that share every pruned A
// stage (accumulators and metadata fill 496 of the 512 tensor-memory columns); dense A never passes
// through shared memory.  Every k-block of A is ranked once per 480 columns of C, which is what
// bounds this variant at large N (the ranking keeps the ALU pipe busier than the MMAs keep the
// tensor pipe); at N <= 480 it reads and ranks A once and saves the round trip of the
// compressed operand through memory.
// All barrier waits are bounded (status codes 1-4 as in the plain kernel, 5 = prune warp waiting
// for a free stage, 6 = MMA warp waiting for pruned A).
#include "s24_common.cuh"
#include "sm100_ptx.cuh"
#include "prune_core.cuh"
#include "spmm_shared.cuh"

namespace s24 {

using namespace ptx;

namespace pin {
constexpr int kG = 2;
constexpr int kNT = 2;                            // column sub-tiles per tile, sharing each A stage
constexpr int kBNSub = 240;                       // one MMA's N (a multiple of 16)
constexpr int kBN = kNT * kBNSub;                 // tile columns
constexpr int kBNCta = kBNSub / kG;               // B columns per CTA and sub-tile
constexpr int kAStages = 4;                       // pruned A: stages of one k-block (128)
constexpr int kBStages = 4;                       // B: stages of half a k-block, so that four loads are in flight
constexpr int kBStageK = kBlockK / 2;
constexpr int kABytes = kRowsPerCta * 128;        // 128 rows x 64 kept values x 2 B
constexpr int kBAtomBytes = kBStageK * 128;       // 64 k-rows x 64 columns x 2 B
constexpr int kBAtoms = (kBNCta + 63) / 64;       // whole 64-column atoms per sub-tile (the last one partly used)
constexpr int kBSubBytes = kBAtoms * kBAtomBytes;
constexpr int kBBytes = kNT * kBSubBytes;
constexpr int kEBytes = 2048;
constexpr int kECol0 = kBN;                       // metadata columns follow the accumulators
constexpr int kEpiWarps = 4;
constexpr int kPruneWarps = 16;                   // 16 rows x 64 columns of the k-block each
constexpr int kFirstPruneWarp = 2 + kEpiWarps;
constexpr int kThreads = 32 * (2 + kEpiWarps + kPruneWarps);
constexpr int kSmemBytes = kAStages * (kABytes + kEBytes) + kBStages * kBBytes + 1024 + 256;
static_assert(kECol0 + 4 * kAStages <= (int)kTmemCols, "tensor memory budget");
static_assert(kSmemBytes <= 232448, "shared memory budget");
static_assert(kBN % 32 == 0 && kBNSub % 16 == 0, "the epilogue walks the two adjacent accumulators in 32-column chunks");
}  // namespace pin

struct PruneInParams {
    GemmParams g;
    const uint16_t* A;   // dense (M, K), row stride lda elements
    int64_t lda;
    int tie;
    int wide;            // 32-byte loads allowed (A and lda 32-byte aligned)
};

template <int DT, int MODE>
__global__ void __launch_bounds__(pin::kThreads, 1)
spmm_prune_in_kernel(const __grid_constant__ CUtensorMap tm_b, const PruneInParams pp)
{
    using namespace pin;
    constexpr int G = kG;
    const GemmParams& p = pp.g;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t smem_a = smem_base;
    const uint32_t smem_b = smem_a + kAStages * kABytes;
    const uint32_t smem_e = smem_b + kBStages * kBBytes;
    const uint32_t bars = smem_e + kAStages * kEBytes;
    const uint32_t bar_b_full = bars;                         // B bytes have landed (leader's barrier counts both CTAs)
    const uint32_t bar_b_empty = bar_b_full + 8 * kBStages;   // the MMAs that read the B stage have completed
    const uint32_t bar_a_ready = bar_b_empty + 8 * kBStages;  // every prune warp of both CTAs has filled the A stage
    const uint32_t bar_a_free = bar_a_ready + 8 * kAStages;   // the MMAs that read the A stage have completed
    const uint32_t bar_acc_full = bar_a_free + 8 * kAStages;
    const uint32_t bar_acc_empty = bar_acc_full + 8;
    const uint32_t tmem_slot = bar_acc_empty + 8;
    const uint32_t abort_addr = tmem_slot + 8;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_addr - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const bool leader = cta_rank == 0;

    constexpr int kTileRows = kRowsPerCta * G;
    const int num_m = (p.M + kTileRows - 1) / kTileRows;
    const int num_n = (p.N + kBN - 1) / kBN;
    const int num_tiles = num_m * num_n;
    const int num_units = (int)gridDim.x / G;
    const int unit = (int)blockIdx.x / G;
    const int kblocks = (p.K + kBlockK - 1) / kBlockK;   // a last block of 64 is padded with zeros

    if (threadIdx.x == 0) {
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(bar_b_full + 8 * s, 1);
            mbar_init(bar_b_empty + 8 * s, 1);
        }
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(bar_a_ready + 8 * s, kPruneWarps * G);
            mbar_init(bar_a_free + 8 * s, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, kEpiWarps * G);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tm_b);   // the descriptor fetch overlaps the rest of the set-up
    }
    if (warp == 1) {
        tmem_alloc<G>(tmem_slot, kTmemCols);
        tmem_relinquish<G>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (B only)
        if (elect_one()) {
            int s = 0;
            uint32_t phase = 0;
            for (int t = unit; t < num_tiles && !*abort_flag; t += num_units) {
                int tm, tn;
                tile_coords(t, num_m, num_n, tm, tn);
                const int nsub = (tn * kBN + kBNSub < p.N) ? kNT : 1;   // the last tile may have one sub-tile only
                for (int kh = 0; kh < 2 * kblocks; ++kh) {   // half k-blocks
                    if (!mbar_wait(bar_b_empty + 8 * s, phase ^ 1u)) {
                        report_timeout(p.status, abort_flag, 1);
                        break;
                    }
                    const uint32_t full = mapa(bar_b_full + 8 * s, 0);   // the leader's barrier
                    if (leader) mbar_arrive_expect_tx(bar_b_full + 8 * s, (uint32_t)(G * nsub * kBSubBytes));
                    for (int n = 0; n < nsub; ++n) {
                        const int col0 = tn * kBN + n * kBNSub + (int)cta_rank * kBNCta;
                        const uint32_t b_dst = smem_b + s * kBBytes + n * kBSubBytes;
#pragma unroll
                        for (int i = 0; i < kBAtoms; ++i)
                            tma_load_2d_pair(b_dst + i * kBAtomBytes, &tm_b, col0 + 64 * i, kh * kBStageK, full);
                    }
                    if (++s == kBStages) { s = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && elect_one()) {
            const uint32_t idesc = make_idesc_sp_f16(p.bf16, kTileRows, kBNSub, 1);
            int sa = 0, sb = 0;
            uint32_t pha = 0, phb = 0, acc_phase = 0;
            for (int t = unit; t < num_tiles && !*abort_flag; t += num_units) {
                int tm, tn;
                tile_coords(t, num_m, num_n, tm, tn);
                const int nsub = (tn * kBN + kBNSub < p.N) ? kNT : 1;
                if (!mbar_wait(bar_acc_empty, acc_phase ^ 1u)) {
                    report_timeout(p.status, abort_flag, 3);
                    break;
                }
                tc_fence_after();
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    if (!mbar_wait(bar_a_ready + 8 * sa, pha)) {
                        report_timeout(p.status, abort_flag, 6);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t e_cols = tmem_base + (uint32_t)(kECol0 + 4 * sa);
                    tc_cp_128x128b<G>(e_cols, make_smem_desc(smem_e + sa * kEBytes, 128, 128, kSwizzleNone));
                    const uint64_t adesc = make_smem_desc(smem_a + sa * kABytes, 16, 1024, kSwizzle128B);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (!mbar_wait(bar_b_full + 8 * sb, phb)) {
                            report_timeout(p.status, abort_flag, 2);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {
                            const int j = 2 * half + jj;   // K = 32 step within the k-block
                            for (int n = 0; n < nsub; ++n) {
                                // B: N-major, 128-byte swizzle; 64-column atoms kBAtomBytes apart, 8-k-row groups
                                // 1024 bytes apart, 32 k-rows (4096 bytes) per step
                                const uint64_t bdesc =
                                    make_smem_desc(smem_b + sb * kBBytes + n * kBSubBytes, kBAtomBytes, 1024, kSwizzle128B);
                                tc_mma_sp_f16<G>(tmem_base + (uint32_t)(n * kBNSub), adesc + (uint64_t)(j * 2),
                                                 bdesc + (uint64_t)(jj * 256), idesc | (uint32_t)(j & 1),
                                                 e_cols + (uint32_t)(j & 2), (kb | j) != 0 ? 1u : 0u);
                            }
                        }
                        tc_commit_pair(bar_b_empty + 8 * sb, 3);
                        if (++sb == kBStages) { sb = 0; phb ^= 1u; }
                    }
                    if (!ok) break;
                    tc_commit_pair(bar_a_free + 8 * sa, 3);
                    if (++sa == kAStages) { sa = 0; pha ^= 1u; }
                }
                if (!ok) break;
                tc_commit_pair(bar_acc_full, 3);
                acc_phase ^= 1u;
            }
        }
    } else if (warp < kFirstPruneWarp) {
        // ------------------------------------------------------------ epilogue warps
        const int quad = warp & 3;   // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
        uint32_t acc_phase = 0;
        const uint32_t acc_empty_leader = mapa(bar_acc_empty, 0);
        for (int t = unit; t < num_tiles && !*abort_flag; t += num_units) {
            int tm, tn;
            tile_coords(t, num_m, num_n, tm, tn);
            if (!mbar_wait(bar_acc_full, acc_phase)) {
                if (lane == 0) report_timeout(p.status, abort_flag, 4);
                break;
            }
            tc_fence_after();
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16);
            const int64_t row = (int64_t)tm * kTileRows + (int)cta_rank * kRowsPerCta + quad * 32 + lane;
            const int col0 = tn * kBN;
            uint16_t* crow = static_cast<uint16_t*>(p.C) + row * p.ldc + col0;
            const bool row_ok = row < p.M;
            const bool wide = ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.ldc * 2)) & 31u) == 0;
            const int nchunks = (min(kBN, p.N - col0) + 31) / 32;   // accumulator columns past N were never written
#pragma unroll 1
            for (int k = 0; k < nchunks; ++k) {
                uint32_t r[32];
                tc_ld_32x32b_x32(tacc + (uint32_t)(32 * k), r);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        q[j] = pack2(__uint_as_float(r[16 * i + 2 * j]), __uint_as_float(r[16 * i + 2 * j + 1]), p.bf16);
                    const int c = 32 * k + 16 * i;
                    if (!row_ok) continue;
                    if (wide && col0 + c + 16 <= p.N) {
                        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(crow + c), "r"(q[0]), "r"(q[1]),
                                     "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7])
                                     : "memory");
                    } else {
                        if (col0 + c < p.N) *reinterpret_cast<uint4*>(crow + c) = make_uint4(q[0], q[1], q[2], q[3]);
                        if (col0 + c + 8 < p.N) *reinterpret_cast<uint4*>(crow + c + 8) = make_uint4(q[4], q[5], q[6], q[7]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader);
            acc_phase ^= 1u;
        }
    } else {
        // ------------------------------------------------------------ prune warps
        const int pw = warp - kFirstPruneWarp;
        const int u = pw >> 1;                   // 16-row group of this CTA's slab
        const int h = pw & 1;                    // 64-column half of the k-block
        // rows 16u+m0 and 16u+m0+8, 16 columns each; eight consecutive lanes take eight different rows
        // so that their 16-byte stores into the swizzled stage fall into eight different chunks
        const int m0 = lane & 7, jq = lane >> 3;
        const uint32_t a_ready_leader = mapa(bar_a_ready, 0);
        // where this lane's 8 kept values per row go inside a stage: 8-row groups are 1024 bytes
        // apart, and the 128-byte swizzle XORs the 16-byte chunk index with row % 8
        const uint32_t a_off = (uint32_t)(2 * u) * 1024u + (uint32_t)m0 * 128u + (uint32_t)((4 * h + jq) ^ m0) * 16u;
        // its metadata word (row r in the low half, row r+8 in the high half) covers logical
        // metadata column 4h+jq of the k-block = 2j + k1: record lane m0 + 8*k1 + 16u, word j
        const uint32_t e_off = (uint32_t)((m0 + 8 * (jq & 1) + 16 * u) * 4 + 2 * h + (jq >> 1)) * 4u;

        uint32_t cur[2][8], nxt[2][8];
        auto fetch = [&](const uint16_t* ptr, bool valid, uint32_t (&d)[2][8]) {
            if (!valid) {
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) d[i][j] = 0u;
                return;
            }
            if (pp.wide) {
                ld256(ptr, d[0]);
                ld256(ptr + 8 * pp.lda, d[1]);
            } else {
                ld128x2(ptr, d[0]);
                ld128x2(ptr + 8 * pp.lda, d[1]);
            }
        };
        // address of this lane's first row at k-block 0 of tile t
        auto tile_ptr = [&](int t, bool& valid) -> const uint16_t* {
            int tm, tn;
            tile_coords(t, num_m, num_n, tm, tn);
            const int64_t row = (int64_t)tm * kTileRows + (int)cta_rank * kRowsPerCta + 16 * u + m0;
            valid = row + 8 < p.M;
            return pp.A + row * pp.lda + h * 64 + jq * 16;
        };

        int s = 0;
        uint32_t phase = 0;
        int t = unit, kb = 0;
        bool have = t < num_tiles, valid = false, nvalid = false;
        const uint16_t* ptr = nullptr;
        if (have) {
            ptr = tile_ptr(t, valid);
            fetch(ptr, valid && h * 64 < p.K, cur);
        }
        while (have && !*abort_flag) {
            // issue the next k-block's loads before working on this one
            int nt = t, nkb = kb + 1;
            const uint16_t* nptr = ptr + kBlockK;
            nvalid = valid;
            if (nkb == kblocks) {
                nkb = 0;
                nt = t + num_units;
                if (nt < num_tiles) nptr = tile_ptr(nt, nvalid);
            }
            const bool have_next = nt < num_tiles;
            if (have_next) fetch(nptr, nvalid && nkb * kBlockK + h * 64 < p.K, nxt);   // beyond K: zeros

            uint32_t va[4], vb[4];
            const uint32_t ca0 = prune_compress_8<DT, MODE>(cur[0][0], cur[0][1], cur[0][2], cur[0][3], pp.tie, va[0], va[1]);
            const uint32_t ca1 = prune_compress_8<DT, MODE>(cur[0][4], cur[0][5], cur[0][6], cur[0][7], pp.tie, va[2], va[3]);
            const uint32_t cb0 = prune_compress_8<DT, MODE>(cur[1][0], cur[1][1], cur[1][2], cur[1][3], pp.tie, vb[0], vb[1]);
            const uint32_t cb1 = prune_compress_8<DT, MODE>(cur[1][4], cur[1][5], cur[1][6], cur[1][7], pp.tie, vb[2], vb[3]);
            // the codes sit in the top byte of each result: 16 columns = one 16-bit word per row
            const uint32_t word = __byte_perm(__byte_perm(ca0, ca1, 0x0073), __byte_perm(cb0, cb1, 0x0073), 0x5410);

            if (!mbar_wait(bar_a_free + 8 * s, phase ^ 1u)) {
                if (lane == 0) report_timeout(p.status, abort_flag, 5);
                break;
            }
            const uint32_t a_dst = smem_a + s * kABytes + a_off;
            st_shared_v4(a_dst, va[0], va[1], va[2], va[3]);
            st_shared_v4(a_dst + 1024u, vb[0], vb[1], vb[2], vb[3]);
            st_shared_u32(smem_e + s * kEBytes + e_off, word);
            fence_proxy_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(a_ready_leader + 8 * s);
            if (++s == kAStages) { s = 0; phase ^= 1u; }

#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) cur[i][j] = nxt[i][j];
            t = nt;
            kb = nkb;
            ptr = nptr;
            valid = nvalid;
            have = have_next;
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<G>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------- host side

template <int DT, int MODE>
static int launch_prune_in(const CUtensorMap& tm_b, const PruneInParams& pp, cudaStream_t stream)
{
    {
        static bool opted_in[64] = {false};
        int dev = 0;
        int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
        if (rc) return rc;
        if (dev < 0 || dev >= 64 || !opted_in[dev]) {
            rc = check_cuda(cudaFuncSetAttribute(spmm_prune_in_kernel<DT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 pin::kSmemBytes),
                            "cudaFuncSetAttribute(max dynamic shared memory)");
            if (rc) return rc;
            if (dev >= 0 && dev < 64) opted_in[dev] = true;
        }
    }
    const int num_m = (pp.g.M + 255) / 256;
    const int num_n = (pp.g.N + pin::kBN - 1) / pin::kBN;   // 480-column tiles
    const int tiles = num_m * num_n;
    int units = sm_count() / pin::kG;
    if (units > tiles) units = tiles;
    if (units < 1) units = 1;

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(units * pin::kG));
    lc.blockDim = dim3(pin::kThreads);
    lc.dynamicSmemBytes = pin::kSmemBytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pin::kG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&lc, spmm_prune_in_kernel<DT, MODE>, tm_b, pp), "fused-input-prune GEMM launch");
}

}  // namespace s24

using namespace s24;

extern "C" int s24_spmm_prune_in(const void* A, int64_t lda, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                 int64_t ldb, int64_t ldc, int dtype, int mode, int tie, void* stream)
{
    const char* who = "spmm_prune_in";
    if (A == nullptr || B == nullptr || C == nullptr) return fail(S24_ERR_INVALID_ARG, "%s: null pointer", who);
    if (dtype != S24_FP16 && dtype != S24_BF16) return fail(S24_ERR_INVALID_ARG, "%s: bad dtype %d", who, dtype);
    if (mode != S24_MODE_SIGNED && mode != S24_MODE_MAGNITUDE) return fail(S24_ERR_INVALID_ARG, "%s: bad mode %d", who, mode);
    if (tie != S24_TIE_REFERENCE && tie != S24_TIE_LOWER && tie != S24_TIE_HIGHER)
        return fail(S24_ERR_INVALID_ARG, "%s: bad tie rule %d", who, tie);
    if (M <= 0 || N <= 0 || K <= 0 || M % 32 != 0 || K % 64 != 0 || N % 8 != 0)
        return fail(S24_ERR_SHAPE, "%s: needs M %% 32 == 0, K %% 64 == 0, N %% 8 == 0 (got M=%lld N=%lld K=%lld)", who,
                    (long long)M, (long long)N, (long long)K);
    if (M > 0x7FFFFF00ll || N > 0x7FFFFF00ll || K > 0x7FFFFF00ll) return fail(S24_ERR_SHAPE, "%s: dimension too large", who);
    if (lda < K || lda % 8 != 0 || ldb < N || ldb % 8 != 0 || ldc < N || ldc % 8 != 0)
        return fail(S24_ERR_SHAPE, "%s: lda >= K, ldb/ldc >= N, all multiples of 8 (got %lld, %lld, %lld)", who, (long long)lda,
                    (long long)ldb, (long long)ldc);
    if (!aligned(A, 16) || !aligned(B, 16) || !aligned(C, 16))
        return fail(S24_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", who);
    int* status = status_word_address();
    if (status == nullptr) return fail(S24_ERR_CUDA, "%s: cannot resolve the device status word", who);

    CUtensorMap tm_b;
    const CUtensorMapDataType dt = dtype == S24_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    int rc = make_map_2d(&tm_b, dt, 2, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, pin::kBStageK, CU_TENSOR_MAP_SWIZZLE_128B, "B");
    if (rc) return rc;

    PruneInParams pp;
    pp.g.C = C;
    pp.g.ldc = ldc;
    pp.g.M = (int)M;
    pp.g.N = (int)N;
    pp.g.K = (int)K;
    pp.g.bf16 = dtype == S24_BF16;
    pp.g.status = status;
    pp.g.c_vals = nullptr;
    pp.g.c_meta_ref = nullptr;
    pp.g.c_meta_tc = nullptr;
    pp.g.n_dst = 0;
    for (int d = 0; d < 8; ++d) pp.g.dst[d] = nullptr;
    pp.A = static_cast<const uint16_t*>(A);
    pp.lda = lda;
    pp.tie = tie;
    pp.wide = aligned(A, 32) && (lda % 16 == 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == S24_FP16) {
        if (mode == S24_MODE_SIGNED) return launch_prune_in<kFp16, kModeSigned>(tm_b, pp, s);
        return launch_prune_in<kFp16, kModeMagnitude>(tm_b, pp, s);
    }
    if (mode == S24_MODE_SIGNED) return launch_prune_in<kBf16, kModeSigned>(tm_b, pp, s);
    return launch_prune_in<kBf16, kModeMagnitude>(tm_b, pp, s);
}
