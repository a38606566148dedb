// spmm_tcgen05.cu -- 2:4 structured-sparse GEMM for B200 on tcgen05.mma.sp.
//
//   C (M, N) = A24 (M, K) . B (K, N),  16-bit inputs, fp32 accumulation in tensor memory.
//
// Replaces the reference's persistent warp-specialised Hopper kernel
// (compression/gluon_ws_sparse.py:105-278, launcher :560-613; tile walk
// compression/common.py:150-162) and, with the pruning epilogue, its fused-output variant
// (compression/kernels/10.1_prune_acc.py:88-154,203-248,359-398).
//
// Design (one CTA, or a CTA pair working as one tile engine):
//   * persistent grid: one CTA (pair) per SM (pair), tiles walked in groups of 8 M-tiles
//     swept along N so that B tiles stay in L2;
//   * warp 0: TMA producer.  Two shared-memory rings with barriers of their own: the A ring
//     holds units of one 128-row sub-tile x one k-block of 128 (A values: 128 rows x 64 values,
//     128-byte swizzle, plus the 2 KB metadata record), the B ring units of one k-block of this
//     CTA's part of B (128 rows x BN_CTA columns as 64-column swizzled atoms).  A k-block
//     consumes MT units of A and one of B; with separate rings a sub-tile's A unit goes back to
//     the producer as soon as its own MMAs are done;
//   * warp 1: MMA issuer (one elected lane).  Per k-block and sub-tile: tcgen05.cp moves the
//     metadata record into 4 TMEM columns, then four tcgen05.mma.sp (K = 32 each) accumulate
//     into TMEM; tcgen05.commit releases the A unit, after the last sub-tile the B unit and,
//     after the last k-block, publishes that sub-tile's accumulator;
//   * warps 2-9: epilogue, two warps per 32-lane TMEM quadrant (they split the tile's columns,
//     or take one row sub-tile each, which has accumulator barriers of its own).  One
//     accumulator row per thread: wide tcgen05.ld (128, then 64 + 32 columns per round trip),
//     round to 16 bits in registers, hand TMEM back to the MMA warp, then 32-byte stores (or,
//     in the pruning epilogue, rank the rounded values and store them compressed);
//   * CTA pairs (cta_group::2): each CTA loads its own 128 rows of A and half of the B
//     tile (no multicast), the leader CTA issues 256-row MMAs that read both CTAs' shared
//     memory, completion is multicast to both CTAs' barriers.  Only the leader's producer
//     arrives on the "full" barrier (with the byte count of both CTAs); the peer's copies
//     complete on that barrier without an arrive of their own;
//   * optionally (MT = 2) a pair owns two 256-row sub-tiles that share every B unit.
// Every barrier wait is bounded; on a timeout the kernel records a code in the status word
// (see s24_device_status), frees its tensor memory and returns.
#include "s24_common.cuh"
#include "sm100_ptx.cuh"
#include "spmm_shared.cuh"
#include "prune_core.cuh"

#include <cuda_fp16.h>
#include <cuda_bf16.h>

// Timing experiments only (never set in a shipped build: the results are wrong).  Bit 0: the
// plain epilogue hands tensor memory back without reading it; bit 1: no A / metadata loads;
// bit 2: no B loads.  They size what each part of the pipeline costs (see the profile notes).
#ifndef S24_TIMING_DIAG
#define S24_TIMING_DIAG 0
#endif

// ring depths of the 512 x 224 tile: 7 A units (3.5 k-blocks) and 3 B units fill the 227 KB
#ifndef S24_NA_224
#define S24_NA_224 7
#endif
#ifndef S24_NB_224
#define S24_NB_224 3
#endif
// ring depths of the 256 x 256 tile
#ifndef S24_NA_256
#define S24_NA_256 4
#endif
#ifndef S24_NB_256
#define S24_NB_256 4
#endif

namespace s24 {

using namespace ptx;

__device__ int g_status_word = 0;  // first device-side failure since the last s24_device_status()

constexpr int kThreads = 320;       // producer warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)

// G = CTAs per tile engine (1 or a pair), BN = tile columns, MT = 128-row sub-tiles per CTA:
// with MT = 2 a CTA pair owns 512 rows as two 256-row MMAs that share every B stage, which cuts
// the bytes brought into each SM per flop by a quarter and deepens the ring in MMA time.
// BT: B is given transposed, (N, K) row-major (activations stored (tokens, hidden)); its tiles are
// then K-major in shared memory like A's, loaded as two 64-wide K atoms per stage.
// SCATTER: the epilogue stores every C tile to several destinations (this GPU's and its peers'
// copies of a replicated result) through a shared-memory transpose that makes the stores whole lines.
template <int G, int BN, int NA, int NB, bool PRUNE_OUT = false, int MT = 1, bool BT = false, bool SCATTER = false>
struct GemmCfg {
    static constexpr bool kPruneOut = PRUNE_OUT;
    static constexpr bool kBT = BT;
    static constexpr bool kScatter = SCATTER;
    static constexpr int kScatterPitch = 272;                   // 256-byte row segments, padded against bank conflicts
    static constexpr int kScatterWarpBytes = 32 * kScatterPitch; // 32 rows x 128 columns x 2 B per epilogue warp
    static constexpr int kScatterBytes = SCATTER ? 8 * kScatterWarpBytes : 0;
    static constexpr int kG = G;
    static constexpr int kBN = BN;
    static constexpr int kMT = MT;
    static constexpr int kNA = NA;                              // A ring: units of (sub-tile, k-block)
    static constexpr int kNB = NB;                              // B ring: units of one k-block
    static constexpr int kTileRows = kRowsPerCta * G * MT;
    static constexpr int kBNCta = BN / G;                       // B columns this CTA feeds to the MMA
    static constexpr int kASubBytes = kRowsPerCta * 128;        // 128 rows x 64 values x 2 B
    static constexpr int kBAtomBytes = kBlockK * 128;           // 128 k-rows x 64 columns x 2 B
    static constexpr int kBAtoms = (kBNCta + 63) / 64;          // 64-column atoms, the last one possibly narrower
    static constexpr int kBBytes = kBAtoms * kBAtomBytes;      // shared-memory footprint of a B unit
    static constexpr int kBtAtomBytes = kBNCta * 128;           // transposed B: N rows x 64 k-values x 2 B
    // columns of the last atom that belong to this CTA: loaded with a narrower box of its own so
    // that no column outside the tile is fetched (0 = the last atom is whole)
    static constexpr int kBTailCols = kBNCta % 64;
    static constexpr int kBLoadBytes = BT ? 2 * kBtAtomBytes
                                          : (kBTailCols ? (kBAtoms - 1) * kBAtomBytes + kBlockK * kBTailCols * 2 : kBBytes);
    static constexpr int kESubBytes = 2048;
    static constexpr int kATxBytes = kASubBytes + kESubBytes;   // bytes one A unit's copies deliver
    static constexpr int kAccCols = BN * MT;                    // one accumulator set
    static constexpr int kAccStages = (kAccCols >= 256) ? 1 : 2;
    static constexpr int kAccBars = kAccStages * MT;            // each sub-tile's accumulator has barriers of its own
    static constexpr int kECol0 = kAccStages * kAccCols;        // metadata columns follow the accumulators
    static constexpr int kBarrierBytes = 8 * (2 * NA + 2 * NB + 2 * kAccBars) + 16;
    static constexpr int kSmemBytes = NA * (kASubBytes + kESubBytes) + NB * kBBytes + kScatterBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static_assert(!SCATTER || (MT == 1 && BN == 256 && !PRUNE_OUT), "the scatter epilogue is written for 128-column warp slices");
    static_assert(kECol0 + 4 * NA <= (int)kTmemCols, "tensor memory budget");
    static_assert(NA >= 2 * MT && NB >= 2, "at least two k-blocks in each ring");
    static_assert(kBarrierBytes <= 256, "barrier block");
    static_assert(kBNCta % 8 == 0 && BN % (16 * G) == 0, "MMA N granularity");
    static_assert(BN % 32 == 0 && (BN / (MT == 2 ? 1 : 2)) % 32 == 0, "the epilogues work in 32-column chunks");
    static_assert(kSmemBytes <= 232448, "shared memory budget (227 KB per CTA)");
};

template <class Cfg>
__global__ void __launch_bounds__(kThreads, 1)
spmm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_b_tail, const __grid_constant__ CUtensorMap tm_e, const GemmParams p)
{
    constexpr int G = Cfg::kG;
    constexpr int BN = Cfg::kBN;
    constexpr int NA = Cfg::kNA;
    constexpr int NB = Cfg::kNB;
    constexpr int ACC = Cfg::kAccStages;
    constexpr int MT = Cfg::kMT;
    constexpr int ACCB = Cfg::kAccBars;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t smem_a = smem_base;
    const uint32_t smem_b = smem_a + NA * Cfg::kASubBytes;
    const uint32_t smem_e = smem_b + NB * Cfg::kBBytes;
    const uint32_t smem_scatter = smem_e + NA * Cfg::kESubBytes;
    const uint32_t bars = smem_scatter + Cfg::kScatterBytes;
    // barrier block: a_full[NA], a_empty[NA], b_full[NB], b_empty[NB], acc_full[ACCB], acc_empty[ACCB], tmem slot, abort flag
    const uint32_t bar_a_full = bars;
    const uint32_t bar_a_empty = bar_a_full + 8 * NA;
    const uint32_t bar_b_full = bar_a_empty + 8 * NA;
    const uint32_t bar_b_empty = bar_b_full + 8 * NB;
    const uint32_t bar_acc_full = bar_b_empty + 8 * NB;
    const uint32_t bar_acc_empty = bar_acc_full + 8 * ACCB;
    const uint32_t tmem_slot = bar_acc_empty + 8 * ACCB;
    const uint32_t abort_addr = tmem_slot + 8;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem_base));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + (abort_addr - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (G == 2) ? cluster_ctarank() : 0u;
    const bool leader = cta_rank == 0;

    const int num_m = (p.M + Cfg::kTileRows - 1) / Cfg::kTileRows;
    const int num_n = (p.N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_units = (int)gridDim.x / G;
    const int unit = (int)blockIdx.x / G;
    const int kblocks = (p.K + kBlockK - 1) / kBlockK;   // a last block of 64 reads zeros beyond K

    if (threadIdx.x == 0) {
        for (int s = 0; s < NA; ++s) {
            mbar_init(bar_a_full + 8 * s, 1);   // one arrive (the leader's producer) + both CTAs' bytes
            mbar_init(bar_a_empty + 8 * s, 1);
        }
        for (int s = 0; s < NB; ++s) {
            mbar_init(bar_b_full + 8 * s, 1);
            mbar_init(bar_b_empty + 8 * s, 1);
        }
        for (int a = 0; a < ACCB; ++a) {
            mbar_init(bar_acc_full + 8 * a, 1);
            mbar_init(bar_acc_empty + 8 * a, (8 / MT) * G);   // the epilogue warps of every CTA that drain this sub-tile
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {   // descriptor fetches overlap the set-up below
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        if (Cfg::kBTailCols != 0 && !Cfg::kBT) prefetch_tensormap(&tm_b_tail);
        prefetch_tensormap(&tm_e);
    }
    if (warp == 1) {
        tmem_alloc<G>(tmem_slot, kTmemCols);
        tmem_relinquish<G>();
    }
    tc_fence_before();
    __syncthreads();
    if (G == 2) cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int sa = 0, sb = 0;
            uint32_t pha = 0, phb = 0;
            bool stopped = false;
            for (int t = unit; t < num_tiles && !stopped && !*abort_flag; t += num_units) {
                int tm, tn;
                tile_coords(t, num_m, num_n, tm, tn);
                // sub-tile m of this CTA: rows row0 + m * 128 * G .. + 127
                const int row0 = tm * Cfg::kTileRows + (int)cta_rank * kRowsPerCta;
                const int col0 = tn * BN + (int)cta_rank * Cfg::kBNCta;
                // The leader announces the bytes of both CTAs on its own barrier; the peer's copies
                // complete on the leader's barrier too (their bytes may run ahead of the
                // announcement, which the transaction count tolerates).
                auto load_a = [&](int kb, int m) -> bool {
                    if (!mbar_wait(bar_a_empty + 8 * sa, pha ^ 1u, p.wait_limit_ns)) return false;
                    const uint32_t full = (G == 2) ? mapa(bar_a_full + 8 * sa, 0) : (bar_a_full + 8 * sa);
                    if (leader) mbar_arrive_expect_tx(bar_a_full + 8 * sa, (S24_TIMING_DIAG & 2) ? 0u : (uint32_t)(G * Cfg::kATxBytes));
                    const int rows = row0 + m * kRowsPerCta * G;
                    const int rec = (rows / kRowsPerCta) * kblocks + kb;
                    if (S24_TIMING_DIAG & 2) {
                    } else if (G == 2) {
                        tma_load_2d_pair(smem_a + sa * Cfg::kASubBytes, &tm_a, kb * 64, rows, full);
                        tma_load_2d_pair(smem_e + sa * Cfg::kESubBytes, &tm_e, 0, rec * 4, full);
                    } else {
                        tma_load_2d(smem_a + sa * Cfg::kASubBytes, &tm_a, kb * 64, rows, full);
                        tma_load_2d(smem_e + sa * Cfg::kESubBytes, &tm_e, 0, rec * 4, full);
                    }
                    if (++sa == NA) { sa = 0; pha ^= 1u; }
                    return true;
                };
                auto load_b = [&](int kb) -> bool {
                    if (!mbar_wait(bar_b_empty + 8 * sb, phb ^ 1u, p.wait_limit_ns)) return false;
                    const uint32_t full = (G == 2) ? mapa(bar_b_full + 8 * sb, 0) : (bar_b_full + 8 * sb);
                    if (leader) mbar_arrive_expect_tx(bar_b_full + 8 * sb, (S24_TIMING_DIAG & 4) ? 0u : (uint32_t)(G * Cfg::kBLoadBytes));
                    const uint32_t b_dst = smem_b + sb * Cfg::kBBytes;
                    if constexpr ((S24_TIMING_DIAG & 4) != 0) {
                    } else if constexpr (Cfg::kBT) {
                        // transposed B: two boxes of (64 k-values x kBNCta rows of N)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (G == 2) tma_load_2d_pair(b_dst + h * Cfg::kBtAtomBytes, &tm_b, kb * kBlockK + 64 * h, col0, full);
                            else tma_load_2d(b_dst + h * Cfg::kBtAtomBytes, &tm_b, kb * kBlockK + 64 * h, col0, full);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < Cfg::kBAtoms; ++i) {
                            // the last atom of a tile whose width is not a multiple of 64 comes through
                            // the narrower box: same 128-byte swizzled rows, only the tile's own columns
                            const CUtensorMap* map = (Cfg::kBTailCols != 0 && i == Cfg::kBAtoms - 1) ? &tm_b_tail : &tm_b;
                            if (G == 2) tma_load_2d_pair(b_dst + i * Cfg::kBAtomBytes, map, col0 + 64 * i, kb * kBlockK, full);
                            else tma_load_2d(b_dst + i * Cfg::kBAtomBytes, map, col0 + 64 * i, kb * kBlockK, full);
                        }
                    }
                    if (++sb == NB) { sb = 0; phb ^= 1u; }
                    return true;
                };
                for (int kb = 0; kb < kblocks; ++kb) {
                    // self-test of the time-out path: stop feeding the rings; nothing is left in flight
                    if (p.selftest_stop_after_kblocks > 0 && kb >= p.selftest_stop_after_kblocks) {
                        stopped = true;
                        break;
                    }
                    // in the order the MMA warp needs them: first sub-tile's A, B, remaining sub-tiles' A
                    bool ok = load_a(kb, 0) && load_b(kb);
#pragma unroll
                    for (int m = 1; m < MT; ++m) ok = ok && load_a(kb, m);
                    if (!ok) {
                        report_timeout(p.status, abort_flag, 1);
                        stopped = true;
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && elect_one()) {
            const uint32_t idesc = make_idesc_sp_f16(p.bf16, kRowsPerCta * G, BN, Cfg::kBT ? 0 : 1);
            int sa = 0, sb = 0, a = 0;
            uint32_t pha = 0, phb = 0, acc_phase = 0;
            bool ok = true;
            for (int t = unit; t < num_tiles && ok && !*abort_flag; t += num_units) {
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    if (!mbar_wait(bar_b_full + 8 * sb, phb, p.wait_limit_ns)) {
                        report_timeout(p.status, abort_flag, 2);
                        ok = false;
                        break;
                    }
                    // B: N-major, 128-byte swizzle; 64-column atoms kBAtomBytes apart (leading),
                    // 8-k-row groups 1024 bytes apart (stride)
                    const uint64_t bdesc = make_smem_desc(smem_b + sb * Cfg::kBBytes, Cfg::kBAtomBytes, 1024, kSwizzle128B);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const int ab = a * MT + m;   // this sub-tile's accumulator
                        if (kb == 0) {
                            if (!mbar_wait(bar_acc_empty + 8 * ab, acc_phase ^ 1u, p.wait_limit_ns)) {
                                report_timeout(p.status, abort_flag, 3);
                                ok = false;
                                break;
                            }
                        }
                        if (!mbar_wait(bar_a_full + 8 * sa, pha, p.wait_limit_ns)) {
                            report_timeout(p.status, abort_flag, 2);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t tmem_d = tmem_base + (uint32_t)(a * Cfg::kAccCols + m * BN);
                        const uint32_t e_cols = tmem_base + (uint32_t)(Cfg::kECol0 + 4 * sa);
                        // metadata record: 128 rows of 16 bytes, 8-row core matrices 128 bytes apart
                        tc_cp_128x128b<G>(e_cols, make_smem_desc(smem_e + sa * Cfg::kESubBytes, 128, 128, kSwizzleNone));
                        // A: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
                        const uint64_t adesc = make_smem_desc(smem_a + sa * Cfg::kASubBytes, 16, 1024, kSwizzle128B);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // K = 32 per instruction: 32 bytes further along A's rows, 32 k-rows (4096 B) into B,
                            // metadata column j (even column address + selector bit).
                            // Transposed B is K-major like A: 64 bytes per K = 32 step inside a 128-byte row,
                            // the second pair of steps in the second 64-wide K atom.
                            const uint64_t bstep = Cfg::kBT
                                ? make_smem_desc(smem_b + sb * Cfg::kBBytes + (j >> 1) * Cfg::kBtAtomBytes + (j & 1) * 64, 16, 1024, kSwizzle128B)
                                : bdesc + (uint64_t)(j * 256);
                            tc_mma_sp_f16<G>(tmem_d, adesc + (uint64_t)(j * 2), bstep, idesc | (uint32_t)(j & 1),
                                             e_cols + (uint32_t)(j & 2), (kb | j) != 0 ? 1u : 0u);
                        }
                        // the A unit goes back to the producer once these MMAs have read it
                        if (G == 2) tc_commit_pair(bar_a_empty + 8 * sa, 3);
                        else tc_commit<1>(bar_a_empty + 8 * sa);
                        if (++sa == NA) { sa = 0; pha ^= 1u; }
                        if (kb == kblocks - 1) {   // this sub-tile's accumulator is complete
                            if (G == 2) tc_commit_pair(bar_acc_full + 8 * ab, 3);
                            else tc_commit<1>(bar_acc_full + 8 * ab);
                        }
                    }
                    if (!ok) break;
                    if (G == 2) tc_commit_pair(bar_b_empty + 8 * sb, 3);
                    else tc_commit<1>(bar_b_empty + 8 * sb);
                    if (++sb == NB) { sb = 0; phb ^= 1u; }
                }
                if (++a == ACC) { a = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int quad = warp & 3;         // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
        const int half = (warp - 2) >> 2;  // second epilogue warp of the quadrant
        // MT == 1: the two warps of a quadrant split the tile's columns; MT == 2: each takes one sub-tile
        constexpr int CW = (MT == 2) ? BN : BN / 2;   // columns per epilogue warp
        const int sub = (MT == 2) ? half : 0;
        const int chalf = (MT == 2) ? 0 : half;
        int a = 0;
        uint32_t acc_phase = 0;
        // each sub-tile's accumulator has its own full / empty pair: this warp's is number a * MT + sub
        const uint32_t acc_empty_leader = ((G == 2) ? mapa(bar_acc_empty, 0) : bar_acc_empty) + 8 * (uint32_t)sub;
        for (int t = unit; t < num_tiles && !*abort_flag; t += num_units) {
            int tm, tn;
            tile_coords(t, num_m, num_n, tm, tn);
            if (!mbar_wait(bar_acc_full + 8 * (a * MT + sub), acc_phase, p.wait_limit_ns)) {
                if (lane == 0) report_timeout(p.status, abort_flag, 4);
                break;
            }
            tc_fence_after();
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * Cfg::kAccCols + sub * BN + chalf * CW);
            const int64_t row = (int64_t)tm * Cfg::kTileRows + (sub * G + (int)cta_rank) * kRowsPerCta + quad * 32 + lane;
            const int col0 = tn * BN + chalf * CW;
            if constexpr (Cfg::kScatter) {
                // One load round trip for this warp's 32 rows x 128 columns, TMEM handed back at once.
                // Each thread then parks its row segment (256 bytes) in a private slice of shared
                // memory and hands it to the bulk-copy engine once per destination: the stores leave
                // the SM as whole 256-byte bursts -- what a peer GPU's memory wants to see across
                // NVLink -- and the warp does not wait for them until it needs the slice again.
                uint32_t r[128];
                tc_ld_32x32b_x128(tacc, r);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * (a * MT));
                const uint32_t stg = smem_scatter + (uint32_t)(warp - 2) * (uint32_t)Cfg::kScatterWarpBytes +
                                     (uint32_t)lane * (uint32_t)Cfg::kScatterPitch;
                bulk_wait_read();   // the previous tile's copies have read this slice
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    st_shared_v4(stg + (uint32_t)(c * 16),
                                 pack2(__uint_as_float(r[8 * c]), __uint_as_float(r[8 * c + 1]), p.bf16),
                                 pack2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]), p.bf16),
                                 pack2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]), p.bf16),
                                 pack2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]), p.bf16));
                fence_proxy_async_shared();
                const int ncols = min(CW, p.N - col0);   // N % 8 == 0: a whole number of 16-byte pieces
                if (row < p.M && ncols > 0) {
                    const int64_t off = row * p.ldc + col0;
                    for (int d = 0; d < p.n_dst; ++d)
                        bulk_store(static_cast<uint16_t*>(p.dst[d]) + off, stg, (uint32_t)(ncols * 2));
                }
                bulk_commit();
            } else {
                // Drain in as few round trips as possible: one tcgen05.ld per 128 (then 64 + 32)
                // columns, round to 16 bits in registers, hand tensor memory back to the MMA warp and
                // only then issue the stores (32 bytes per thread to rows that lie ldc apart, which
                // the load/store unit takes a sector at a time): the next tile's main loop starts
                // while this tile is still on its way to memory.  The pruning epilogue does the same
                // and ranks the rounded values after the release.
                uint16_t* crow = Cfg::kPruneOut ? nullptr : static_cast<uint16_t*>(p.C) + row * p.ldc + col0;
                const bool row_ok = row < p.M;
                // 16 columns = 32 bytes = one full L2 sector per store when C allows it
                const bool wide = ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.ldc * 2)) & 31u) == 0;
                auto store16 = [&](const uint32_t* q, int c) {   // 16 columns starting at tile column c
                    if (!row_ok) return;
                    if (wide && col0 + c + 16 <= p.N) {
                        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(crow + c), "r"(q[0]), "r"(q[1]),
                                     "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7])
                                     : "memory");
                    } else {
                        if (col0 + c < p.N) *reinterpret_cast<uint4*>(crow + c) = make_uint4(q[0], q[1], q[2], q[3]);
                        if (col0 + c + 8 < p.N) *reinterpret_cast<uint4*>(crow + c + 8) = make_uint4(q[4], q[5], q[6], q[7]);
                    }
                };
                static_assert(CW % 32 == 0, "epilogue works in 32-column pieces");
                uint32_t q[CW / 2];
                auto pack = [&](const uint32_t* r, int c_off, int width) {
#pragma unroll
                    for (int j = 0; j < width / 2; ++j)
                        q[c_off / 2 + j] = pack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), p.bf16);
                };
                if constexpr ((S24_TIMING_DIAG & 1) != 0) {   // timing experiment: nothing is read
#pragma unroll
                    for (int j = 0; j < CW / 2; ++j) q[j] = 0u;
                } else {
                    int done = 0;
#pragma unroll
                    for (int k = 0; k < CW / 128; ++k) {
                        uint32_t r[128];
                        tc_ld_32x32b_x128(tacc + (uint32_t)done, r);
                        tc_wait_ld();
                        pack(r, done, 128);
                        done += 128;
                    }
                    if constexpr ((CW % 128) == 96) {
                        uint32_t r[64], r2[32];
                        tc_ld_32x32b_x64(tacc + (uint32_t)done, r);
                        tc_ld_32x32b_x32(tacc + (uint32_t)(done + 64), r2);
                        tc_wait_ld();
                        pack(r, done, 64);
                        pack(r2, done + 64, 32);
                    } else if constexpr ((CW % 128) == 64) {
                        uint32_t r[64];
                        tc_ld_32x32b_x64(tacc + (uint32_t)done, r);
                        tc_wait_ld();
                        pack(r, done, 64);
                    } else if constexpr ((CW % 128) == 32) {
                        uint32_t r[32];
                        tc_ld_32x32b_x32(tacc + (uint32_t)done, r);
                        tc_wait_ld();
                        pack(r, done, 32);
                    }
                }
                // every accumulator column of this warp has been read: hand TMEM back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * (a * MT));
                if constexpr (!Cfg::kPruneOut) {
#pragma unroll
                    for (int i = 0; i < CW / 16; ++i) store16(q + 8 * i, 16 * i);
                } else {
                    // Fused output prune (compression/kernels/10.1_prune_acc.py:88-154): per 32 columns keep 16
                    // values and 32 metadata bits.  The groups are ranked on the accumulators as rounded to
                    // the output type, with the packed 16-bit SIMD arithmetic of the stand-alone
                    // prune+compress kernel (signed keys, the lower index survives a tie, codes from the
                    // keep mask): the result is exactly compress(prune(C)) of the C the plain kernel
                    // would have stored, and differs from a ranking of the unrounded fp32 sums only where
                    // the second and third largest of a group round to the same 16-bit value.
                    constexpr int NCH = CW / 32;     // 32-column chunks of this warp
                    constexpr int NPAIR = NCH / 2;   // pairs of chunks
                    uint32_t vals[CW / 4];           // packed 16-bit pairs: 8 registers per chunk
                    uint32_t meta[NCH];              // codes of 8 groups, group g in bits 4g..4g+3
#pragma unroll
                    for (int c = 0; c < NCH; ++c) {
                        uint32_t code[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {   // 8 columns = two groups at a time
                            const uint32_t* in = q + 16 * c + 4 * i;
                            code[i] = p.bf16 ? prune_compress_8_from_mask<kBf16>(in[0], in[1], in[2], in[3], vals[c * 8 + 2 * i], vals[c * 8 + 2 * i + 1])
                                             : prune_compress_8_from_mask<kFp16>(in[0], in[1], in[2], in[3], vals[c * 8 + 2 * i], vals[c * 8 + 2 * i + 1]);
                        }
                        meta[c] = gather_code_bytes(code[0], code[1], code[2], code[3]);
                    }

                    if (row_ok) {
                        uint16_t* vrow = static_cast<uint16_t*>(p.c_vals) + row * (int64_t)(p.N / 2) + col0 / 2;
                        // rows of C_vals are N bytes long (N % 128 == 0) and chunks 32 bytes: aligned if the base is
                        const bool wide_vals = (reinterpret_cast<uintptr_t>(p.c_vals) & 31u) == 0;
#pragma unroll
                        for (int c = 0; c < NCH; ++c) {
                            if (col0 + c * 32 < p.N) {
                                if (wide_vals) {   // 16 values = 32 bytes = one whole sector per store
                                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(vrow + c * 16),
                                                 "r"(vals[c * 8]), "r"(vals[c * 8 + 1]), "r"(vals[c * 8 + 2]), "r"(vals[c * 8 + 3]),
                                                 "r"(vals[c * 8 + 4]), "r"(vals[c * 8 + 5]), "r"(vals[c * 8 + 6]), "r"(vals[c * 8 + 7])
                                                 : "memory");
                                } else {
                                    *reinterpret_cast<uint4*>(vrow + c * 16) =
                                        make_uint4(vals[c * 8], vals[c * 8 + 1], vals[c * 8 + 2], vals[c * 8 + 3]);
                                    *reinterpret_cast<uint4*>(vrow + c * 16 + 8) =
                                        make_uint4(vals[c * 8 + 4], vals[c * 8 + 5], vals[c * 8 + 6], vals[c * 8 + 7]);
                                }
                            }
                        }
                    }
                    // Metadata words pair row r (low half) with row r+8 (high half): lanes l and l^8 of this
                    // warp.  A 32-column chunk gives two words (16 columns each).  Chunks are handled in
                    // pairs: the lane with bit 3 clear assembles the two words of the first chunk, its
                    // partner those of the second, so each writes 8 adjacent bytes; an odd last chunk is
                    // written by the lower lanes alone.
                    const bool upper = (lane & 8) != 0;
                    const int m0 = lane & 7;
                    const int64_t row16 = row >> 4;
                    auto write_words = [&](uint32_t w0, uint32_t w1, int ncol) {   // ncol: first column of w0
                        if (!row_ok || ncol >= p.N) return;
                        const int cidx = ncol >> 4;                                  // logical metadata column of w0
                        if (p.c_meta_ref != nullptr) {
                            uint32_t* e = p.c_meta_ref + row16 * (int64_t)(p.N / 2) + (cidx >> 2) * 32 + m0 * 4 + (cidx & 3);
                            *reinterpret_cast<uint2*>(e) = make_uint2(w0, w1);
                        }
                        if (p.c_meta_tc != nullptr) {
                            const int64_t t128 = row >> 7;
                            const int m2 = (int)((row >> 4) & 7);
                            const int kb = cidx >> 3, j = (cidx & 7) >> 1;
                            uint32_t* rec = p.c_meta_tc + ((t128 * (int64_t)((p.N + 127) >> 7) + kb) * 128 + m0 + 16 * m2) * 4 + j;
                            rec[0] = w0;
                            rec[32] = w1;
                        }
                    };
#pragma unroll
                    for (int c2 = 0; c2 < NPAIR; ++c2) {
                        const uint32_t xa = __shfl_xor_sync(0xFFFFFFFFu, meta[2 * c2], 8);
                        const uint32_t xb = __shfl_xor_sync(0xFFFFFFFFu, meta[2 * c2 + 1], 8);
                        if (!upper) write_words(__byte_perm(meta[2 * c2], xa, 0x5410), __byte_perm(meta[2 * c2], xa, 0x7632), col0 + c2 * 64);
                        else write_words(__byte_perm(xb, meta[2 * c2 + 1], 0x5410), __byte_perm(xb, meta[2 * c2 + 1], 0x7632), col0 + c2 * 64 + 32);
                    }
                    if constexpr (NCH % 2 == 1) {
                        const uint32_t xa = __shfl_xor_sync(0xFFFFFFFFu, meta[NCH - 1], 8);
                        if (!upper) write_words(__byte_perm(meta[NCH - 1], xa, 0x5410), __byte_perm(meta[NCH - 1], xa, 0x7632), col0 + (NCH - 1) * 32);
                    }
                }
            }
            if (++a == ACC) { a = 0; acc_phase ^= 1u; }
        }
    }

    // ------------------------------------------------------------ teardown
    if constexpr (Cfg::kScatter) bulk_wait_all();   // every thread's own bulk stores have been performed
    tc_fence_before();
    __syncthreads();
    if (G == 2) cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<G>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

int make_map_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t inner,
                       uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                       CUtensorMapSwizzle swz, const char* what)
{
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return fail(S24_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    CUresult r = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(S24_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return S24_OK;
}

struct GemmArgs {
    bool bt;   // B given transposed: (N, K) row-major, ldb = its row stride
    const void* vals;
    const void* meta_tc;
    const void* B;
    int64_t M, N, K, ldb;
    int dtype;
    GemmParams p;
};

template <class Cfg>
static int launch_cfg(const GemmArgs& g, cudaStream_t stream)
{
    CUtensorMap tm_a, tm_b, tm_b_tail, tm_e;
    const CUtensorMapDataType dt = g.dtype == S24_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    int rc = make_map_2d(&tm_a, dt, 2, g.vals, (uint64_t)(g.K / 2), (uint64_t)g.M, (uint64_t)g.K, 64, kRowsPerCta,
                         CU_TENSOR_MAP_SWIZZLE_128B, "A values");
    if (rc) return rc;
    if (Cfg::kBT)
        rc = make_map_2d(&tm_b, dt, 2, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb * 2, 64, Cfg::kBNCta,
                         CU_TENSOR_MAP_SWIZZLE_128B, "B (transposed)");
    else
        rc = make_map_2d(&tm_b, dt, 2, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb * 2, 64, kBlockK,
                         CU_TENSOR_MAP_SWIZZLE_128B, "B");
    if (rc) return rc;
    tm_b_tail = tm_b;
    if (!Cfg::kBT && Cfg::kBTailCols != 0) {
        rc = make_map_2d(&tm_b_tail, dt, 2, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb * 2, Cfg::kBTailCols, kBlockK,
                         CU_TENSOR_MAP_SWIZZLE_128B, "B (last atom)");
        if (rc) return rc;
    }
    const uint64_t records = (uint64_t)((g.M + 127) / 128) * (uint64_t)((g.K + 127) / 128);
    rc = make_map_2d(&tm_e, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, g.meta_tc, 128, records * 4, 512, 128, 4,
                     CU_TENSOR_MAP_SWIZZLE_NONE, "metadata");
    if (rc) return rc;

    {
        // opt in to the large dynamic shared-memory size once per device and kernel variant
        static bool opted_in[64] = {false};
        int dev = 0;
        rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
        if (rc) return rc;
        if (dev < 0 || dev >= 64 || !opted_in[dev]) {
            rc = check_cuda(cudaFuncSetAttribute(spmm_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                            "cudaFuncSetAttribute(max dynamic shared memory)");
            if (rc) return rc;
            if (dev >= 0 && dev < 64) opted_in[dev] = true;
        }
    }
    const int num_m = (int)((g.M + Cfg::kTileRows - 1) / Cfg::kTileRows);
    const int num_n = (int)((g.N + Cfg::kBN - 1) / Cfg::kBN);
    const int tiles = num_m * num_n;
    int units = sm_count() / Cfg::kG;
    if (units > tiles) units = tiles;
    if (units < 1) units = 1;

    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(units * Cfg::kG));
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = Cfg::kSmemBytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = Cfg::kG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&lc, spmm_kernel<Cfg>, tm_a, tm_b, tm_b_tail, tm_e, g.p), "sparse GEMM launch");
}

int* status_word_address()
{
    // device address of g_status_word for the current device (looked up once per device)
    static int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_status_word) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int*>(ptr);
    }
    return cached[dev];
}

static int run_spmm(const void* vals, const void* meta_tc, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                    int64_t ldb, int64_t ldc, int dtype, const s24_tile_cfg* cfg, cudaStream_t stream,
                    bool prune_out = false, void* c_vals = nullptr, void* c_meta_ref = nullptr, void* c_meta_tc = nullptr,
                    bool bt = false, void* const* dsts = nullptr, int n_dst = 0, unsigned long long wait_limit_ns = kWaitTimeoutNs,
                    int selftest_stop_after_kblocks = 0)
{
    const char* who = prune_out ? "spmm_prune_out" : (bt ? "spmm_bt" : (dsts ? "spmm_scatter" : "spmm"));
    if (dsts != nullptr) {
        if (prune_out || bt) return fail(S24_ERR_UNSUPPORTED, "%s: plain row-major product only", who);
        if (n_dst < 1 || n_dst > 8) return fail(S24_ERR_INVALID_ARG, "%s: 1 to 8 destinations (got %d)", who, n_dst);
        for (int d = 0; d < n_dst; ++d)
            if (dsts[d] == nullptr || !aligned(dsts[d], 16))
                return fail(S24_ERR_INVALID_ARG, "%s: destination %d is null or not 16-byte aligned", who, d);
        C = dsts[0];
    }
    if (bt && prune_out) return fail(S24_ERR_UNSUPPORTED, "spmm_prune_out: transposed B is not supported");
    if (vals == nullptr || meta_tc == nullptr || B == nullptr || (!prune_out && C == nullptr) || (prune_out && c_vals == nullptr))
        return fail(S24_ERR_INVALID_ARG, "%s: null pointer", who);
    if (dtype != S24_FP16 && dtype != S24_BF16) return fail(S24_ERR_INVALID_ARG, "%s: bad dtype %d", who, dtype);
    // the shapes compress_dense_to_sparse accepts (compress_2_4.py:49-65): tiles of 128 rows and
    // k-blocks of 128 that are only partly covered read zeros (TMA out-of-range fill) for the rest
    if (M <= 0 || N <= 0 || K <= 0 || M % 32 != 0 || K % 64 != 0 || N % 8 != 0)
        return fail(S24_ERR_SHAPE, "%s: needs M %% 32 == 0, K %% 64 == 0, N %% 8 == 0 (got M=%lld N=%lld K=%lld)", who,
                    (long long)M, (long long)N, (long long)K);
    if (prune_out && N % 128 != 0)
        return fail(S24_ERR_SHAPE, "%s: needs N %% 128 == 0 (got N=%lld)", who, (long long)N);
    if (M > 0x7FFFFF00ll || N > 0x7FFFFF00ll || K > 0x7FFFFF00ll) return fail(S24_ERR_SHAPE, "%s: dimension too large", who);
    if (ldb < (bt ? K : N) || ldb % 8 != 0 || (!prune_out && (ldc < N || ldc % 8 != 0)))
        return fail(S24_ERR_SHAPE, "%s: ldb/ldc must be >= N and multiples of 8 (got %lld, %lld)", who, (long long)ldb, (long long)ldc);
    if (!aligned(vals, 16) || !aligned(meta_tc, 16) || !aligned(B, 16) || !aligned(C, 16) || !aligned(c_vals, 16) ||
        !aligned(c_meta_ref, 16) || !aligned(c_meta_tc, 16))
        return fail(S24_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", who);
    int* status = status_word_address();
    if (status == nullptr) return fail(S24_ERR_CUDA, "%s: cannot resolve the device status word", who);

    GemmArgs g;
    g.vals = vals;
    g.meta_tc = meta_tc;
    g.B = B;
    g.M = M;
    g.N = N;
    g.K = K;
    g.ldb = ldb;
    g.bt = bt;
    g.dtype = dtype;
    g.p.C = C;
    g.p.ldc = ldc;
    g.p.M = (int)M;
    g.p.N = (int)N;
    g.p.K = (int)K;
    g.p.bf16 = dtype == S24_BF16;
    g.p.status = status;
    g.p.c_vals = c_vals;
    g.p.c_meta_ref = static_cast<uint32_t*>(c_meta_ref);
    g.p.c_meta_tc = static_cast<uint32_t*>(c_meta_tc);
    g.p.wait_limit_ns = wait_limit_ns;
    g.p.selftest_stop_after_kblocks = selftest_stop_after_kblocks;
    g.p.n_dst = dsts ? n_dst : 0;
    for (int d = 0; d < 8; ++d) g.p.dst[d] = (dsts && d < n_dst) ? dsts[d] : nullptr;
    if (dsts != nullptr) return launch_cfg<GemmCfg<2, 256, 3, 3, false, 1, false, true>>(g, stream);
    if (prune_out && c_meta_tc != nullptr && M % 128 != 0) {
        // the last 128-row record group is only partly written by the epilogue: give the rest a valid code
        int rc = check_cuda(cudaMemsetAsync(c_meta_tc, 0x44, s24_meta_tc_bytes(M, N), stream), "output metadata prefill");
        if (rc) return rc;
    }

    int bm = cfg ? cfg->bm : 0, bn = cfg ? cfg->bn : 0;
    // Heuristic when the caller names no tile: score = (useful fraction of the persistent waves)
    // x (relative throughput of the tile shape measured at large sizes on B200).  The 512x224
    // tile moves a quarter fewer bytes into each SM per flop and is the most energy-efficient
    // variant, which is what counts once the part is power capped; the smaller tiles win only
    // when they fill the last wave better.
    if (bm == 0 && bn == 0) {
        struct Cand { int bm, bn, g; double eff; bool plain_only; };
        const Cand cands[4] = {{512, 224, 2, 1.00, false}, {256, 256, 2, 0.97, false}, {256, 128, 2, 0.78, false},
                               {128, 128, 1, 0.55, false}};
        double best = -1.0;
        for (const Cand& c : cands) {
            if (c.plain_only && prune_out) continue;
            if (c.bn > N + 127) continue;
            const double useful = ((double)M / c.bm) * ((double)N / c.bn);
            const int64_t tiles = ((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
            const int64_t units = sm_count() / c.g;
            const int64_t waves = (tiles + units - 1) / units;
            const double slots = (double)waves * (double)(tiles < units ? tiles : units);
            const double score = useful / slots * c.eff;
            if (score > best) { best = score; bm = c.bm; bn = c.bn; }
        }
    }
    if (bm == 0) bm = (M % 256 == 0 || M > 1024) ? 256 : 128;
    if (bn == 0) bn = (bm == 512) ? 224 : ((bm == 256 && N >= 256) ? 256 : 128);
    if (prune_out) {
        if (bm == 512 && bn == 224) return launch_cfg<GemmCfg<2, 224, S24_NA_224, S24_NB_224, true, 2>>(g, stream);
        if (bm == 256 && bn == 256) return launch_cfg<GemmCfg<2, 256, S24_NA_256, S24_NB_256, true>>(g, stream);
        if (bm == 256 && bn == 128) return launch_cfg<GemmCfg<2, 128, 6, 6, true>>(g, stream);
        if (bm == 128 && bn == 128) return launch_cfg<GemmCfg<1, 128, 4, 4, true>>(g, stream);
    } else if (bt) {
        if (bm == 512 && bn == 224) return launch_cfg<GemmCfg<2, 224, S24_NA_224, S24_NB_224, false, 2, true>>(g, stream);
        if (bm == 256 && bn == 256) return launch_cfg<GemmCfg<2, 256, S24_NA_256, S24_NB_256, false, 1, true>>(g, stream);
        if (bm == 256 && bn == 128) return launch_cfg<GemmCfg<2, 128, 6, 6, false, 1, true>>(g, stream);
        if (bm == 128 && bn == 128) return launch_cfg<GemmCfg<1, 128, 4, 4, false, 1, true>>(g, stream);
    } else {
        if (bm == 512 && bn == 224) return launch_cfg<GemmCfg<2, 224, S24_NA_224, S24_NB_224, false, 2>>(g, stream);
        if (bm == 256 && bn == 256) return launch_cfg<GemmCfg<2, 256, S24_NA_256, S24_NB_256>>(g, stream);
        if (bm == 256 && bn == 128) return launch_cfg<GemmCfg<2, 128, 6, 6>>(g, stream);
        if (bm == 128 && bn == 128) return launch_cfg<GemmCfg<1, 128, 4, 4>>(g, stream);
    }
    return fail(S24_ERR_UNSUPPORTED, "%s: no kernel for tile %d x %d (have 512x224, 256x256, 256x128, 128x128)", who, bm, bn);
}

// shape rules of the entry points that take the reference's metadata layout, checked before any
// size is derived from M and K (compress_2_4.py:49-65 and :10 give the divisibility rules)
static int check_ref_meta_shape(const char* who, int64_t M, int64_t K)
{
    if (M <= 0 || K <= 0 || M % 32 != 0 || K % 64 != 0)
        return fail(S24_ERR_SHAPE, "%s: needs positive M %% 32 == 0 and K %% 64 == 0 (got M=%lld K=%lld)", who, (long long)M,
                    (long long)K);
    if (M > 0x7FFFFF00ll || K > 0x7FFFFF00ll) return fail(S24_ERR_SHAPE, "%s: dimension too large", who);
    return S24_OK;
}

}  // namespace s24

using namespace s24;

extern "C" int s24_spmm(const void* vals, const void* meta_tc, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                        int64_t ldb, int64_t ldc, int dtype, const s24_tile_cfg* cfg, void* stream)
{
    return run_spmm(vals, meta_tc, B, C, M, N, K, ldb, ldc, dtype, cfg, static_cast<cudaStream_t>(stream));
}

extern "C" int s24_spmm_bt(const void* vals, const void* meta_tc, const void* Bt, void* C, int64_t M, int64_t N, int64_t K,
                           int64_t ldbt, int64_t ldc, int dtype, const s24_tile_cfg* cfg, void* stream)
{
    return run_spmm(vals, meta_tc, Bt, C, M, N, K, ldbt, ldc, dtype, cfg, static_cast<cudaStream_t>(stream), false, nullptr,
                    nullptr, nullptr, true);
}

extern "C" int s24_spmm_scatter(const void* vals, const void* meta_tc, const void* B, void* const* dsts, int n_dst, int64_t M,
                                int64_t N, int64_t K, int64_t ldb, int64_t ldc, int dtype, void* stream)
{
    if (dsts == nullptr) return fail(S24_ERR_INVALID_ARG, "spmm_scatter: null destination list");
    return run_spmm(vals, meta_tc, B, nullptr, M, N, K, ldb, ldc, dtype, nullptr, static_cast<cudaStream_t>(stream), false,
                    nullptr, nullptr, nullptr, false, dsts, n_dst);
}

extern "C" int s24_spmm_ref_meta(const void* vals, const void* meta_ref, const void* B, void* C, int64_t M, int64_t N,
                                 int64_t K, int64_t ldb, int64_t ldc, int dtype, const s24_tile_cfg* cfg,
                                 void* workspace, size_t workspace_bytes, void* stream)
{
    int rc = check_ref_meta_shape("spmm_ref_meta", M, K);
    if (rc) return rc;
    if (workspace == nullptr || workspace_bytes < s24_meta_tc_bytes(M, K))
        return fail(S24_ERR_INVALID_ARG, "spmm_ref_meta: workspace of %zu bytes needed, %zu given", s24_meta_tc_bytes(M, K),
                    workspace_bytes);
    if (!aligned(workspace, 16)) return fail(S24_ERR_INVALID_ARG, "spmm_ref_meta: workspace must be 16-byte aligned");
    rc = s24_meta_convert(meta_ref, S24_META_REF, workspace, S24_META_TC, M, K, stream);
    if (rc) return rc;
    return run_spmm(vals, workspace, B, C, M, N, K, ldb, ldc, dtype, cfg, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- scratch owned by the library
//
// Workspace for s24_spmm_ref_meta_noalloc: callers with a device-memory budget fixed at
// start-up (or a loop that cannot afford cudaMalloc's synchronisation) have no buffer to lend
// us, so the converted metadata lives in this array inside the library image.  In host code
// the name g_static_scratch is only a handle for the runtime, not a device address: the
// address kernels can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
static __device__ __align__(256) unsigned char g_static_scratch[S24_STATIC_SCRATCH_BYTES];

// Device address of the built-in scratch on the current device.  Cached per device ordinal: the
// look-up always yields the same value for a device, so concurrent first calls write the same
// pointer (one CUDA context per device is assumed, see the header).
static int static_scratch_address(void** out)
{
    static void* cached[64] = {nullptr};
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return fail(S24_ERR_UNSUPPORTED, "static scratch: device ordinal %d out of range (0..63)", dev);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        rc = check_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
        if (rc) return rc;
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return S24_OK;
}

extern "C" int s24_spmm_ref_meta_noalloc(const void* vals, const void* meta_ref, const void* B, void* C, int64_t M,
                                         int64_t N, int64_t K, int64_t ldb, int64_t ldc, int dtype,
                                         const s24_tile_cfg* cfg, void* stream)
{
    int rc = check_ref_meta_shape("spmm_ref_meta_noalloc", M, K);
    if (rc) return rc;
    const size_t need = s24_meta_tc_bytes(M, K);
    if (need > (size_t)S24_STATIC_SCRATCH_BYTES)
        return fail(S24_ERR_SHAPE,
                    "spmm_ref_meta_noalloc: metadata of a %lld x %lld matrix needs %zu bytes of scratch but the "
                    "library's built-in buffer holds %zu; use s24_spmm_ref_meta with your own workspace",
                    (long long)M, (long long)K, need, (size_t)S24_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);   // first call per device: address lookup, no allocation
    if (rc) return rc;
    rc = s24_meta_convert(meta_ref, S24_META_REF, scratch, S24_META_TC, M, K, stream);
    if (rc) return rc;
    return run_spmm(vals, scratch, B, C, M, N, K, ldb, ldc, dtype, cfg, static_cast<cudaStream_t>(stream));
}

extern "C" int s24_spmm_prune_out(const void* vals, const void* meta_tc, const void* B, void* C_vals, void* C_meta_ref,
                                  void* C_meta_tc, int64_t M, int64_t N, int64_t K, int64_t ldb, int dtype,
                                  const s24_tile_cfg* cfg, void* stream)
{
    return run_spmm(vals, meta_tc, B, nullptr, M, N, K, ldb, N, dtype, cfg, static_cast<cudaStream_t>(stream), true,
                    C_vals, C_meta_ref, C_meta_tc);
}

// ---------------------------------------------------------------- self-test of the time-out path
//
// A wait that nothing will ever satisfy, with a one-millisecond limit: the thread initialises a
// barrier, waits on it, sees the wait give up and reports code 7 exactly as the GEMM's roles
// report theirs.  Bounded by construction; leaves the context usable.
__global__ void wait_timeout_probe_kernel(int* status, unsigned long long limit_ns)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        const uint32_t b = s24::ptx::smem_u32(&bar);
        s24::ptx::mbar_init(b, 1);
        s24::ptx::fence_barrier_init();
        abort_flag = 0;
        if (!s24::ptx::mbar_wait(b, 0, limit_ns)) s24::report_timeout(status, &abort_flag, 7);
    }
}

extern "C" int s24_selftest_timeout(int kind, const void* vals, const void* meta_tc, const void* B, void* C, int64_t M,
                                    int64_t N, int64_t K, int dtype, const s24_tile_cfg* cfg, void* stream)
{
    constexpr unsigned long long kOneMs = 1000000ull;
    if (kind == 0) {
        int* status = status_word_address();
        if (status == nullptr) return fail(S24_ERR_CUDA, "selftest_timeout: cannot resolve the device status word");
        wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, kOneMs);
        return check_cuda(cudaGetLastError(), "selftest_timeout launch");
    }
    if (kind == 1) {   // the GEMM with its producer stopped after the first k-block and 1 ms waits
        if (K < 2 * kBlockK) return fail(S24_ERR_SHAPE, "selftest_timeout: kind 1 needs K >= %d (got %lld)", 2 * kBlockK, (long long)K);
        return run_spmm(vals, meta_tc, B, C, M, N, K, N, N, dtype, cfg, static_cast<cudaStream_t>(stream), false, nullptr,
                        nullptr, nullptr, false, nullptr, 0, kOneMs, 1);
    }
    return fail(S24_ERR_INVALID_ARG, "selftest_timeout: kind must be 0 (bare wait) or 1 (starved GEMM), got %d", kind);
}

extern "C" int s24_device_status(void* stream)
{
    int* status = status_word_address();
    if (status == nullptr) return fail(S24_ERR_CUDA, "device_status: cannot resolve the device status word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    int rc = check_cuda(cudaMemcpyAsync(&host, status, sizeof(int), cudaMemcpyDeviceToHost, s), "device_status copy");
    if (rc) return rc;
    rc = check_cuda(cudaStreamSynchronize(s), "device_status sync");
    if (rc) return rc;
    if (host == 0) return S24_OK;
    cudaMemsetAsync(status, 0, sizeof(int), s);
    cudaStreamSynchronize(s);
    return fail(S24_ERR_TIMEOUT, "a device-side wait timed out (code %d: 1 producer/empty, 2 mma/full, 3 mma/accumulator, 4 epilogue, 5 prune warp, 6 mma/pruned A, 7 self-test)", host);
}
