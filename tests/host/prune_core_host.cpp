// Host build of csrc/prune_core.cuh: lets the packed bit logic of the CUDA kernels be
// checked exhaustively on a CPU against the oracle.  Test infrastructure only -- the
// library itself has no CPU path.
#include <cstdint>
#include "prune_core.cuh"

using namespace s24;

template <int DT, int MODE>
static void run_pc(const uint16_t* A, int64_t M, int64_t K, int tie, uint16_t* vals, uint16_t* meta)
{
    for (int64_t r = 0; r < M; ++r)
        for (int64_t c8 = 0; c8 < K / 8; ++c8) {
            const uint16_t* a = A + r * K + 8 * c8;
            uint32_t in[4];
            for (int i = 0; i < 4; ++i) in[i] = a[2 * i] | ((uint32_t)a[2 * i + 1] << 16);
            uint32_t lo, hi;
            uint32_t codes = prune_compress_8<DT, MODE>(in[0], in[1], in[2], in[3], tie, lo, hi) >> 24;
            uint16_t* v = vals + r * (K / 2) + 4 * c8;
            v[0] = lo & 0xFFFF; v[1] = lo >> 16; v[2] = hi & 0xFFFF; v[3] = hi >> 16;
            uint16_t& w = meta[r * (K / 16) + c8 / 2];
            if (c8 % 2 == 0) w = (uint16_t)codes; else w |= (uint16_t)(codes << 8);
        }
}

template <int DT, int MODE>
static void run_p(const uint16_t* A, int64_t numel, int tie, uint16_t* out)
{
    for (int64_t i8 = 0; i8 < numel / 8; ++i8) {
        const uint16_t* a = A + 8 * i8;
        uint32_t in[4], o[4];
        for (int i = 0; i < 4; ++i) in[i] = a[2 * i] | ((uint32_t)a[2 * i + 1] << 16);
        prune_8<DT, MODE>(in[0], in[1], in[2], in[3], tie, o[0], o[1], o[2], o[3]);
        for (int i = 0; i < 4; ++i) { out[8 * i8 + 2 * i] = o[i] & 0xFFFF; out[8 * i8 + 2 * i + 1] = o[i] >> 16; }
    }
}

// the GEMM epilogue's variant: signed keys, lower index on ties, codes from the keep mask
template <int DT>
static void run_pc_mask(const uint16_t* A, int64_t M, int64_t K, uint16_t* vals, uint16_t* meta)
{
    for (int64_t r = 0; r < M; ++r)
        for (int64_t c8 = 0; c8 < K / 8; ++c8) {
            const uint16_t* a = A + r * K + 8 * c8;
            uint32_t in[4];
            for (int i = 0; i < 4; ++i) in[i] = a[2 * i] | ((uint32_t)a[2 * i + 1] << 16);
            uint32_t lo, hi;
            uint32_t codes = prune_compress_8_from_mask<DT>(in[0], in[1], in[2], in[3], lo, hi) >> 24;
            uint16_t* v = vals + r * (K / 2) + 4 * c8;
            v[0] = lo & 0xFFFF; v[1] = lo >> 16; v[2] = hi & 0xFFFF; v[3] = hi >> 16;
            uint16_t& w = meta[r * (K / 16) + c8 / 2];
            if (c8 % 2 == 0) w = (uint16_t)codes; else w |= (uint16_t)(codes << 8);
        }
}

extern "C" {
void host_prune_compress_from_mask(const uint16_t* A, int64_t M, int64_t K, int dtype, uint16_t* vals, uint16_t* meta_logical)
{
    if (dtype == kBf16) run_pc_mask<kBf16>(A, M, K, vals, meta_logical);
    else run_pc_mask<kFp16>(A, M, K, vals, meta_logical);
}
void host_prune_compress(const uint16_t* A, int64_t M, int64_t K, int dtype, int mode, int tie,
                         uint16_t* vals, uint16_t* meta_logical)
{
#define PC(DT)                                                                           \
    if (mode == kModeSigned) run_pc<DT, kModeSigned>(A, M, K, tie, vals, meta_logical);     \
    else if (mode == kModeMagnitude) run_pc<DT, kModeMagnitude>(A, M, K, tie, vals, meta_logical); \
    else run_pc<DT, kModeNone>(A, M, K, tie, vals, meta_logical);
    if (dtype == kBf16) { PC(kBf16) } else { PC(kFp16) }
#undef PC
}
void host_prune(const uint16_t* A, int64_t numel, int dtype, int mode, int tie, uint16_t* out)
{
    if (dtype == kBf16) {
        if (mode == kModeMagnitude) run_p<kBf16, kModeMagnitude>(A, numel, tie, out);
        else run_p<kBf16, kModeSigned>(A, numel, tie, out);
    } else {
        if (mode == kModeMagnitude) run_p<kFp16, kModeMagnitude>(A, numel, tie, out);
        else run_p<kFp16, kModeSigned>(A, numel, tie, out);
    }
}
unsigned host_keep_mask(const float* k, int tie) { return keep_mask_scalar(k, tie); }
}
