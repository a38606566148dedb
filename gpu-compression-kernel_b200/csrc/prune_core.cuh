// prune_core.cuh -- the per-group arithmetic of 2:4 prune + compress.
//
// Everything here is host+device so the same source can be compiled by g++ for an
// exhaustive CPU check of the bit logic (tests/test_prune_core_host.py) and by nvcc for
// the kernels.  The semantics follow the reference project:
//   keep mask       compression/prune.py:85-91 (drop the two smallest keys of a group of 4)
//   flags -> codes  compression/compress_2_4.py:69-72,113-121,131
//   stored values   compression/compress_2_4.py:123-127
//
// Two groups are processed at a time in "packed" form: register Pj holds element j of
// group G in its low 16 bits and element j of group G+1 in its high 16 bits, so one
// half2 comparison ranks both groups.  Comparison results are 0xFFFF / 0x0000 per half.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#define S24_HD __host__ __device__ __forceinline__
#else
#include <string.h>
#define S24_HD inline
#endif

namespace s24 {

enum : int { kFp16 = 0, kBf16 = 1 };
enum : int { kModeSigned = 0, kModeMagnitude = 1, kModeNone = 2 };  // None: compress only
enum : int { kTieReference = 0, kTieLower = 1, kTieHigher = 2 };

// ---------------------------------------------------------------- scalar helpers

S24_HD float bits_to_float(uint32_t v16, int dtype)
{
#if defined(__CUDA_ARCH__)
    if (dtype == kBf16) return __uint_as_float(v16 << 16);
    return __half2float(__ushort_as_half((unsigned short)v16));
#else
    uint32_t out;
    if (dtype == kBf16) {
        out = v16 << 16;
    } else {
        uint32_t sign = (v16 & 0x8000u) << 16, exp = (v16 >> 10) & 0x1Fu, man = v16 & 0x3FFu;
        if (exp == 0) {
            if (man == 0) out = sign;
            else {
                int shift = 0;
                while (!(man & 0x400u)) { man <<= 1; ++shift; }
                out = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3FFu) << 13);
            }
        } else if (exp == 31) out = sign | 0x7F800000u | (man << 13);
        else out = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
#endif
}

S24_HD uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel)
{
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, sel);
#else
    uint64_t v = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) r |= (uint32_t)((v >> (8 * ((sel >> (4 * i)) & 7))) & 0xFF) << (8 * i);
    return r;
#endif
}

// per-half comparisons of packed 16-bit floats -> 0xFFFF / 0 masks
template <int DT>
S24_HD uint32_t ge2(uint32_t a, uint32_t b)
{
#if defined(__CUDA_ARCH__)
    if (DT == kBf16) return __hge2_mask(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return __hge2_mask(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
#else
    uint32_t lo = bits_to_float(a & 0xFFFF, DT) >= bits_to_float(b & 0xFFFF, DT) ? 0xFFFFu : 0u;
    uint32_t hi = bits_to_float(a >> 16, DT) >= bits_to_float(b >> 16, DT) ? 0xFFFF0000u : 0u;
    return lo | hi;
#endif
}

template <int DT>
S24_HD uint32_t eq2(uint32_t a, uint32_t b)
{
#if defined(__CUDA_ARCH__)
    if (DT == kBf16) return __heq2_mask(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return __heq2_mask(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
#else
    uint32_t lo = bits_to_float(a & 0xFFFF, DT) == bits_to_float(b & 0xFFFF, DT) ? 0xFFFFu : 0u;
    uint32_t hi = bits_to_float(a >> 16, DT) == bits_to_float(b >> 16, DT) ? 0xFFFF0000u : 0u;
    return lo | hi;
#endif
}

// non-zero flags; +0.0 and -0.0 are both "zero" (dense != 0, compress_2_4.py:72)
S24_HD uint32_t nz2(uint32_t a)
{
#if defined(__CUDA_ARCH__)
    // an fp16 compare against +0.0; bf16 zeros have the same two bit patterns
    uint32_t m = a & 0x7FFF7FFFu;  // (also keeps NaN payloads from comparing unordered)
    return __vcmpne2(m, 0u);
#else
    uint32_t m = a & 0x7FFF7FFFu;
    return ((m & 0xFFFFu) ? 0xFFFFu : 0u) | ((m >> 16) ? 0xFFFF0000u : 0u);
#endif
}

S24_HD uint32_t sel(uint32_t mask, uint32_t a, uint32_t b) { return (a & mask) | (b & ~mask); }
S24_HD uint32_t maj(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | (a & c) | (b & c); }

// ---------------------------------------------------------------- encoder (shared)

// From keep masks and the elements, produce the two stored values of each group and the
// 4-bit codes.  pm_j marks the elements that survive pruning with their bits intact, m_j
// the survivors that are also non-zero (the flags the reference's encoder sees).
//   V0/V1: stored value 0 / 1 of group G (low half) and G+1 (high half)
//   codes: bits 0-3 code of group G, bits 16-19 code of group G+1
struct PairOut {
    uint32_t v0, v1, codes;
};

S24_HD PairOut encode_pair(uint32_t P0, uint32_t P1, uint32_t P2, uint32_t P3,
                           uint32_t k0, uint32_t k1, uint32_t k2, uint32_t k3, uint32_t keep_zero_bits)
{
    // keep_zero_bits = ~0 : a surviving zero keeps its bit pattern (signed mode, -0.0 stays)
    //                =  0 : surviving zeros read +0.0 (magnitude mode)
    uint32_t n0 = nz2(P0), n1 = nz2(P1), n2 = nz2(P2), n3 = nz2(P3);
    uint32_t p0 = P0 & k0 & (n0 | keep_zero_bits);
    uint32_t p1 = P1 & k1 & (n1 | keep_zero_bits);
    uint32_t p2 = P2 & k2 & (n2 | keep_zero_bits);
    uint32_t p3 = P3 & k3 & (n3 | keep_zero_bits);
    uint32_t m0 = k0 & n0, m1 = k1 & n1, m3 = k3 & n3;
    (void)n2;
    // compress_2_4.py:113-121
    uint32_t both = m0 & m1;        // expr0
    uint32_t only1 = ~m0 & m1;      // expr1 -> bit0
    uint32_t none = ~(m0 | m1);     // expr2 -> bit1
    uint32_t bit2 = both | none | m3;
    uint32_t bit3 = ~both;          // expr1 | ~m1
    PairOut o;
    o.v0 = sel(m0, p0, sel(m1, p1, p2));                    // idx0 in {0,1,2}
    o.v1 = sel(both, p1, sel(none | m3, p3, p2));           // idx1 in {1,2,3}
    o.codes = (only1 & 0x00010001u) | (none & 0x00020002u) | (bit2 & 0x00040004u) | (bit3 & 0x00080008u);
    return o;
}

// ---------------------------------------------------------------- tie handling (scalar)

// Keep mask of one group from its four keys under a tie rule.
//   kTieLower / kTieHigher : rank by (key desc, index asc / desc)
//   kTieReference          : what the reference's CPU torch.topk(k=2, largest=False) does
//     (prune.py:85).  Measured over all 75 weak orderings it equals "lower index survives"
//     except when element 0 is the strict minimum: then elements 1..3 are ranked with
//     "higher index survives", and if all three are equal elements 1 and 3 survive.
S24_HD uint32_t keep_mask_scalar(const float k[4], int tie)
{
    if (tie == kTieReference) {
        if (k[0] < k[1] && k[0] < k[2] && k[0] < k[3]) {
            if (k[1] == k[2] && k[2] == k[3]) return 0xAu;  // {1,3}
            // drop the smallest of 1..3, the lowest index among equals
            if (k[1] <= k[2] && k[1] <= k[3]) return 0xCu;  // {2,3}
            if (k[2] <= k[3]) return 0xAu;                  // {1,3}
            return 0x6u;                                    // {1,2}
        }
        tie = kTieLower;
    }
    uint32_t mask = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int beaten = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j == i) continue;
            bool first = (tie == kTieLower) ? (j < i) : (j > i);
            if (k[j] > k[i] || (k[j] == k[i] && first)) ++beaten;
        }
        if (beaten < 2) mask |= 1u << i;
    }
    return mask;
}

// ---------------------------------------------------------------- the packed fast path

// Result of pruning + encoding two groups.  tie != 0 in a half means that group has a key
// tie across the keep / drop boundary and must be redone with keep_mask_scalar.
struct PairResult {
    uint32_t v0, v1, codes, tie;
};

// keymask: 0xFFFFFFFF signed keys, 0x7FFF7FFF magnitude keys.
// force_keep: 0xFFFFFFFF turns pruning off (compress-only), else 0.
template <int DT>
S24_HD PairResult prune_encode_pair(uint32_t P0, uint32_t P1, uint32_t P2, uint32_t P3,
                                    uint32_t keymask, uint32_t force_keep, uint32_t keep_zero_bits)
{
    uint32_t K0 = P0 & keymask, K1 = P1 & keymask, K2 = P2 & keymask, K3 = P3 & keymask;
    uint32_t g01 = ge2<DT>(K0, K1), g02 = ge2<DT>(K0, K2), g03 = ge2<DT>(K0, K3);
    uint32_t g12 = ge2<DT>(K1, K2), g13 = ge2<DT>(K1, K3), g23 = ge2<DT>(K2, K3);
    // element i survives when it beats at least two others; i beats j>i on >=, j beats i on >
    uint32_t k0 = maj(g01, g02, g03);
    uint32_t k1 = maj(~g01, g12, g13);
    uint32_t k2 = maj(~g02, ~g12, g23);
    uint32_t k3 = maj(~g03, ~g13, ~g23);
    uint32_t e01 = eq2<DT>(K0, K1), e02 = eq2<DT>(K0, K2), e03 = eq2<DT>(K0, K3);
    uint32_t e12 = eq2<DT>(K1, K2), e13 = eq2<DT>(K1, K3), e23 = eq2<DT>(K2, K3);
    uint32_t tie = (e01 & (k0 ^ k1)) | (e02 & (k0 ^ k2)) | (e03 & (k0 ^ k3)) |
                   (e12 & (k1 ^ k2)) | (e13 & (k1 ^ k3)) | (e23 & (k2 ^ k3));
    PairOut o = encode_pair(P0, P1, P2, P3, k0 | force_keep, k1 | force_keep, k2 | force_keep,
                            k3 | force_keep, keep_zero_bits);
    PairResult r;
    r.v0 = o.v0;
    r.v1 = o.v1;
    r.codes = o.codes;
    r.tie = tie & ~force_keep;
    return r;
}

// Redo one group (half = 0 low / 1 high of the packed registers) with the scalar tie rule
// and patch the packed outputs.
template <int DT>
S24_HD void fix_tied_group(uint32_t P0, uint32_t P1, uint32_t P2, uint32_t P3, int half, int mode, int tie,
                           PairResult& r)
{
    const int sh = 16 * half;
    float k[4];
    uint32_t e[4] = {(P0 >> sh) & 0xFFFFu, (P1 >> sh) & 0xFFFFu, (P2 >> sh) & 0xFFFFu, (P3 >> sh) & 0xFFFFu};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v = bits_to_float(e[i], DT);
        k[i] = (mode == kModeMagnitude) ? (v < 0.f ? -v : v) : v;
    }
    uint32_t m = keep_mask_scalar(k, tie);
    uint32_t hm = 0xFFFFu << sh;
    uint32_t k0 = (m & 1u) ? hm : 0u, k1 = (m & 2u) ? hm : 0u, k2 = (m & 4u) ? hm : 0u, k3 = (m & 8u) ? hm : 0u;
    PairOut o = encode_pair(P0 & hm, P1 & hm, P2 & hm, P3 & hm, k0, k1, k2, k3,
                            mode == kModeMagnitude ? 0u : 0xFFFFFFFFu);
    r.v0 = (r.v0 & ~hm) | (o.v0 & hm);
    r.v1 = (r.v1 & ~hm) | (o.v1 & hm);
    r.codes = (r.codes & ~hm) | (o.codes & hm);
}

// Complete treatment of 8 consecutive elements (two groups) held as four registers in
// memory order: in0 = (a0,a1) of group G, in1 = (a2,a3) of G, in2 = (a0,a1) of G+1, in3.
//   out_lo / out_hi : the 4 stored values in memory order (v0_G, v1_G) / (v0_G+1, v1_G+1)
//   returns the two 4-bit codes as one byte: code_G | code_G+1 << 4
template <int DT>
S24_HD uint32_t prune_compress_8(uint32_t in0, uint32_t in1, uint32_t in2, uint32_t in3, int mode, int tie,
                                 uint32_t keymask, uint32_t force_keep, uint32_t keep_zero_bits,
                                 uint32_t& out_lo, uint32_t& out_hi)
{
    uint32_t P0 = byte_perm(in0, in2, 0x5410), P1 = byte_perm(in0, in2, 0x7632);
    uint32_t P2 = byte_perm(in1, in3, 0x5410), P3 = byte_perm(in1, in3, 0x7632);
    PairResult r = prune_encode_pair<DT>(P0, P1, P2, P3, keymask, force_keep, keep_zero_bits);
    if (r.tie != 0 && tie != kTieLower) {  // rare: a tie across the keep/drop boundary
        if (r.tie & 0xFFFFu) fix_tied_group<DT>(P0, P1, P2, P3, 0, mode, tie, r);
        if (r.tie >> 16) fix_tied_group<DT>(P0, P1, P2, P3, 1, mode, tie, r);
    }
    out_lo = byte_perm(r.v0, r.v1, 0x5410);
    out_hi = byte_perm(r.v0, r.v1, 0x7632);
    return (r.codes & 0xFu) | ((r.codes >> 12) & 0xF0u);
}

// Keep masks only (dense prune output): returns the 8 elements with dropped ones zeroed.
template <int DT>
S24_HD void prune_8(uint32_t in0, uint32_t in1, uint32_t in2, uint32_t in3, int mode, int tie, uint32_t keymask,
                    uint32_t keep_zero_bits, uint32_t& o0, uint32_t& o1, uint32_t& o2, uint32_t& o3)
{
    uint32_t P0 = byte_perm(in0, in2, 0x5410), P1 = byte_perm(in0, in2, 0x7632);
    uint32_t P2 = byte_perm(in1, in3, 0x5410), P3 = byte_perm(in1, in3, 0x7632);
    uint32_t K0 = P0 & keymask, K1 = P1 & keymask, K2 = P2 & keymask, K3 = P3 & keymask;
    uint32_t g01 = ge2<DT>(K0, K1), g02 = ge2<DT>(K0, K2), g03 = ge2<DT>(K0, K3);
    uint32_t g12 = ge2<DT>(K1, K2), g13 = ge2<DT>(K1, K3), g23 = ge2<DT>(K2, K3);
    uint32_t k0 = maj(g01, g02, g03), k1 = maj(~g01, g12, g13), k2 = maj(~g02, ~g12, g23), k3 = maj(~g03, ~g13, ~g23);
    uint32_t e01 = eq2<DT>(K0, K1), e02 = eq2<DT>(K0, K2), e03 = eq2<DT>(K0, K3);
    uint32_t e12 = eq2<DT>(K1, K2), e13 = eq2<DT>(K1, K3), e23 = eq2<DT>(K2, K3);
    uint32_t tiebits = (e01 & (k0 ^ k1)) | (e02 & (k0 ^ k2)) | (e03 & (k0 ^ k3)) |
                       (e12 & (k1 ^ k2)) | (e13 & (k1 ^ k3)) | (e23 & (k2 ^ k3));
    if (tiebits != 0 && tie != kTieLower) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int sh = 16 * half;
            if (((tiebits >> sh) & 0xFFFFu) == 0) continue;
            float k[4];
            uint32_t e[4] = {(P0 >> sh) & 0xFFFFu, (P1 >> sh) & 0xFFFFu, (P2 >> sh) & 0xFFFFu, (P3 >> sh) & 0xFFFFu};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = bits_to_float(e[i], DT);
                k[i] = (mode == kModeMagnitude) ? (v < 0.f ? -v : v) : v;
            }
            uint32_t m = keep_mask_scalar(k, tie);
            uint32_t hm = 0xFFFFu << sh;
            k0 = (k0 & ~hm) | ((m & 1u) ? hm : 0u);
            k1 = (k1 & ~hm) | ((m & 2u) ? hm : 0u);
            k2 = (k2 & ~hm) | ((m & 4u) ? hm : 0u);
            k3 = (k3 & ~hm) | ((m & 8u) ? hm : 0u);
        }
    }
    uint32_t p0 = P0 & k0 & (nz2(P0) | keep_zero_bits), p1 = P1 & k1 & (nz2(P1) | keep_zero_bits);
    uint32_t p2 = P2 & k2 & (nz2(P2) | keep_zero_bits), p3 = P3 & k3 & (nz2(P3) | keep_zero_bits);
    o0 = byte_perm(p0, p1, 0x5410);
    o2 = byte_perm(p0, p1, 0x7632);
    o1 = byte_perm(p2, p3, 0x5410);
    o3 = byte_perm(p2, p3, 0x7632);
}

}  // namespace s24
