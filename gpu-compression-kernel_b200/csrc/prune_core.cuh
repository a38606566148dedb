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

// per-half max / min of packed 16-bit floats (either operand may be returned for +0 / -0)
template <int DT>
S24_HD uint32_t max2(uint32_t a, uint32_t b)
{
#if defined(__CUDA_ARCH__)
    if (DT == kBf16) {
        __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    __half2 r = __hmax2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
#else
    uint32_t lo = bits_to_float(a & 0xFFFF, DT) >= bits_to_float(b & 0xFFFF, DT) ? (a & 0xFFFFu) : (b & 0xFFFFu);
    uint32_t hi = bits_to_float(a >> 16, DT) >= bits_to_float(b >> 16, DT) ? (a & 0xFFFF0000u) : (b & 0xFFFF0000u);
    return lo | hi;
#endif
}

template <int DT>
S24_HD uint32_t min2(uint32_t a, uint32_t b)
{
#if defined(__CUDA_ARCH__)
    if (DT == kBf16) {
        __nv_bfloat162 r = __hmin2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    __half2 r = __hmin2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
#else
    uint32_t lo = bits_to_float(a & 0xFFFF, DT) <= bits_to_float(b & 0xFFFF, DT) ? (a & 0xFFFFu) : (b & 0xFFFFu);
    uint32_t hi = bits_to_float(a >> 16, DT) <= bits_to_float(b >> 16, DT) ? (a & 0xFFFF0000u) : (b & 0xFFFF0000u);
    return lo | hi;
#endif
}

// non-zero flags; +0.0 and -0.0 are both "zero" (dense != 0, compress_2_4.py:72)
template <int DT>
S24_HD uint32_t nz2(uint32_t a)
{
#if defined(__CUDA_ARCH__)
    uint32_t zero = 0;
    if (DT == kBf16) return __hne2_mask(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&zero));
    return __hne2_mask(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&zero));
#else
    uint32_t m = a & 0x7FFF7FFFu;
    return ((m & 0xFFFFu) ? 0xFFFFu : 0u) | ((m >> 16) ? 0xFFFF0000u : 0u);
#endif
}

S24_HD uint32_t sel(uint32_t mask, uint32_t a, uint32_t b) { return (a & mask) | (b & ~mask); }

// ---------------------------------------------------------------- encoder (shared)

// From the surviving elements p_j (dropped ones already zeroed) produce the two stored values
// of each group and the 4-bit codes, exactly as compress_2_4.py:113-131 does from the
// non-zero flags m_j = (p_j != 0):
//   idx0 = 0 if m0, 1 if !m0 & m1, else 2;  idx1 = 1 if m0 & m1, 3 if (!m0 & !m1) | m3, else 2
//   code = idx0 | idx1 << 2, which over (m0, m1) reads 0100 / 1001 / 1000 / 1110 for
//   (1,1) / (0,1) / (1,0) / (0,0), with bit 2 also set by m3.
//   v0/v1: stored value 0 / 1 of group G (low half) and G+1 (high half)
//   codes: bits 0-3 code of group G, bits 16-19 code of group G+1
struct PairOut {
    uint32_t v0, v1, codes;
};

// the same from given "stored" flags m0, m1, m3 (0xFFFF / 0 per half) instead of non-zero flags
S24_HD PairOut encode_pair_flags(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, uint32_t m0, uint32_t m1, uint32_t m3);

template <int DT, bool ZERO_SIGN_CLEAR>
S24_HD PairOut encode_pair(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3)
{
    const uint32_t m0 = nz2<DT>(p0), m1 = nz2<DT>(p1), m3 = nz2<DT>(p3);
    if (ZERO_SIGN_CLEAR) {  // magnitude mode: a surviving -0.0 reads +0.0
        p0 &= m0;
        p1 &= m1;
        p2 &= nz2<DT>(p2);
        p3 &= m3;
    }
    return encode_pair_flags(p0, p1, p2, p3, m0, m1, m3);
}

S24_HD PairOut encode_pair_flags(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, uint32_t m0, uint32_t m1, uint32_t m3)
{
    const uint32_t both = m0 & m1;
    const uint32_t none_or_m3 = ~(m0 | m1) | m3;
    PairOut o;
    o.v0 = sel(m0, p0, sel(m1, p1, p2));
    o.v1 = sel(both, p1, sel(none_or_m3, p3, p2));
    o.codes = ((0x000E000Eu ^ (m0 & 0x00060006u)) ^ (m1 & 0x00070007u) ^ (both & 0x000B000Bu)) | (m3 & 0x00040004u);
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

// Keep masks of two groups at once.  The second and third largest keys of a group are the
// two "middle" elements {min(max(a0,a1), max(a2,a3)), max(min(a0,a1), min(a2,a3))}; an
// element survives when its key reaches the second largest.  That is exact unless second ==
// third (a tie across the keep/drop boundary), which `tie` reports per half so that the
// group can be redone with keep_mask_scalar.  All comparisons are fp16/bf16 SIMD compares.
template <int DT, int MODE>
S24_HD void keep_masks(uint32_t P0, uint32_t P1, uint32_t P2, uint32_t P3, uint32_t& k0, uint32_t& k1, uint32_t& k2,
                       uint32_t& k3, uint32_t& tie)
{
    if (MODE == kModeNone) {
        k0 = k1 = k2 = k3 = 0xFFFFFFFFu;
        tie = 0;
        return;
    }
    const uint32_t km = MODE == kModeMagnitude ? 0x7FFF7FFFu : 0xFFFFFFFFu;
    const uint32_t K0 = P0 & km, K1 = P1 & km, K2 = P2 & km, K3 = P3 & km;
    const uint32_t hi01 = max2<DT>(K0, K1), lo01 = min2<DT>(K0, K1);
    const uint32_t hi23 = max2<DT>(K2, K3), lo23 = min2<DT>(K2, K3);
    const uint32_t x = min2<DT>(hi01, hi23), y = max2<DT>(lo01, lo23);
    const uint32_t second = max2<DT>(x, y);
    tie = eq2<DT>(x, y);
    k0 = ge2<DT>(K0, second);
    k1 = ge2<DT>(K1, second);
    k2 = ge2<DT>(K2, second);
    k3 = ge2<DT>(K3, second);
}

S24_HD uint32_t maj3(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | (a & c) | (b & c); }

// Groups with a tie across the keep/drop boundary (tiebits = 0xFFFF in their half): redo the keep
// masks with pairwise comparisons under the requested tie rule, still two groups at a time and
// without branches, and patch them in.  Element i "beats" j when it ranks ahead of it; an element
// survives when it beats at least two others.
//   kTieLower      i < j: i beats j on >=
//   kTieHigher     i < j: i beats j on >  (the higher index wins equal keys)
//   kTieReference  as kTieLower, except where element 0 is the strict minimum: then the smallest
//                  of elements 1..3 is dropped, the lowest index among equals, and if all three
//                  are equal elements 1 and 3 survive (keep_mask_scalar states the same rule and
//                  is checked against the table measured from the reference)
template <int DT, int MODE>
S24_HD void fix_tied_masks(uint32_t P0, uint32_t P1, uint32_t P2, uint32_t P3, uint32_t tiebits, int tie, uint32_t& k0,
                           uint32_t& k1, uint32_t& k2, uint32_t& k3)
{
    const uint32_t km = MODE == kModeMagnitude ? 0x7FFF7FFFu : 0xFFFFFFFFu;
    const uint32_t K0 = P0 & km, K1 = P1 & km, K2 = P2 & km, K3 = P3 & km;
    uint32_t b01, b02, b03, b12, b13, b23;
    if (tie == kTieHigher) {
        b01 = ~ge2<DT>(K1, K0); b02 = ~ge2<DT>(K2, K0); b03 = ~ge2<DT>(K3, K0);
        b12 = ~ge2<DT>(K2, K1); b13 = ~ge2<DT>(K3, K1); b23 = ~ge2<DT>(K3, K2);
    } else {
        b01 = ge2<DT>(K0, K1); b02 = ge2<DT>(K0, K2); b03 = ge2<DT>(K0, K3);
        b12 = ge2<DT>(K1, K2); b13 = ge2<DT>(K1, K3); b23 = ge2<DT>(K2, K3);
    }
    uint32_t n0 = maj3(b01, b02, b03), n1 = maj3(~b01, b12, b13), n2 = maj3(~b02, ~b12, b23), n3 = maj3(~b03, ~b13, ~b23);
    if (tie == kTieReference) {
        const uint32_t r21 = ge2<DT>(K2, K1), r31 = ge2<DT>(K3, K1), r32 = ge2<DT>(K3, K2);
        const uint32_t zero_min = ~(b01 | b02 | b03);          // a0 < a1, a2, a3
        const uint32_t alleq = b12 & r21 & b23 & r32;          // a1 == a2 == a3
        const uint32_t one_min = r21 & r31;                    // a1 <= a2 and a1 <= a3
        const uint32_t d1 = one_min & ~alleq;
        const uint32_t d2 = (~one_min & r32) | alleq;
        const uint32_t d3 = ~one_min & ~r32;
        n0 = n0 & ~zero_min;
        n1 = sel(zero_min, ~d1, n1);
        n2 = sel(zero_min, ~d2, n2);
        n3 = sel(zero_min, ~d3, n3);
    }
    k0 = sel(tiebits, n0, k0);
    k1 = sel(tiebits, n1, k1);
    k2 = sel(tiebits, n2, k2);
    k3 = sel(tiebits, n3, k3);
}

// Complete treatment of 8 consecutive elements (two groups) held as four registers in
// memory order: in0 = (a0,a1) of group G, in1 = (a2,a3) of G, in2 = (a0,a1) of G+1, in3.
//   out_lo / out_hi : the 4 stored values in memory order (v0_G, v1_G) / (v0_G+1, v1_G+1)
//   returns a word whose top byte is code_G | code_G+1 << 4 (lower bytes are scratch)
template <int DT, int MODE>
S24_HD uint32_t prune_compress_8(uint32_t in0, uint32_t in1, uint32_t in2, uint32_t in3, int tie, uint32_t& out_lo,
                                 uint32_t& out_hi)
{
    const uint32_t P0 = byte_perm(in0, in2, 0x5410), P1 = byte_perm(in0, in2, 0x7632);
    const uint32_t P2 = byte_perm(in1, in3, 0x5410), P3 = byte_perm(in1, in3, 0x7632);
    uint32_t k0, k1, k2, k3, tiebits;
    keep_masks<DT, MODE>(P0, P1, P2, P3, k0, k1, k2, k3, tiebits);
    if (tiebits != 0) fix_tied_masks<DT, MODE>(P0, P1, P2, P3, tiebits, tie, k0, k1, k2, k3);  // rare
    const PairOut o = encode_pair<DT, MODE == kModeMagnitude>(P0 & k0, P1 & k1, P2 & k2, P3 & k3);
    out_lo = byte_perm(o.v0, o.v1, 0x5410);
    out_hi = byte_perm(o.v0, o.v1, 0x7632);
    // codes = lo + hi * 2^16; times (2^24 + 2^12) puts lo at bits 24-27 and hi at bits 28-31
    return o.codes * 0x01001000u;
}

// The same for a fused GEMM epilogue (compression/kernels/10.1_prune_acc.py:100-117): signed keys, the
// lower index survives a tie, and the codes come from the keep masks themselves, so a surviving
// exact zero is still recorded where it stands (the reference's kernel encodes from its mask, not
// from non-zero flags).
template <int DT>
S24_HD uint32_t prune_compress_8_from_mask(uint32_t in0, uint32_t in1, uint32_t in2, uint32_t in3, uint32_t& out_lo,
                                           uint32_t& out_hi)
{
    const uint32_t P0 = byte_perm(in0, in2, 0x5410), P1 = byte_perm(in0, in2, 0x7632);
    const uint32_t P2 = byte_perm(in1, in3, 0x5410), P3 = byte_perm(in1, in3, 0x7632);
    uint32_t k0, k1, k2, k3, tiebits;
    keep_masks<DT, kModeSigned>(P0, P1, P2, P3, k0, k1, k2, k3, tiebits);
    if (tiebits != 0) fix_tied_masks<DT, kModeSigned>(P0, P1, P2, P3, tiebits, kTieLower, k0, k1, k2, k3);
    const PairOut o = encode_pair_flags(P0 & k0, P1 & k1, P2 & k2, P3 & k3, k0, k1, k3);
    out_lo = byte_perm(o.v0, o.v1, 0x5410);
    out_hi = byte_perm(o.v0, o.v1, 0x7632);
    return o.codes * 0x01001000u;
}

// gather the top bytes of four such words into one 32-bit metadata word
S24_HD uint32_t gather_code_bytes(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3)
{
    return byte_perm(byte_perm(c0, c1, 0x0073), byte_perm(c2, c3, 0x0073), 0x5410);
}

// Keep masks only (dense prune output): the 8 elements with dropped ones zeroed.
template <int DT, int MODE>
S24_HD void prune_8(uint32_t in0, uint32_t in1, uint32_t in2, uint32_t in3, int tie, uint32_t& o0, uint32_t& o1,
                    uint32_t& o2, uint32_t& o3)
{
    const uint32_t P0 = byte_perm(in0, in2, 0x5410), P1 = byte_perm(in0, in2, 0x7632);
    const uint32_t P2 = byte_perm(in1, in3, 0x5410), P3 = byte_perm(in1, in3, 0x7632);
    uint32_t k0, k1, k2, k3, tiebits;
    keep_masks<DT, MODE>(P0, P1, P2, P3, k0, k1, k2, k3, tiebits);
    if (tiebits != 0) fix_tied_masks<DT, MODE>(P0, P1, P2, P3, tiebits, tie, k0, k1, k2, k3);
    uint32_t p0 = P0 & k0, p1 = P1 & k1, p2 = P2 & k2, p3 = P3 & k3;
    if (MODE == kModeMagnitude) {  // defined as where(prune(|A|) != 0, A, 0): surviving -0.0 reads +0.0
        p0 &= nz2<DT>(p0);
        p1 &= nz2<DT>(p1);
        p2 &= nz2<DT>(p2);
        p3 &= nz2<DT>(p3);
    }
    o0 = byte_perm(p0, p1, 0x5410);
    o2 = byte_perm(p0, p1, 0x7632);
    o1 = byte_perm(p2, p3, 0x5410);
    o3 = byte_perm(p2, p3, 0x7632);
}

// 32 elements of one row -> 16 stored values + 32 metadata bits
template <int DT, int MODE>
S24_HD uint32_t row_span(const uint32_t (&lo)[8], const uint32_t (&hi)[8], int tie, uint32_t (&out)[8])
{
    const uint32_t c0 = prune_compress_8<DT, MODE>(lo[0], lo[1], lo[2], lo[3], tie, out[0], out[1]);
    const uint32_t c1 = prune_compress_8<DT, MODE>(lo[4], lo[5], lo[6], lo[7], tie, out[2], out[3]);
    const uint32_t c2 = prune_compress_8<DT, MODE>(hi[0], hi[1], hi[2], hi[3], tie, out[4], out[5]);
    const uint32_t c3 = prune_compress_8<DT, MODE>(hi[4], hi[5], hi[6], hi[7], tie, out[6], out[7]);
    return gather_code_bytes(c0, c1, c2, c3);
}

#if defined(__CUDACC__)
// 32-byte (or 2 x 16-byte) streaming loads of dense input, bypassing L1
__device__ __forceinline__ void ld256(const void* p, uint32_t (&r)[8])
{
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}

__device__ __forceinline__ void ld128x2(const void* p, uint32_t (&r)[8])
{
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "l"(p));
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(static_cast<const char*>(p) + 16));
}
#endif

}  // namespace s24
