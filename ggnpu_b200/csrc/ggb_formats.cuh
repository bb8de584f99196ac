// GGUF block formats as they live in HBM, and their exact decoders.
//
// At upload every weight matrix is re-laid-out ("packed once") from GGUF's
// array-of-blocks into a few streams, each a dense array over all (row, block)
// pairs, so that the hot loops issue only naturally aligned 16-byte loads:
//
//   Q4_K   144 B : hdr[16] (d, dmin, scales[12]) | qs[128]
//   Q5_K   176 B : hdr[16]                       | qh[32]  | qs[128]
//   Q6_K   210 B : ql[128] | qh[64] | scales[16] | d[2]
//   Q2_K    84 B : scales[16] | qs[64] | d,dmin[4]
//   Q3_K   110 B : hmask[32] | qs[64] | scales[12] | d[2]
//   Q8_0    34 B : d[2] | qs[32]
//   Q4_0/IQ4_NL 18 B : d[2] | qs[16]        Q4_1 20 B : d,m[4] | qs[16]
//   IQ4_XS 136 B : hdr[8] (d, scales_h, scales_l[4]) | qs[128]
//   F32 / F16 / BF16 : unchanged
//
// Each stream is a slice [off, off+size) of the GGUF block, so the re-layout is
// a pure permutation of bytes and total bytes equal the GGUF bytes (plus
// alignment padding between streams).  Decoders below reproduce, value for
// value and rounding for rounding, the reference decoders of
// include/ggnpu/quant/kquant.h:70-202, src/quant/q4_0.cpp:18-26,
// src/quant/q4_1.cpp:20-29, src/quant/q8_0.cpp:19-25, src/quant/iq4_nl.cpp:24-31,
// src/quant/iq4_xs.cpp:21-39 and src/utils/bf16.cpp:15-46.  All arithmetic is
// fp32; fp16 scales are widened exactly (subnormals kept), nothing is flushed.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ggb {

enum : uint32_t {
    T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
    T_Q5_K = 13, T_Q6_K = 14, T_IQ4_NL = 20, T_IQ4_XS = 23, T_BF16 = 30,
    // grid-coded formats (their codebooks are generated at build time, see GGB_HAVE_IQ_GRIDS below)
    T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ1_M = 29
};

// The codebooks of the grid-coded formats come from a file generated at build time (iq_tables.py writes
// it from the gguf package).  Where it is absent the library is built without these formats.
#if defined(__has_include)
#if __has_include("ggb_iq_grids.inc")
#define GGB_HAVE_IQ_GRIDS 1
#endif
#endif

constexpr int kMaxStreams = 4;

struct FormatInfo {
    int block_elems;       // 0 => unsupported type
    int block_bytes;
    int n_streams;
    int off[kMaxStreams];  // slice of the GGUF block that forms stream i
    int size[kMaxStreams];
};

__host__ __device__ inline FormatInfo format_info(uint32_t t) {
    switch (t) {
    case T_F32:    return {1, 4, 1, {0, 0, 0, 0}, {4, 0, 0, 0}};
    case T_F16:    return {1, 2, 1, {0, 0, 0, 0}, {2, 0, 0, 0}};
    case T_BF16:   return {1, 2, 1, {0, 0, 0, 0}, {2, 0, 0, 0}};
    case T_Q4_0:   return {32, 18, 2, {0, 2, 0, 0}, {2, 16, 0, 0}};
    case T_IQ4_NL: return {32, 18, 2, {0, 2, 0, 0}, {2, 16, 0, 0}};
    case T_Q4_1:   return {32, 20, 2, {0, 4, 0, 0}, {4, 16, 0, 0}};
    case T_Q8_0:   return {32, 34, 2, {0, 2, 0, 0}, {2, 32, 0, 0}};
    case T_Q2_K:   return {256, 84, 3, {0, 16, 80, 0}, {16, 64, 4, 0}};
    case T_Q3_K:   return {256, 110, 4, {0, 32, 96, 108}, {32, 64, 12, 2}};
    case T_Q4_K:   return {256, 144, 2, {0, 16, 0, 0}, {16, 128, 0, 0}};
    case T_Q5_K:   return {256, 176, 3, {0, 16, 48, 0}, {16, 32, 128, 0}};
    case T_Q6_K:   return {256, 210, 4, {0, 128, 192, 208}, {128, 64, 16, 2}};
    case T_IQ4_XS: return {256, 136, 2, {0, 8, 0, 0}, {8, 128, 0, 0}};
#ifdef GGB_HAVE_IQ_GRIDS
    // one stream: the block as it is in the file (include/ggnpu/quant/iquants.h:40-46 for the sizes)
    case T_IQ2_XXS: return {256, 66, 1, {0, 0, 0, 0}, {66, 0, 0, 0}};
    case T_IQ2_XS:  return {256, 74, 1, {0, 0, 0, 0}, {74, 0, 0, 0}};
    case T_IQ2_S:   return {256, 82, 1, {0, 0, 0, 0}, {82, 0, 0, 0}};
    case T_IQ3_XXS: return {256, 98, 1, {0, 0, 0, 0}, {98, 0, 0, 0}};
    case T_IQ3_S:   return {256, 110, 1, {0, 0, 0, 0}, {110, 0, 0, 0}};
    case T_IQ1_S:   return {256, 50, 1, {0, 0, 0, 0}, {50, 0, 0, 0}};
    case T_IQ1_M:   return {256, 56, 1, {0, 0, 0, 0}, {56, 0, 0, 0}};
#endif
    default:       return {0, 0, 0, {0, 0, 0, 0}, {0, 0, 0, 0}};
    }
}

// A weight matrix [N rows][K] resident in HBM in the stream layout.
// layout 0: streams indexed [row][block].  layout 1 ("row-group major", Q4_K and Q6_K; Q4_K shown): rows are taken in
// groups of 16 (N padded with zero rows), streams indexed [group][block][...] with the quant bytes
// ordered as the A-operand fragments of an m16n8k32 int8 tensor-core instruction:
//   hdr : [group][block][row16][16 B]
//   qs  : [group][block][j = 0..3][lane = 0..31][16 B], lane (g = lane/4, t = lane%4) holding the four
//         32-bit words  {row g, bytes 32j+4t..}, {row g+8, same}, {row g, bytes 32j+16+4t..}, {row g+8, same}
//         (low nibbles = sub-block 2j, high nibbles = sub-block 2j+1 of the GGUF block).
// Any (group, block range) is then one contiguous byte range of each stream.
struct PackedW {
    const uint8_t* s[kMaxStreams];
    int64_t N;
    int K;
    int nb;          // blocks per row = K / block_elems
    uint32_t type;
    int layout;
};

// Byte offsets inside the streams of a Q4_K weight, for either layout.  blk = row * nb + block.
__host__ __device__ __forceinline__ int64_t q4k_hdr_off(int layout, int nb, int64_t blk) {
    if (layout == 0) return blk * 16;
    const int64_t row = blk / nb; const int b = static_cast<int>(blk - row * nb);
    return (((row >> 4) * nb + b) * 16 + (row & 15)) * 16;
}
__host__ __device__ __forceinline__ int64_t q4k_qs_off(int layout, int nb, int64_t blk, int qi) {   // qi = 0..127
    if (layout == 0) return blk * 128 + qi;
    const int64_t row = blk / nb; const int b = static_cast<int>(blk - row * nb);
    const int r = static_cast<int>(row & 15), j = qi >> 5, within = qi & 31;
    const int word = ((within >> 4) << 1) | (r >> 3), lane = ((r & 7) << 2) | ((within & 15) >> 2);
    return ((((row >> 4) * nb + b) * 4 + j) * 32 + lane) * 16 + word * 4 + (within & 3);
}

// Q6_K in layout 1 (row groups of 16, A-operand fragments of m16n8k16 int8 instructions):
//   s0 : [group][block][combo = 2*half + c][lane][16 B] = words {ql_a row g, ql_b row g, ql_a row g+8, ql_b row g+8}
//        with ql_a = ql[64*half + 16c + 4t ..+3], ql_b = ql[64*half + 32 + 16c + 4t ..+3]   (lane = 4g + t)
//   s1 : [group][block][half][lane][16 B] = words {qh(c=0) row g, qh(c=0) row g+8, qh(c=1) row g, qh(c=1) row g+8},
//        qh(c) = qh[32*half + 16c + 4t ..+3]
//   s2 : [group][block][row16][16 B] int8 scales      s3 : [group][block][row16][2 B] fp16 d
__host__ __device__ __forceinline__ int64_t q6k_ql_off(int layout, int nb, int64_t blk, int qi) {      // qi = 0..127
    if (layout == 0) return blk * 128 + qi;
    const int64_t row = blk / nb; const int b = static_cast<int>(blk - row * nb);
    const int r = static_cast<int>(row & 15), hf = qi >> 6, w64 = qi & 63, ab = w64 >> 5, c = (w64 >> 4) & 1, t = (w64 & 15) >> 2;
    return (((((row >> 4) * nb + b) * 4 + 2 * hf + c) * 32 + ((r & 7) << 2) + t) * 4 + ab + 2 * (r >> 3)) * 4 + (qi & 3);
}
__host__ __device__ __forceinline__ int64_t q6k_qh_off(int layout, int nb, int64_t blk, int qi) {      // qi = 0..63
    if (layout == 0) return blk * 64 + qi;
    const int64_t row = blk / nb; const int b = static_cast<int>(blk - row * nb);
    const int r = static_cast<int>(row & 15), hf = qi >> 5, c = (qi >> 4) & 1, t = (qi & 15) >> 2;
    return (((((row >> 4) * nb + b) * 2 + hf) * 32 + ((r & 7) << 2) + t) * 4 + 2 * c + (r >> 3)) * 4 + (qi & 3);
}
__host__ __device__ __forceinline__ int64_t q6k_row_slot(int layout, int nb, int64_t blk) {           // index of (row, block) in s2 / s3
    if (layout == 0) return blk;
    const int64_t row = blk / nb; const int b = static_cast<int>(blk - row * nb);
    return ((row >> 4) * nb + b) * 16 + (row & 15);
}

__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));      // exact widening, subnormals included
}
__device__ __forceinline__ float ld_f16(const uint8_t* p) {   // p 2-byte aligned
    return f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(p));
}

__device__ __constant__ const int8_t kIq4Codebook[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                                         1, 13, 25, 38, 53, 69, 89, 113};

__host__ __device__ constexpr bool is_grid_type(uint32_t t) {
    return t == T_IQ2_XXS || t == T_IQ2_XS || t == T_IQ2_S || t == T_IQ3_XXS || t == T_IQ3_S || t == T_IQ1_S || t == T_IQ1_M;
}

#ifdef GGB_HAVE_IQ_GRIDS
#define GGB_IQ_TABLE(ctype, name, rows, cols) static __device__ const ctype name[rows][cols]
#include "ggb_iq_grids.inc"
#undef GGB_IQ_TABLE

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return p[0] | (static_cast<uint32_t>(p[1]) << 8); }
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }

// Values 8*g8 .. 8*g8+7 of the 256-value block at p (a block is only 2-byte aligned), bit-exact with
// the reference decoders src/quant/iquants.cpp:37-203: eight values share one codebook row (two rows
// of four for the IQ3 formats) and one sign byte; the scale is formed with the reference's roundings
// ((d * (0.5 + s)) * 0.25 etc.), then scale * grid value, then the sign.
template <uint32_t TYPE>
__device__ __forceinline__ void iq_decode8(const uint8_t* p, int g8, float (&out)[8]) {
    const int ib = g8 >> 2, l = g8 & 3;
    if constexpr (TYPE == T_IQ1_S || TYPE == T_IQ1_M) {
        float dl, delta;
        uint32_t idx;
        if constexpr (TYPE == T_IQ1_S) {
            const float d = ld_f16(p);
            const uint32_t qh = ld_u16(p + 34 + 2 * ib);
            dl = __fmul_rn(d, __int2float_rn(2 * static_cast<int>((qh >> 12) & 7) + 1));
            delta = (qh & 0x8000u) ? -0.125f : 0.125f;
            idx = p[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8);
        } else {
            const uint32_t s0 = ld_u16(p + 48), s1 = ld_u16(p + 50), s2 = ld_u16(p + 52), s3 = ld_u16(p + 54);
            const float d = f16_bits_to_f32(static_cast<uint16_t>((s0 >> 12) | ((s1 >> 8) & 0x00F0u) | ((s2 >> 4) & 0x0F00u) | (s3 & 0xF000u)));
            const uint32_t sc = ld_u16(p + 48 + 2 * (ib >> 1));
            dl = __fmul_rn(d, __int2float_rn(2 * static_cast<int>((sc >> (6 * (ib & 1) + 3 * (l >> 1))) & 7) + 1));
            const uint32_t qh = p[32 + 2 * ib + (l >> 1)];
            delta = (qh & ((l & 1) ? 0x80u : 0x08u)) ? -0.125f : 0.125f;
            idx = p[4 * ib + l] | ((qh << ((l & 1) ? 4 : 8)) & 0x700u);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) out[j] = __fmul_rn(dl, __int2float_rn(kIq1sGrid[idx][j]) + delta);
    } else if constexpr (TYPE == T_IQ2_XXS || TYPE == T_IQ2_XS || TYPE == T_IQ2_S) {
        const float d = ld_f16(p);
        float db;
        uint32_t signs;
        const uint8_t* grid;
        if constexpr (TYPE == T_IQ2_XXS) {
            const uint32_t aux = ld_u32(p + 2 + 8 * ib + 4);
            db = __fmul_rn(__fmul_rn(d, 0.5f + __uint2float_rn(aux >> 28)), 0.25f);
            signs = kIqSigns[0][(aux >> (7 * l)) & 127];
            grid = kIq2xxsGrid[p[2 + 8 * ib + l]];
        } else {
            const uint32_t sc = p[(TYPE == T_IQ2_XS ? 66 : 74) + ib];
            db = __fmul_rn(__fmul_rn(d, 0.5f + __uint2float_rn(l < 2 ? (sc & 15) : (sc >> 4))), 0.25f);
            if constexpr (TYPE == T_IQ2_XS) {
                const uint32_t q = ld_u16(p + 2 + 2 * (4 * ib + l));
                signs = kIqSigns[0][q >> 9];
                grid = kIq2xsGrid[q & 511];
            } else {
                signs = p[2 + 32 + 4 * ib + l];
                grid = kIq2sGrid[p[2 + 4 * ib + l] | ((static_cast<uint32_t>(p[66 + ib]) << (8 - 2 * l)) & 0x300u)];
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float v = __fmul_rn(db, __uint2float_rn(grid[j]));
            out[j] = (signs >> j) & 1 ? -v : v;
        }
    } else {
        const float d = ld_f16(p);
        float db;
        uint32_t signs;
        const uint8_t* g1;
        const uint8_t* g2;
        if constexpr (TYPE == T_IQ3_XXS) {
            const uint32_t aux = ld_u32(p + 66 + 4 * ib);
            db = __fmul_rn(__fmul_rn(d, 0.5f + __uint2float_rn(aux >> 28)), 0.5f);
            signs = kIqSigns[0][(aux >> (7 * l)) & 127];
            g1 = kIq3xxsGrid[p[2 + 8 * ib + 2 * l]];
            g2 = kIq3xxsGrid[p[2 + 8 * ib + 2 * l + 1]];
        } else {
            const uint32_t sc = p[106 + (ib >> 1)];
            db = __fmul_rn(d, __int2float_rn(1 + 2 * static_cast<int>((ib & 1) ? (sc >> 4) : (sc & 15))));
            const uint32_t qh = p[66 + ib];
            signs = p[74 + 4 * ib + l];
            g1 = kIq3sGrid[p[2 + 8 * ib + 2 * l] | ((qh << (8 - 2 * l)) & 256u)];
            g2 = kIq3sGrid[p[2 + 8 * ib + 2 * l + 1] | ((qh << (7 - 2 * l)) & 256u)];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float v1 = __fmul_rn(db, __uint2float_rn(g1[j])), v2 = __fmul_rn(db, __uint2float_rn(g2[j]));
            out[j] = (signs >> j) & 1 ? -v1 : v1;
            out[j + 4] = (signs >> (j + 4)) & 1 ? -v2 : v2;
        }
    }
}

template <uint32_t TYPE>
__device__ __forceinline__ float iq_decode_one(const uint8_t* p, int j) {
    float v[8];
    iq_decode8<TYPE>(p, j >> 3, v);
    float r = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) r = (j & 7) == i ? v[i] : r;
    return r;
}
#endif  // GGB_HAVE_IQ_GRIDS

// 6-bit (scale, min) pair j of the 12-byte Q4_K/Q5_K pack.
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* p, int& sc, int& mn) {
    if (j < 4) { sc = p[j] & 63; mn = p[j + 4] & 63; }
    else { sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4); mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}

// Element j of block `blk` (= row * nb + block-in-row), bit-exact with the
// reference decoder of its type.  Products are formed in the reference's
// order; the one rounding of the min-type formats is the final subtract/add
// (an FMA there yields the same bits because the product is exact).
__device__ inline float decode_elem(const PackedW& w, int64_t blk, int j) {
    switch (w.type) {
    case T_F32: return reinterpret_cast<const float*>(w.s[0])[blk];
    case T_F16: return f16_bits_to_f32(reinterpret_cast<const uint16_t*>(w.s[0])[blk]);
    case T_BF16: return __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(w.s[0])[blk]) << 16);
    case T_Q4_0: {
        const float d = ld_f16(w.s[0] + blk * 2);
        const uint8_t b = w.s[1][blk * 16 + (j & 15)];
        return __int2float_rn(static_cast<int>(j < 16 ? (b & 15) : (b >> 4)) - 8) * d;
    }
    case T_Q4_1: {
        const float d = ld_f16(w.s[0] + blk * 4), m = ld_f16(w.s[0] + blk * 4 + 2);
        const uint8_t b = w.s[1][blk * 16 + (j & 15)];
        return __fadd_rn(__fmul_rn(__int2float_rn(j < 16 ? (b & 15) : (b >> 4)), d), m);
    }
    case T_Q8_0: {
        const float d = ld_f16(w.s[0] + blk * 2);
        return __int2float_rn(static_cast<int8_t>(w.s[1][blk * 32 + j])) * d;
    }
    case T_IQ4_NL: {
        const float d = ld_f16(w.s[0] + blk * 2);
        const uint8_t b = w.s[1][blk * 16 + (j & 15)];
        return d * __int2float_rn(kIq4Codebook[j < 16 ? (b & 15) : (b >> 4)]);
    }
    case T_IQ4_XS: {
        const uint8_t* h = w.s[0] + blk * 8;
        const float d = ld_f16(h);
        const unsigned sh = h[2] | (h[3] << 8);
        const int ib = j >> 5, l = j & 31;
        const int ls = ((h[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
        const float dl = d * __int2float_rn(ls - 32);
        const uint8_t b = w.s[1][blk * 128 + 16 * ib + (l & 15)];
        return dl * __int2float_rn(kIq4Codebook[l < 16 ? (b & 15) : (b >> 4)]);
    }
    case T_Q4_K: case T_Q5_K: {
        const uint8_t* h = w.s[0] + q4k_hdr_off(w.layout, w.nb, blk);
        const float d = ld_f16(h), dmin = ld_f16(h + 2);
        const int sb = j >> 5, l = j & 31, g = sb >> 1;
        int sc, mn;
        k4_scale_min(sb, h + 4, sc, mn);
        const uint8_t b = w.type == T_Q4_K ? w.s[1][q4k_qs_off(w.layout, w.nb, blk, 32 * g + l)] : w.s[2][blk * 128 + 32 * g + l];
        int q = (sb & 1) ? (b >> 4) : (b & 15);
        if (w.type == T_Q5_K) q += ((w.s[1][blk * 32 + l] >> sb) & 1) ? 16 : 0;
        return __fsub_rn(__fmul_rn(d * __int2float_rn(sc), __int2float_rn(q)), dmin * __int2float_rn(mn));
    }
    case T_Q6_K: {
        const int64_t slot = q6k_row_slot(w.layout, w.nb, blk);
        const float d = ld_f16(w.s[3] + slot * 2);
        const int hf = j >> 7, r = j & 127, quarter = r >> 5, l = r & 31;
        const uint8_t qh = w.s[1][q6k_qh_off(w.layout, w.nb, blk, 32 * hf + l)];
        const uint8_t lo = w.s[0][q6k_ql_off(w.layout, w.nb, blk, 64 * hf + l + 32 * (quarter & 1))];
        const int q = static_cast<int>(((quarter & 2) ? (lo >> 4) : (lo & 15)) | (((qh >> (2 * quarter)) & 3) << 4)) - 32;
        const int sc = static_cast<int8_t>(w.s[2][slot * 16 + 8 * hf + 2 * quarter + (l >> 4)]);
        return __fmul_rn(__fmul_rn(d, __int2float_rn(sc)), __int2float_rn(q));
    }
    case T_Q2_K: {
        const float d = ld_f16(w.s[2] + blk * 4), dmin = ld_f16(w.s[2] + blk * 4 + 2);
        const int sb = j >> 4, l = j & 15, hf = sb >> 3, sh = (sb >> 1) & 3, odd = sb & 1;
        const uint8_t s = w.s[0][blk * 16 + sb];
        const int q = (w.s[1][blk * 64 + 32 * hf + 16 * odd + l] >> (2 * sh)) & 3;
        return __fsub_rn(__fmul_rn(d * __int2float_rn(s & 15), __int2float_rn(q)), dmin * __int2float_rn(s >> 4));
    }
    case T_Q3_K: {
        const float d = ld_f16(w.s[3] + blk * 2);
        const int sb = j >> 4, l = j & 15, hf = sb >> 3, sh = (sb >> 1) & 3, odd = sb & 1;
        const uint8_t* s = w.s[2] + blk * 12;
        const int lo = (sb < 8) ? (s[sb] & 15) : (s[sb - 8] >> 4);
        const int hi = (s[8 + (sb & 3)] >> (2 * (sb >> 2))) & 3;
        const float dl = d * __int2float_rn((lo | (hi << 4)) - 32);
        const int q = (w.s[1][blk * 64 + 32 * hf + 16 * odd + l] >> (2 * sh)) & 3;
        const int hbit = (w.s[0][blk * 32 + 16 * odd + l] >> (4 * hf + sh)) & 1;
        return dl * __int2float_rn(q - (hbit ? 0 : 4));
    }
#ifdef GGB_HAVE_IQ_GRIDS
    case T_IQ2_XXS: return iq_decode_one<T_IQ2_XXS>(w.s[0] + blk * 66, j);
    case T_IQ2_XS: return iq_decode_one<T_IQ2_XS>(w.s[0] + blk * 74, j);
    case T_IQ2_S: return iq_decode_one<T_IQ2_S>(w.s[0] + blk * 82, j);
    case T_IQ3_XXS: return iq_decode_one<T_IQ3_XXS>(w.s[0] + blk * 98, j);
    case T_IQ3_S: return iq_decode_one<T_IQ3_S>(w.s[0] + blk * 110, j);
    case T_IQ1_S: return iq_decode_one<T_IQ1_S>(w.s[0] + blk * 50, j);
    case T_IQ1_M: return iq_decode_one<T_IQ1_M>(w.s[0] + blk * 56, j);
#endif
    default: return 0.0f;
    }
}

}  // namespace ggb
