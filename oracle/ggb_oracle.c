/*
 * ggb_oracle.c -- CPU restatement of ggnpu's CPU arithmetic for the Backend
 * operator path.  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA kernels
 * are compared against, never a product path and never a fallback.
 *
 * Every function names the reference file:line (paths relative to the ggnpu
 * tree) whose arithmetic, operation order and rounding it restates.  Parity is
 * pinned: tests compare this file bit-for-bit with the reference's own
 * functions compiled from the reference tree (oracle/_ref) and with the golden
 * vectors of the reference's tests/test_quant.cpp and tests/test_arch.cpp.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (see oracle/Makefile); the
 * reference is built -O3 for baseline x86-64 (no FMA, no reassociation), so a
 * sequential float loop here rounds exactly like the reference's.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GGO_API __attribute__((visibility("default")))

/* ggml type ids, include/ggnpu/tensor.h:11-42 */
enum {
    GGO_F32 = 0, GGO_F16 = 1, GGO_Q4_0 = 2, GGO_Q4_1 = 3, GGO_Q8_0 = 8,
    GGO_Q2_K = 10, GGO_Q3_K = 11, GGO_Q4_K = 12, GGO_Q5_K = 13, GGO_Q6_K = 14,
    GGO_IQ4_NL = 20, GGO_IQ4_XS = 23, GGO_BF16 = 30,
    GGO_IQ2_XXS = 16, GGO_IQ2_XS = 17, GGO_IQ3_XXS = 18, GGO_IQ1_S = 19, GGO_IQ3_S = 21, GGO_IQ2_S = 22, GGO_IQ1_M = 29
};

/* Codebooks of the grid-coded formats: generated at build time from the gguf package (the file
 * ggnpu_b200/iq_tables.py writes).  Without it those formats are reported as unsupported. */
#if defined(__has_include)
#if __has_include("ggb_iq_grids.inc")
#define GGO_HAVE_IQ_GRIDS 1
#define GGB_IQ_TABLE(ctype, name, rows, cols) static const ctype name[rows][cols]
#include "ggb_iq_grids.inc"
#undef GGB_IQ_TABLE
#endif
#endif

/* ---- scalar conversions ------------------------------------------------- */

/* include/ggnpu/quant/kquant.h:30-53 and src/utils/bf16.cpp:22-46 (both give
 * the exact IEEE widening, subnormals included). */
GGO_API float ggo_f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, u;
    if (e == 31u) u = s | 0x7F800000u | (m << 13);
    else if (e) u = s | ((e + 112u) << 23) | (m << 13);
    else if (!m) u = s;
    else {
        int sh = 0;
        while (!(m & 1024u)) { m <<= 1; ++sh; }
        u = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
    }
    float f; memcpy(&f, &u, 4); return f;
}

/* src/utils/bf16.cpp:15-20 */
GGO_API float ggo_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f;
}

/* src/utils/bf16.cpp:6-13: round-to-nearest-even by bias add, no NaN case. */
GGO_API uint16_t ggo_f32_to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float rd_f16(const uint8_t* p) { return ggo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

/* ---- block geometry: src/gguf/tensor.cpp:18-38 --------------------------- */

GGO_API int ggo_block_elems(uint32_t t) {
    switch (t) {
    case GGO_F32: case GGO_F16: case GGO_BF16: return 1;
    case GGO_Q4_0: case GGO_Q4_1: case GGO_Q8_0: case GGO_IQ4_NL: return 32;
    case GGO_Q2_K: case GGO_Q3_K: case GGO_Q4_K: case GGO_Q5_K: case GGO_Q6_K: case GGO_IQ4_XS: return 256;
#ifdef GGO_HAVE_IQ_GRIDS
    case GGO_IQ2_XXS: case GGO_IQ2_XS: case GGO_IQ2_S: case GGO_IQ3_XXS: case GGO_IQ3_S: case GGO_IQ1_S: case GGO_IQ1_M: return 256;
#endif
    default: return 0;
    }
}

GGO_API int ggo_block_bytes(uint32_t t) {
    switch (t) {
    case GGO_F32: return 4; case GGO_F16: case GGO_BF16: return 2;
    case GGO_Q4_0: return 18; case GGO_Q4_1: return 20; case GGO_Q8_0: return 34;
    case GGO_Q2_K: return 84; case GGO_Q3_K: return 110; case GGO_Q4_K: return 144;
    case GGO_Q5_K: return 176; case GGO_Q6_K: return 210;
    case GGO_IQ4_NL: return 18; case GGO_IQ4_XS: return 136;
#ifdef GGO_HAVE_IQ_GRIDS
    /* include/ggnpu/quant/iquants.h:40-46 */
    case GGO_IQ2_XXS: return 66; case GGO_IQ2_XS: return 74; case GGO_IQ2_S: return 82;
    case GGO_IQ3_XXS: return 98; case GGO_IQ3_S: return 110; case GGO_IQ1_S: return 50; case GGO_IQ1_M: return 56;
#endif
    default: return 0;
    }
}

/* ---- block decoders ------------------------------------------------------ */

/* src/quant/iq4_nl.cpp:16-18 (same table in src/quant/iq4_xs.cpp:14-16) */
static const int8_t kIq4Codebook[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* src/quant/q4_0.cpp:18-26: (nibble-8)*d, int first then one float multiply. */
static void dq_q4_0(const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    for (int j = 0; j < 16; ++j) {
        y[j] = (float)((int)(b[2 + j] & 15) - 8) * d;
        y[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d;
    }
}

/* src/quant/q4_1.cpp:20-29: nibble*d + m (product then add, two roundings). */
static void dq_q4_1(const uint8_t* b, float* y) {
    const float d = rd_f16(b), m = rd_f16(b + 2);
    for (int j = 0; j < 16; ++j) {
        y[j] = (float)(int)(b[4 + j] & 15) * d + m;
        y[j + 16] = (float)(int)(b[4 + j] >> 4) * d + m;
    }
}

/* src/quant/q8_0.cpp:19-25 */
static void dq_q8_0(const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)b[2 + j] * d;
}

/* src/quant/iq4_nl.cpp:24-31 */
static void dq_iq4_nl(const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    for (int j = 0; j < 16; ++j) {
        y[j] = d * (float)kIq4Codebook[b[2 + j] & 15];
        y[j + 16] = d * (float)kIq4Codebook[b[2 + j] >> 4];
    }
}

/* src/quant/iq4_xs.cpp:21-39: 8 sub-blocks of 32; 6-bit scale = 4 low bits
 * from scales_l, 2 high bits from the u16 scales_h; dl = d*(ls-32). */
static void dq_iq4_xs(const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    const unsigned sh = (unsigned)(b[2] | (b[3] << 8));
    for (int ib = 0; ib < 8; ++ib) {
        const int ls = (int)((b[4 + ib / 2] >> (4 * (ib & 1))) & 15) | (int)(((sh >> (2 * ib)) & 3u) << 4);
        const float dl = d * (float)(ls - 32);
        const uint8_t* q = b + 8 + 16 * ib;
        for (int j = 0; j < 16; ++j) {
            y[32 * ib + j] = dl * (float)kIq4Codebook[q[j] & 15];
            y[32 * ib + j + 16] = dl * (float)kIq4Codebook[q[j] >> 4];
        }
    }
}

/* include/ggnpu/quant/kquant.h:56-64: 6-bit (scale, min) pair j of a 12-byte pack. */
static void k4_scale_min(int j, const uint8_t* p, int* sc, int* mn) {
    if (j < 4) { *sc = p[j] & 63; *mn = p[j + 4] & 63; }
    else { *sc = (p[j + 4] & 15) | ((p[j - 4] >> 6) << 4); *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}

/* include/ggnpu/quant/kquant.h:70-91: dl = d*(sc&15), ml = dmin*(sc>>4),
 * y = dl*q - ml; sub-blocks of 16, two per shift step, 128 values per half. */
static void dq_q2_k(const uint8_t* b, float* y) {
    const float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
    for (int sb = 0; sb < 16; ++sb) {          /* sub-block sb covers y[16*sb .. 16*sb+15] */
        const int half = sb >> 3, j = (sb >> 1) & 3, odd = sb & 1;
        const uint8_t s = b[sb];
        const float dl = d * (float)(s & 15), ml = dmin * (float)(s >> 4);
        const uint8_t* q = b + 16 + 32 * half + 16 * odd;
        for (int l = 0; l < 16; ++l) y[16 * sb + l] = dl * (float)((q[l] >> (2 * j)) & 3) - ml;
    }
}

/* include/ggnpu/quant/kquant.h:96-130: 16 signed 6-bit scales rebuilt from
 * 12 bytes; value = dl * (q2 - (hmask bit ? 0 : 4)), dl = d*(scale-32). */
static void dq_q3_k(const uint8_t* b, float* y) {
    const float d = rd_f16(b + 108);
    const uint8_t* s = b + 96;
    for (int sb = 0; sb < 16; ++sb) {
        /* scale sb: low 4 bits from bytes 0..7 (nibble), high 2 bits from bytes 8..11 */
        const int lo = (sb < 8) ? (s[sb] & 15) : (s[sb - 8] >> 4);
        const int hi = (s[8 + (sb & 3)] >> (2 * (sb >> 2))) & 3;
        const float dl = d * (float)((int)(int8_t)(lo | (hi << 4)) - 32);
        const int half = sb >> 3, j = (sb >> 1) & 3, odd = sb & 1;
        const uint8_t* q = b + 32 + 32 * half + 16 * odd;
        const uint8_t* hm = b + 16 * odd;
        const uint8_t mbit = (uint8_t)(1u << (4 * half + j));
        for (int l = 0; l < 16; ++l)
            y[16 * sb + l] = dl * (float)((int)((q[l] >> (2 * j)) & 3) - ((hm[l] & mbit) ? 0 : 4));
    }
}

/* include/ggnpu/quant/kquant.h:133-151 */
static void dq_q4_k(const uint8_t* b, float* y) {
    const float d = rd_f16(b), dmin = rd_f16(b + 2);
    for (int g = 0; g < 4; ++g) {
        int s1, m1, s2, m2;
        k4_scale_min(2 * g, b + 4, &s1, &m1);
        k4_scale_min(2 * g + 1, b + 4, &s2, &m2);
        const float d1 = d * (float)s1, n1 = dmin * (float)m1, d2 = d * (float)s2, n2 = dmin * (float)m2;
        const uint8_t* q = b + 16 + 32 * g;
        for (int l = 0; l < 32; ++l) {
            y[64 * g + l] = d1 * (float)(q[l] & 15) - n1;
            y[64 * g + 32 + l] = d2 * (float)(q[l] >> 4) - n2;
        }
    }
}

/* include/ggnpu/quant/kquant.h:157-179 */
static void dq_q5_k(const uint8_t* b, float* y) {
    const float d = rd_f16(b), dmin = rd_f16(b + 2);
    const uint8_t* qh = b + 16;
    for (int g = 0; g < 4; ++g) {
        int s1, m1, s2, m2;
        k4_scale_min(2 * g, b + 4, &s1, &m1);
        k4_scale_min(2 * g + 1, b + 4, &s2, &m2);
        const float d1 = d * (float)s1, n1 = dmin * (float)m1, d2 = d * (float)s2, n2 = dmin * (float)m2;
        const uint8_t* q = b + 48 + 32 * g;
        for (int l = 0; l < 32; ++l) {
            y[64 * g + l] = d1 * (float)((q[l] & 15) + (((qh[l] >> (2 * g)) & 1) ? 16 : 0)) - n1;
            y[64 * g + 32 + l] = d2 * (float)((q[l] >> 4) + (((qh[l] >> (2 * g + 1)) & 1) ? 16 : 0)) - n2;
        }
    }
}

/* include/ggnpu/quant/kquant.h:182-202: y = (d * sc) * q, left to right. */
static void dq_q6_k(const uint8_t* b, float* y) {
    const float d = rd_f16(b + 208);
    for (int h = 0; h < 2; ++h) {
        const uint8_t* ql = b + 64 * h;
        const uint8_t* qh = b + 128 + 32 * h;
        const int8_t* sc = (const int8_t*)(b + 192 + 8 * h);
        float* o = y + 128 * h;
        for (int l = 0; l < 32; ++l) {
            const int is = l >> 4;
            const int q1 = (int)((ql[l] & 15) | ((qh[l] & 3) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 15) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            o[l] = d * (float)sc[is] * (float)q1;
            o[l + 32] = d * (float)sc[is + 2] * (float)q2;
            o[l + 64] = d * (float)sc[is + 4] * (float)q3;
            o[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
    }
}

#ifdef GGO_HAVE_IQ_GRIDS
/* Grid-coded formats, src/quant/iquants.cpp:37-203.  A 256-value block is 8 sub-blocks of 32; a
 * sub-block is 4 runs of 8 values that share one codebook row (IQ3: two rows of 4) and one byte of
 * signs.  Value = (sub-block scale * codebook entry), negated where the sign bit is set; the scale
 * roundings follow the reference: (d * (0.5 + s)) * 0.25 for IQ2, * 0.5 for IQ3_XXS, d * (2 s + 1)
 * for IQ3_S and IQ1; IQ1 adds a sub-block offset of +-1/8 to the ternary codebook entry first. */
static uint32_t rd_u16(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }
static uint32_t rd_u32(const uint8_t* p) { return rd_u16(p) | (rd_u16(p + 2) << 16); }

static void put8(float* y, float scale, const uint8_t* row, int n, int first_bit, uint32_t signs) {
    for (int j = 0; j < n; ++j) {
        const float v = scale * (float)row[j];
        y[j] = ((signs >> (first_bit + j)) & 1) ? -v : v;
    }
}

static void dq_iq2(uint32_t type, const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    for (int ib = 0; ib < 8; ++ib) {
        for (int l = 0; l < 4; ++l, y += 8) {
            if (type == GGO_IQ2_XXS) {                            /* iquants.cpp:37-54 */
                const uint8_t* q = b + 2 + 8 * ib;
                const uint32_t aux = rd_u32(q + 4);
                const float db = d * (0.5f + (float)(aux >> 28)) * 0.25f;
                put8(y, db, kIq2xxsGrid[q[l]], 8, 0, kIqSigns[0][(aux >> (7 * l)) & 127]);
            } else {
                const uint32_t sc = b[(type == GGO_IQ2_XS ? 66 : 74) + ib];
                const float db = d * (0.5f + (float)(l < 2 ? (sc & 15) : (sc >> 4))) * 0.25f;
                if (type == GGO_IQ2_XS) {                         /* iquants.cpp:56-73 */
                    const uint32_t q = rd_u16(b + 2 + 2 * (4 * ib + l));
                    put8(y, db, kIq2xsGrid[q & 511], 8, 0, kIqSigns[0][q >> 9]);
                } else {                                          /* iquants.cpp:75-97 */
                    const uint32_t idx = b[2 + 4 * ib + l] | (((uint32_t)b[66 + ib] << (8 - 2 * l)) & 0x300u);
                    put8(y, db, kIq2sGrid[idx], 8, 0, b[34 + 4 * ib + l]);
                }
            }
        }
    }
}

static void dq_iq3(uint32_t type, const uint8_t* b, float* y) {
    const float d = rd_f16(b);
    for (int ib = 0; ib < 8; ++ib) {
        for (int l = 0; l < 4; ++l, y += 8) {
            const uint8_t* q = b + 2 + 8 * ib + 2 * l;
            if (type == GGO_IQ3_XXS) {                            /* iquants.cpp:99-121 */
                const uint32_t aux = rd_u32(b + 66 + 4 * ib);
                const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
                const uint32_t signs = kIqSigns[0][(aux >> (7 * l)) & 127];
                put8(y, db, kIq3xxsGrid[q[0]], 4, 0, signs);
                put8(y + 4, db, kIq3xxsGrid[q[1]], 4, 4, signs);
            } else {                                              /* iquants.cpp:123-159 */
                const uint32_t sc = b[106 + (ib >> 1)], qh = b[66 + ib], signs = b[74 + 4 * ib + l];
                const float db = d * (float)(1 + 2 * (int)((ib & 1) ? (sc >> 4) : (sc & 15)));
                put8(y, db, kIq3sGrid[q[0] | ((qh << (8 - 2 * l)) & 256u)], 4, 0, signs);
                put8(y + 4, db, kIq3sGrid[q[1] | ((qh << (7 - 2 * l)) & 256u)], 4, 4, signs);
            }
        }
    }
}

static void dq_iq1(uint32_t type, const uint8_t* b, float* y) {
    float d;
    if (type == GGO_IQ1_S) d = rd_f16(b);                         /* iquants.cpp:161-178 */
    else {                                                        /* iquants.cpp:180-203: d is spread over the scale words */
        const uint32_t s0 = rd_u16(b + 48), s1 = rd_u16(b + 50), s2 = rd_u16(b + 52), s3 = rd_u16(b + 54);
        d = ggo_f16_to_f32((uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00F0u) | ((s2 >> 4) & 0x0F00u) | (s3 & 0xF000u)));
    }
    for (int ib = 0; ib < 8; ++ib) {
        for (int l = 0; l < 4; ++l, y += 8) {
            float dl, delta;
            uint32_t idx;
            if (type == GGO_IQ1_S) {
                const uint32_t qh = rd_u16(b + 34 + 2 * ib);
                dl = d * (float)(2 * (int)((qh >> 12) & 7) + 1);
                delta = (qh & 0x8000u) ? -0.125f : 0.125f;
                idx = b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8);
            } else {
                const uint32_t sc = rd_u16(b + 48 + 2 * (ib >> 1)), qh = b[32 + 2 * ib + (l >> 1)];
                dl = d * (float)(2 * (int)((sc >> (6 * (ib & 1) + 3 * (l >> 1))) & 7) + 1);
                delta = (qh & ((l & 1) ? 0x80u : 0x08u)) ? -0.125f : 0.125f;
                idx = b[4 * ib + l] | ((qh << ((l & 1) ? 4 : 8)) & 0x700u);
            }
            for (int j = 0; j < 8; ++j) y[j] = dl * ((float)kIq1sGrid[idx][j] + delta);
        }
    }
}
#endif  /* GGO_HAVE_IQ_GRIDS */

/* One block of any supported type -> fp32.  Returns 0, or -1 for an
 * unsupported type. */
GGO_API int ggo_dequant_block(uint32_t type, const uint8_t* blk, float* out) {
    switch (type) {
    case GGO_F32: memcpy(out, blk, 4); return 0;
    case GGO_F16: out[0] = ggo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))); return 0;
    case GGO_BF16: out[0] = ggo_bf16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))); return 0;
    case GGO_Q4_0: dq_q4_0(blk, out); return 0;
    case GGO_Q4_1: dq_q4_1(blk, out); return 0;
    case GGO_Q8_0: dq_q8_0(blk, out); return 0;
    case GGO_Q2_K: dq_q2_k(blk, out); return 0;
    case GGO_Q3_K: dq_q3_k(blk, out); return 0;
    case GGO_Q4_K: dq_q4_k(blk, out); return 0;
    case GGO_Q5_K: dq_q5_k(blk, out); return 0;
    case GGO_Q6_K: dq_q6_k(blk, out); return 0;
    case GGO_IQ4_NL: dq_iq4_nl(blk, out); return 0;
    case GGO_IQ4_XS: dq_iq4_xs(blk, out); return 0;
#ifdef GGO_HAVE_IQ_GRIDS
    case GGO_IQ2_XXS: case GGO_IQ2_XS: case GGO_IQ2_S: dq_iq2(type, blk, out); return 0;
    case GGO_IQ3_XXS: case GGO_IQ3_S: dq_iq3(type, blk, out); return 0;
    case GGO_IQ1_S: case GGO_IQ1_M: dq_iq1(type, blk, out); return 0;
#endif
    default: return -1;
    }
}

GGO_API int ggo_dequant_blocks(uint32_t type, const uint8_t* data, int64_t n_blocks, float* out) {
    const int be = ggo_block_elems(type), bb = ggo_block_bytes(type);
    if (!be) return -1;
    for (int64_t i = 0; i < n_blocks; ++i) ggo_dequant_block(type, data + i * bb, out + i * be);
    return 0;
}

/* src/cli/main.cpp:36-261 (dequant_tensor_row): row `row` of a [N rows][K]
 * weight; a row is ceil(K/blk) consecutive blocks; values past K are dropped. */
GGO_API int ggo_dequant_row(uint32_t type, const uint8_t* data, int64_t row, int K, float* out) {
    const int be = ggo_block_elems(type), bb = ggo_block_bytes(type);
    if (!be || K <= 0) return -1;
    const int64_t bpr = ((int64_t)K + be - 1) / be;
    const uint8_t* r = data + row * bpr * bb;
    float tmp[256];
    for (int64_t b = 0; b < bpr; ++b) {
        ggo_dequant_block(type, r + b * bb, tmp);
        for (int j = 0; j < be; ++j) { const int64_t k = b * be + j; if (k < K) out[k] = tmp[j]; }
    }
    return 0;
}

/* ---- matmul --------------------------------------------------------------- */

/* src/cli/main.cpp:1379-1388 (GGNPU_FP32_MATMUL path, the exact CPU matmul for
 * every format) and :270-327 compute_logits' CPU branch: dequantise row n,
 * one running fp32 sum over k in order.  Applied per activation row m. */
GGO_API int ggo_matmul_exact(const float* A, int M, int lda, const uint8_t* W, uint32_t type,
                             int N, int K, float* C, int ldc) {
    float* w = (float*)malloc(sizeof(float) * (size_t)K);
    if (!w) return -1;
    for (int n = 0; n < N; ++n) {
        if (ggo_dequant_row(type, W, n, K, w)) { free(w); return -1; }
        for (int m = 0; m < M; ++m) {
            const float* a = A + (size_t)m * lda;
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += a[k] * w[k];
            C[(size_t)m * ldc + n] = acc;
        }
    }
    free(w);
    return 0;
}

/* src/backends/cpu_ref/cpu_ref.cpp:87-117 (Q4_K / Q6_K only): one partial sum
 * per 256-block, added into C in block order.  lda/ldc are ignored (K, N). */
GGO_API int ggo_matmul_cpu_ref_k(const float* A, int M, const uint8_t* W, uint32_t type,
                                 int N, int K, float* C) {
    if (type != GGO_Q4_K && type != GGO_Q6_K) return -1;
    const int bb = ggo_block_bytes(type);
    const int64_t bpr = ((int64_t)K + 255) / 256;
    memset(C, 0, sizeof(float) * (size_t)M * N);
    float w[256];
    for (int n = 0; n < N; ++n)
        for (int64_t b = 0; b < bpr; ++b) {
            ggo_dequant_block(type, W + ((int64_t)n * bpr + b) * bb, w);
            for (int m = 0; m < M; ++m) {
                float s = 0.0f;
                for (int j = 0; j < 256; ++j) { const int64_t k = b * 256 + j; if (k < K) s += A[(size_t)m * K + k] * w[j]; }
                C[(size_t)m * N + n] += s;
            }
        }
    return 0;
}

/* src/backends/cpu_ref/cpu_ref.cpp:119-133: F32 B is [K][N]. */
GGO_API void ggo_matmul_f32_kn(const float* A, const float* B, float* C, int M, int N, int K) {
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float s = 0.0f;
            for (int k = 0; k < K; ++k) s += A[(size_t)m * K + k] * B[(size_t)k * N + n];
            C[(size_t)m * N + n] = s;
        }
}

/* ---- elementwise / norm / attention: src/backends/cpu_ref/cpu_ref.cpp ----- */

/* cpu_ref.cpp:139-156 */
GGO_API void ggo_rms_norm(const float* x, float* y, int n, float eps, const float* w) {
    float v = 0.0f;
    for (int i = 0; i < n; ++i) v += x[i] * x[i];
    v /= (float)n;
    v += eps;
    const float inv = 1.0f / sqrtf(v);
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv * (w ? w[i] : 1.0f);
}

/* src/cli/main.cpp:3294-3299 (per-head QK-norm, sum of squares in double) */
GGO_API void ggo_rms_norm_head_f64(float* v, int n, float eps, const float* w) {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += (double)v[i] * v[i];
    const float inv = 1.0f / sqrtf((float)(ss / n) + eps);
    for (int i = 0; i < n; ++i) v[i] = v[i] * inv * w[i];
}

/* cpu_ref.cpp:200-209 */
GGO_API void ggo_silu(const float* x, float* y, int n) {
    for (int i = 0; i < n; ++i) y[i] = x[i] / (1.0f + expf(-x[i]));
}

/* cpu_ref.cpp:211-221 */
GGO_API void ggo_gelu(const float* x, float* y, int n) {
    const float k = 0.7978845608f;
    for (int i = 0; i < n; ++i) y[i] = 0.5f * x[i] * (1.0f + tanhf(k * (x[i] + 0.044715f * x[i] * x[i] * x[i])));
}

/* cpu_ref.cpp:176-198 */
GGO_API void ggo_softmax(const float* x, float* y, int rows, int cols) {
    for (int r = 0; r < rows; ++r) {
        const float* xi = x + (size_t)r * cols; float* yo = y + (size_t)r * cols;
        float mx = -INFINITY, s = 0.0f;
        for (int c = 0; c < cols; ++c) if (xi[c] > mx) mx = xi[c];
        for (int c = 0; c < cols; ++c) { yo[c] = expf(xi[c] - mx); s += yo[c]; }
        for (int c = 0; c < cols; ++c) yo[c] /= s;
    }
}

/* cpu_ref.cpp:223-280: Q [nh][hd]; K,V [nh][ctx][hd] already GQA-expanded;
 * keys j > query_pos masked to -inf; scale 1/sqrt(hd); query_pos<0 => ctx-1. */
GGO_API int ggo_flash_attn(const float* Q, const float* K, const float* V, float* out,
                           int nh, int hd, int64_t ctx, int64_t qpos) {
    if (qpos < 0) qpos = ctx - 1;
    const float scale = 1.0f / sqrtf((float)hd);
    float* sc = (float*)malloc(sizeof(float) * (size_t)ctx);
    if (!sc) return -1;
    for (int h = 0; h < nh; ++h) {
        const float* q = Q + (size_t)h * hd;
        const float* k = K + (size_t)h * ctx * hd;
        const float* v = V + (size_t)h * ctx * hd;
        float* o = out + (size_t)h * hd;
        for (int64_t j = 0; j < ctx; ++j) sc[j] = -INFINITY;
        for (int64_t j = 0; j <= qpos && j < ctx; ++j) {
            float s = 0.0f;
            for (int d = 0; d < hd; ++d) s += q[d] * k[j * hd + d];
            sc[j] = s * scale;
        }
        float mx = -INFINITY, sum = 0.0f;
        for (int64_t j = 0; j < ctx; ++j) if (sc[j] > mx) mx = sc[j];
        for (int64_t j = 0; j < ctx; ++j) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
        for (int64_t j = 0; j < ctx; ++j) sc[j] /= sum;
        for (int d = 0; d < hd; ++d) o[d] = 0.0f;
        for (int64_t j = 0; j < ctx; ++j)
            for (int d = 0; d < hd; ++d) o[d] += sc[j] * v[j * hd + d];
    }
    free(sc);
    return 0;
}

/* cpu_ref.cpp:158-174: Backend::rope of the CPU backend (base fixed at 10000,
 * adjacent pairs, angle = offset * 10000^(-i/n_dims) * freq_scale). */
GGO_API void ggo_rope_cpu_ref(float* x, int n_dims, int64_t offset, float freq_scale, int64_t rope_dims) {
    for (int64_t i = 0; i < rope_dims; i += 2) {
        const float ratio = 1.0f / powf(10000.0f, (float)i / (float)n_dims);
        const float a = (float)offset * ratio * freq_scale;
        const float c = cosf(a), s = sinf(a), v0 = x[i], v1 = x[i + 1];
        x[i] = v0 * c - v1 * s;
        x[i + 1] = v0 * s + v1 * c;
    }
}

/* src/cli/main.cpp:665-692 (RopeCache::build): tables [max_pos][n_dims/2],
 * angle = scale*pos / (base^(2i/n_dims) * ff_i), all in float; ff 0 => 1. */
GGO_API void ggo_rope_table(int64_t max_pos, int n_dims, float freq_scale, float freq_base,
                            const float* ff, int n_ff, float* cos_out, float* sin_out) {
    const int pairs = n_dims / 2;
    for (int64_t p = 0; p < max_pos; ++p)
        for (int i = 0; i < pairs; ++i) {
            float f = (ff && i < n_ff) ? ff[i] : 1.0f;
            if (f == 0.0f) f = 1.0f;
            const float wl = powf(freq_base, 2.0f * (float)i / (float)n_dims);
            const float a = freq_scale * (float)p / (wl * f);
            cos_out[p * pairs + i] = cosf(a);
            sin_out[p * pairs + i] = sinf(a);
        }
}

/* src/cli/main.cpp:1294-1308 (adjacent pairs; neox=0) and :3328-3341 (NeoX
 * split-half; neox=1), both from the table row of position `pos`.
 * rot_dims <= head_dim rotates only the leading dims (main.cpp:906-920). */
GGO_API void ggo_rope_apply(float* out, const float* in, int n_heads, int head_dim, int rot_dims,
                            const float* cos_row, const float* sin_row, int neox) {
    const int half = rot_dims / 2;
    for (int h = 0; h < n_heads; ++h) {
        const float* ih = in + (size_t)h * head_dim; float* oh = out + (size_t)h * head_dim;
        if (out != in) for (int i = rot_dims; i < head_dim; ++i) oh[i] = ih[i];
        for (int i = 0; i < half; ++i) {
            const float c = cos_row[i], s = sin_row[i];
            const int i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
            const float v0 = ih[i0], v1 = ih[i1];
            oh[i0] = v0 * c - v1 * s;
            oh[i1] = v0 * s + v1 * c;
        }
    }
}

/* src/cli/main.cpp:827-838: greedy = first index whose logit is strictly greater. */
GGO_API int ggo_argmax_first(const float* x, int n) {
    int best = 0; float bv = -INFINITY;
    for (int i = 0; i < n; ++i) if (x[i] > bv) { bv = x[i]; best = i; }
    return best;
}

/* src/cli/main.cpp:839-864: temperature sampling.  The reference draws with std::mt19937 and
 * std::discrete_distribution<int>; both are restated here from their published definitions (ISO C++ [rand.eng.mers],
 * [rand.dist.samp.discrete]; the distribution's arithmetic as GNU libstdc++ implements it, which is what the
 * reference links against):
 *   - mt19937: the 32-bit Mersenne Twister, state seeded from (seed mod 2^32) by x[i] = 1812433253 *
 *     (x[i-1] ^ (x[i-1] >> 30)) + i;
 *   - the caller's seed is replaced by the generator's first output (main.cpp:862);
 *   - probs_i = exp((v_i - max) / temp) / sum_exp, float, sum_exp accumulated sequentially in float (:849-859);
 *   - the distribution divides the probs by their double sum, forms running sums in double, sets the last to 1
 *     and returns the first index whose running sum is >= u, where u = (r1 + r2 * 2^32) / 2^64 in double from the
 *     generator's next two outputs (generate_canonical<double, 53>), stepped just below 1 if it rounds to 1.
 * Pinned by the sampled streams the reference CLI prints (tests/golden/ref_cli.npz). */
typedef struct { uint32_t x[624]; int idx; } ggo_mt19937;
static void ggo_mt_seed(ggo_mt19937* g, uint32_t seed) {
    g->x[0] = seed;
    for (int i = 1; i < 624; ++i) g->x[i] = 1812433253u * (g->x[i - 1] ^ (g->x[i - 1] >> 30)) + (uint32_t)i;
    g->idx = 624;
}
static uint32_t ggo_mt_next(ggo_mt19937* g) {
    if (g->idx >= 624) {
        for (int i = 0; i < 624; ++i) {
            const uint32_t y = (g->x[i] & 0x80000000u) | (g->x[(i + 1) % 624] & 0x7FFFFFFFu);
            g->x[i] = g->x[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908B0DFu : 0u);
        }
        g->idx = 0;
    }
    uint32_t y = g->x[g->idx++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9D2C5680u;
    y ^= (y << 15) & 0xEFC60000u;
    y ^= y >> 18;
    return y;
}
GGO_API int ggo_sample_token(const float* logits, int n, float temp, uint64_t* seed) {
    if (temp <= 0.0f) return ggo_argmax_first(logits, n);
    ggo_mt19937 g;
    ggo_mt_seed(&g, (uint32_t)(*seed & 0xFFFFFFFFu));
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    float* probs = (float*)malloc(sizeof(float) * (size_t)n);
    double* cp = (double*)malloc(sizeof(double) * (size_t)n);
    float sum_exp = 0.0f;
    for (int i = 0; i < n; ++i) { probs[i] = expf((logits[i] - mx) / temp); sum_exp += probs[i]; }
    for (int i = 0; i < n; ++i) probs[i] /= sum_exp;
    *seed = ggo_mt_next(&g);
    int pick = 0;
    if (n >= 2) {
        double sum = 0.0;
        for (int i = 0; i < n; ++i) sum += (double)probs[i];
        double run = 0.0;
        for (int i = 0; i < n; ++i) { run += (double)probs[i] / sum; cp[i] = run; }
        cp[n - 1] = 1.0;
        const double r1 = (double)ggo_mt_next(&g), r2 = (double)ggo_mt_next(&g);
        double u = (r1 + r2 * 4294967296.0) / 18446744073709551616.0;
        if (u >= 1.0) u = nextafter(1.0, 0.0);
        int lo = 0, hi = n;                      /* std::lower_bound: first cp[i] >= u */
        while (lo < hi) { const int mid = lo + (hi - lo) / 2; if (cp[mid] < u) lo = mid + 1; else hi = mid; }
        pick = lo;
    }
    free(probs); free(cp);
    return pick;
}

/* ---- generic (llama / qwen2 / qwen3) forward: src/cli/main.cpp:2367-2375,
 * 3235-3512, 3593-3599 ------------------------------------------------------ */

typedef struct { const uint8_t* data; uint32_t type; } ggo_weight;

typedef struct {
    ggo_weight attn_q, attn_k, attn_v, attn_o, ffn_gate, ffn_up, ffn_down;
    const float *attn_norm, *ffn_norm;          /* F32 [hidden] */
    const float *bq, *bk, *bv;                  /* optional F32 biases */
    const float *q_norm, *k_norm;               /* optional F32 [head_dim] */
    /* lfm2 gated short-convolution layer (present instead of attn_*): in_proj [3 hidden][hidden],
     * out_proj [hidden][hidden], conv F32 [hidden][taps] (tap-contiguous) */
    ggo_weight sc_in, sc_out;
    const float* sc_conv;
} ggo_layer;

typedef struct {
    int n_layer, hidden, n_head, n_kv, head_dim, ffn, vocab, ctx;
    int rope_neox;                               /* 1 for qwen3 */
    float rms_eps, rope_base, rope_scale;
    ggo_weight tok_embd, output;                 /* output = tok_embd when tied */
    const float* output_norm;
    const float* rope_ff; int n_rope_ff;
    const ggo_layer* layers;
    /* state owned by the model object */
    float *kcache, *vcache;                      /* [L][ctx][n_kv][hd], K post-RoPE (src/runtime/kv_cache.cpp:38-48) */
    float *rope_cos, *rope_sin;                  /* [ctx][hd/2] */
    /* lfm2 (src/cli/main.cpp:2145-2167, 2680-2856): taps of the short convolution, the state of every layer
     * [n_layer][taps - 1][hidden] (oldest first), and whether RoPE goes through the CPU backend's rope() */
    int lfm2, conv_taps, cpu_rope;
    float* conv_state;
} ggo_model;

GGO_API ggo_model* ggo_model_new(int n_layer, int hidden, int n_head, int n_kv, int head_dim, int ffn,
                                 int vocab, int ctx, float rms_eps, float rope_base, float rope_scale,
                                 int rope_neox) {
    ggo_model* m = (ggo_model*)calloc(1, sizeof(ggo_model));
    if (!m) return NULL;
    m->n_layer = n_layer; m->hidden = hidden; m->n_head = n_head; m->n_kv = n_kv; m->head_dim = head_dim;
    m->ffn = ffn; m->vocab = vocab; m->ctx = ctx; m->rms_eps = rms_eps; m->rope_base = rope_base;
    m->rope_scale = rope_scale; m->rope_neox = rope_neox;
    m->layers = (ggo_layer*)calloc((size_t)n_layer, sizeof(ggo_layer));
    const size_t kv = (size_t)n_layer * ctx * n_kv * head_dim;
    m->kcache = (float*)calloc(kv, sizeof(float));
    m->vcache = (float*)calloc(kv, sizeof(float));
    m->rope_cos = (float*)malloc(sizeof(float) * (size_t)ctx * (head_dim / 2));
    m->rope_sin = (float*)malloc(sizeof(float) * (size_t)ctx * (head_dim / 2));
    return m;
}

GGO_API void ggo_model_free(ggo_model* m) {
    if (!m) return;
    free((void*)m->layers); free(m->kcache); free(m->vcache); free(m->rope_cos); free(m->rope_sin); free(m->conv_state); free(m);
}

/* Switch the model to the lfm2 branch: per-head QK-norm through the backend's rms_norm (g_rmsnorm, :2231-2245),
 * final norm = token_embd_norm (pass it as output_norm), layers with sc_in set run the short convolution.
 * cpu_rope = 1 restates what the reference CLI does on its CPU backend: g_rope (:2250-2268) calls
 * Backend::rope_batched, whose default (include/ggnpu/backend.h:123-141) loops the CPU backend's rope()
 * (cpu_ref.cpp:158-174): adjacent pairs at base 10000, whatever freq_base and neox_split_half say.
 * cpu_rope = 0 is what the branch asks its backend for (split-half pairs at the model's base), from the table. */
GGO_API void ggo_model_set_lfm2(ggo_model* m, int conv_taps, int cpu_rope) {
    m->lfm2 = 1; m->conv_taps = conv_taps; m->cpu_rope = cpu_rope;
    free(m->conv_state);
    m->conv_state = (float*)calloc((size_t)m->n_layer * (size_t)(conv_taps > 1 ? conv_taps - 1 : 1) * m->hidden, sizeof(float));
}

/* A new sequence: the convolution states start at zero (lconv_state, :2159). */
GGO_API void ggo_model_reset_conv(ggo_model* m) {
    if (m->conv_state) memset(m->conv_state, 0, sizeof(float) * (size_t)m->n_layer * (size_t)(m->conv_taps > 1 ? m->conv_taps - 1 : 1) * m->hidden);
}

GGO_API void ggo_model_set_globals(ggo_model* m, const uint8_t* tok_embd, uint32_t tok_type,
                                   const uint8_t* output, uint32_t out_type, const float* output_norm,
                                   const float* rope_ff, int n_rope_ff) {
    m->tok_embd.data = tok_embd; m->tok_embd.type = tok_type;
    m->output.data = output ? output : tok_embd; m->output.type = output ? out_type : tok_type;
    m->output_norm = output_norm; m->rope_ff = rope_ff; m->n_rope_ff = n_rope_ff;
    /* head_dim-wide table built once per run (main.cpp:1272-1273) */
    ggo_rope_table(m->ctx, m->head_dim, m->rope_scale, m->rope_base, rope_ff, n_rope_ff, m->rope_cos, m->rope_sin);
}

/* which: 0 q,1 k,2 v,3 o,4 gate,5 up,6 down,7 shortconv in_proj,8 shortconv out_proj */
GGO_API void ggo_model_set_weight(ggo_model* m, int layer, int which, const uint8_t* data, uint32_t type) {
    ggo_layer* l = (ggo_layer*)&m->layers[layer];
    ggo_weight* w[9] = {&l->attn_q, &l->attn_k, &l->attn_v, &l->attn_o, &l->ffn_gate, &l->ffn_up, &l->ffn_down, &l->sc_in, &l->sc_out};
    w[which]->data = data; w[which]->type = type;
}

/* which: 0 attn_norm,1 ffn_norm,2 bq,3 bk,4 bv,5 q_norm,6 k_norm,7 shortconv conv */
GGO_API void ggo_model_set_vec(ggo_model* m, int layer, int which, const float* v) {
    ggo_layer* l = (ggo_layer*)&m->layers[layer];
    const float** p[8] = {&l->attn_norm, &l->ffn_norm, &l->bq, &l->bk, &l->bv, &l->q_norm, &l->k_norm, &l->sc_conv};
    *p[which] = v;
}

/* Mixture-of-experts FFN of one token, src/cli/main.cpp:3110-3193 (qwen35moe branch).
 * The reference keeps this block inside main(), so it cannot be called from the reference-built checker;
 * it is restated line by line from the cited source and pinned end to end through ggo_q35_forward against
 * the unmodified reference CLI's logits and greedy stream on synthetic qwen35moe models.
 *   router logits  :3117-3125  F32 [n_expert][hidden] . x, one running fp32 sum per expert
 *   top-k          :3128-3131  std::partial_sort by logit, descending (ties: unspecified there; lowest index here)
 *   weights        :3132-3135  exp(l - max) / sum over the k chosen
 *   expert e       :3140-3170  slice e of the 3-D tensors; act = silu(gate x) * up x; out = down act; moe += w * out
 *   shared expert  :3177-3191  the same with its own matrices, weight = sigmoid(gate_inp_shexp . x) (1 if absent)
 * x is the FFN-normed hidden row; moe_out (hidden floats) is what the caller adds to the residual stream.
 * Expert tensors: gate / up [n_expert][eff][hidden], down [n_expert][hidden][eff], GGUF rows of their type. */
GGO_API int ggo_moe_ffn(const float* x, int hidden, const float* router, int n_expert, int top_k, int eff,
                        const uint8_t* gate_exps, const uint8_t* up_exps, uint32_t type_gu,
                        const uint8_t* down_exps, uint32_t type_d,
                        const uint8_t* sh_gate, const uint8_t* sh_up, uint32_t sh_type_gu, const uint8_t* sh_down, uint32_t sh_type_d,
                        int eff_sh, const float* sh_gate_inp, float* moe_out, int32_t* sel_ids, float* sel_w) {
    if (top_k < 1 || top_k > n_expert) return -1;
    float* rl = (float*)malloc(sizeof(float) * (size_t)n_expert);
    char* used = (char*)calloc((size_t)n_expert, 1);
    int maxeff = eff > eff_sh ? eff : eff_sh;
    float* eg = (float*)malloc(sizeof(float) * (size_t)maxeff);
    float* eu = (float*)malloc(sizeof(float) * (size_t)maxeff);
    float* ea = (float*)malloc(sizeof(float) * (size_t)maxeff);
    float* ed = (float*)malloc(sizeof(float) * (size_t)hidden);
    int rc = 0;
    for (int e = 0; e < n_expert; ++e) {
        const float* wr = router + (size_t)e * hidden;
        float acc = 0.0f;
        for (int i = 0; i < hidden; ++i) acc += x[i] * wr[i];
        rl[e] = acc;
    }
    for (int j = 0; j < top_k; ++j) {
        int best = -1;
        for (int e = 0; e < n_expert; ++e)
            if (!used[e] && (best < 0 || rl[e] > rl[best])) best = e;
        used[best] = 1;
        sel_ids[j] = best;
    }
    {
        const float mx = rl[sel_ids[0]];
        float wsum = 0.0f;
        for (int j = 0; j < top_k; ++j) { sel_w[j] = expf(rl[sel_ids[j]] - mx); wsum += sel_w[j]; }
        for (int j = 0; j < top_k; ++j) sel_w[j] /= wsum;
    }
    for (int i = 0; i < hidden; ++i) moe_out[i] = 0.0f;
    const size_t gu_bytes = (size_t)eff * ((size_t)hidden / ggo_block_elems(type_gu)) * ggo_block_bytes(type_gu);
    const size_t d_bytes = (size_t)hidden * ((size_t)eff / ggo_block_elems(type_d)) * ggo_block_bytes(type_d);
    for (int j = 0; j <= top_k && rc == 0; ++j) {
        const uint8_t *g, *u, *d;
        uint32_t tgu, td;
        int f;
        float weight;
        if (j < top_k) {
            g = gate_exps + gu_bytes * sel_ids[j]; u = up_exps + gu_bytes * sel_ids[j]; d = down_exps + d_bytes * sel_ids[j];
            tgu = type_gu; td = type_d; f = eff; weight = sel_w[j];
        } else {
            if (!sh_gate || !sh_up || !sh_down) break;
            weight = 1.0f;
            if (sh_gate_inp) {
                float acc = 0.0f;
                for (int i = 0; i < hidden; ++i) acc += x[i] * sh_gate_inp[i];
                weight = 1.0f / (1.0f + expf(-acc));
            }
            sel_w[top_k] = weight;
            g = sh_gate; u = sh_up; d = sh_down; tgu = sh_type_gu; td = sh_type_d; f = eff_sh;
        }
        rc |= ggo_matmul_exact(x, 1, hidden, g, tgu, f, hidden, eg, f);
        rc |= ggo_matmul_exact(x, 1, hidden, u, tgu, f, hidden, eu, f);
        for (int i = 0; i < f; ++i) ea[i] = (eg[i] / (1.0f + expf(-eg[i]))) * eu[i];
        rc |= ggo_matmul_exact(ea, 1, f, d, td, hidden, f, ed, hidden);
        for (int i = 0; i < hidden; ++i) moe_out[i] += weight * ed[i];
    }
    free(rl); free(used); free(eg); free(eu); free(ea); free(ed);
    return rc;
}

/* One token of a Gated DeltaNet (linear attention) layer after its projections,
 * src/cli/main.cpp:2925-3023 (qwen35 / qwen35moe branch).  Pinned like ggo_moe_ffn: end to end through
 * ggo_q35_forward against the reference CLI (the reference keeps the block inside main()).
 *   conv      :2925-2941  causal depthwise conv1d (conv_k taps, newest = this token) + SiLU; the state
 *                         holds the previous conv_k - 1 inputs [tap][channel] and is rolled
 *   q, k      :2956-2968  per key head L2-normalised over sk (eps 1e-6); q also scaled by 1/sqrt(sk)
 *   per V head:2976-3011  key head = h % n_khead; beta = sigmoid(b); g = exp(ssm_a * softplus(a + dt_bias));
 *                         S *= g; pred = S^T k; delta = beta (v - pred); S += k (x) delta; o = S^T q
 *   output    :3016-3023  rms_norm(o) * ssm_norm * silu(z)
 * mixed = [q: n_khead*sk | k: n_khead*sk | v: n_vhead*sk] of this token (the attn_qkv projection). */
GGO_API int ggo_deltanet_step(const float* mixed, const float* zgate, const float* araw, const float* braw,
                              const float* conv_w, const float* ssm_a, const float* dt_bias, const float* ssm_norm,
                              float* conv_state, float* rec_state, float* out,
                              int n_khead, int n_vhead, int sk, int conv_k, float rms_eps) {
    const int key_dim = n_khead * sk, value_dim = n_vhead * sk, conv_dim = 2 * key_dim + value_dim, ckm1 = conv_k - 1;
    float* conv = (float*)malloc(sizeof(float) * (size_t)conv_dim);
    float* qn = (float*)malloc(sizeof(float) * (size_t)key_dim);
    float* kn = (float*)malloc(sizeof(float) * (size_t)key_dim);
    float* pred = (float*)malloc(sizeof(float) * (size_t)sk);
    float* delta = (float*)malloc(sizeof(float) * (size_t)sk);
    float* oh = (float*)malloc(sizeof(float) * (size_t)sk);
    for (int ch = 0; ch < conv_dim; ++ch) {
        float acc = conv_w[ch * conv_k + ckm1] * mixed[ch];
        for (int t = 0; t < ckm1; ++t) acc += conv_w[ch * conv_k + t] * conv_state[(size_t)t * conv_dim + ch];
        conv[ch] = acc / (1.0f + expf(-acc));
        for (int t = 0; t < ckm1 - 1; ++t) conv_state[(size_t)t * conv_dim + ch] = conv_state[(size_t)(t + 1) * conv_dim + ch];
        if (ckm1 > 0) conv_state[(size_t)(ckm1 - 1) * conv_dim + ch] = mixed[ch];
    }
    const float *qc = conv, *kc = conv + key_dim, *vc = conv + 2 * key_dim;
    for (int h = 0; h < n_khead; ++h) {
        const float *qh = qc + h * sk, *kh = kc + h * sk;
        float sq = 0.0f, s2 = 0.0f;
        for (int i = 0; i < sk; ++i) { sq += qh[i] * qh[i]; s2 += kh[i] * kh[i]; }
        const float rq = (1.0f / sqrtf(sq + 1e-6f)) / sqrtf((float)sk);
        const float rk = 1.0f / sqrtf(s2 + 1e-6f);
        for (int i = 0; i < sk; ++i) { qn[h * sk + i] = qh[i] * rq; kn[h * sk + i] = kh[i] * rk; }
    }
    for (int h = 0; h < n_vhead; ++h) {
        const int kh = h % n_khead;
        const float *qh = qn + kh * sk, *khp = kn + kh * sk, *vh = vc + h * sk;
        const float beta = 1.0f / (1.0f + expf(-braw[h]));
        const float a = araw[h] + dt_bias[h];
        const float sp = (a > 20.0f) ? a : log1pf(expf(a));
        const float g = expf(ssm_a[h] * sp);
        float* Sh = rec_state + (size_t)h * sk * sk;
        for (int v = 0; v < sk; ++v) { pred[v] = 0.0f; oh[v] = 0.0f; }
        for (int kk = 0; kk < sk; ++kk) {
            const float kval = khp[kk];
            float* row = Sh + (size_t)kk * sk;
            for (int v = 0; v < sk; ++v) { row[v] *= g; pred[v] += row[v] * kval; }
        }
        for (int v = 0; v < sk; ++v) delta[v] = beta * (vh[v] - pred[v]);
        for (int kk = 0; kk < sk; ++kk) {
            const float kval = khp[kk], qval = qh[kk];
            float* row = Sh + (size_t)kk * sk;
            for (int v = 0; v < sk; ++v) { row[v] += kval * delta[v]; oh[v] += row[v] * qval; }
        }
        const float* zh = zgate + h * sk;
        float ss = 0.0f;
        for (int v = 0; v < sk; ++v) ss += oh[v] * oh[v];
        const float r = 1.0f / sqrtf(ss / (float)sk + rms_eps);
        float* od = out + h * sk;
        for (int v = 0; v < sk; ++v) od[v] = (oh[v] * r * ssm_norm[v]) * (zh[v] / (1.0f + expf(-zh[v])));
    }
    free(conv); free(qn); free(kn); free(pred); free(delta); free(oh);
    return 0;
}

/* One forward over n_tok tokens at absolute positions pos..pos+n_tok-1,
 * writing the KV cache and (if logits != NULL) the logits of the LAST row
 * (main.cpp:3593-3598).  Matmuls follow the exact path (ggo_matmul_exact).
 * hidden_out (optional) receives the final-normed hidden rows [n_tok][hidden]. */
GGO_API int ggo_forward(ggo_model* m, const int32_t* tokens, int n_tok, int pos, float* logits, float* hidden_out) {
    const int H = m->hidden, hd = m->head_dim, qd = m->n_head * hd, kvd = m->n_kv * hd, F = m->ffn;
    if (pos + n_tok > m->ctx) return -1;
    const size_t T = (size_t)n_tok;
    float* x = (float*)malloc(sizeof(float) * T * H);
    float* xn = (float*)malloc(sizeof(float) * T * H);
    float* q = (float*)malloc(sizeof(float) * T * qd);
    float* k = (float*)malloc(sizeof(float) * T * kvd);
    float* v = (float*)malloc(sizeof(float) * T * kvd);
    float* qr = (float*)malloc(sizeof(float) * T * qd);
    float* kr = (float*)malloc(sizeof(float) * T * kvd);
    float* att = (float*)malloc(sizeof(float) * T * qd);
    float* proj = (float*)malloc(sizeof(float) * T * H);
    float* g = (float*)malloc(sizeof(float) * T * F);
    float* u = (float*)malloc(sizeof(float) * T * F);
    const int64_t ctx_len = pos + n_tok;
    float* kexp = (float*)malloc(sizeof(float) * (size_t)m->n_head * ctx_len * hd);
    float* vexp = (float*)malloc(sizeof(float) * (size_t)m->n_head * ctx_len * hd);
    const int grp = m->n_head / m->n_kv;

    for (int t = 0; t < n_tok; ++t) ggo_dequant_row(m->tok_embd.type, m->tok_embd.data, tokens[t], H, x + (size_t)t * H);

    for (int L = 0; L < m->n_layer; ++L) {
        const ggo_layer* l = &m->layers[L];
        for (int t = 0; t < n_tok; ++t) ggo_rms_norm(x + (size_t)t * H, xn + (size_t)t * H, H, m->rms_eps, l->attn_norm);
        if (m->lfm2 && l->sc_in.data) {
            /* gated short convolution, main.cpp:2693-2732: bcx = in_proj(xn) = [B | C | x]; bx = B * x; depthwise causal
             * conv over the last `taps` values of bx (newest = this token); y = C * conv; out_proj(y) joins the residual.
             * Tokens in order: the state of the layer carries from one to the next. */
            const int taps = m->conv_taps, dcm1 = taps - 1;
            float* bcx = (float*)malloc(sizeof(float) * T * 3 * H);
            float* yc = (float*)malloc(sizeof(float) * T * H);
            float* st = m->conv_state + (size_t)L * (size_t)(dcm1 > 0 ? dcm1 : 1) * H;
            ggo_matmul_exact(xn, n_tok, H, l->sc_in.data, l->sc_in.type, 3 * H, H, bcx, 3 * H);
            for (int t = 0; t < n_tok; ++t) {
                const float *b = bcx + (size_t)t * 3 * H, *c = b + H, *xx = b + 2 * H;
                for (int ch = 0; ch < H; ++ch) {
                    const float bx = b[ch] * xx[ch];
                    float acc = l->sc_conv[ch * taps + dcm1] * bx;
                    for (int kk = 0; kk < dcm1; ++kk) acc += l->sc_conv[ch * taps + kk] * st[(size_t)kk * H + ch];
                    yc[(size_t)t * H + ch] = c[ch] * acc;
                    for (int kk = 0; kk < dcm1 - 1; ++kk) st[(size_t)kk * H + ch] = st[(size_t)(kk + 1) * H + ch];
                    if (dcm1 > 0) st[(size_t)(dcm1 - 1) * H + ch] = bx;
                }
            }
            ggo_matmul_exact(yc, n_tok, H, l->sc_out.data, l->sc_out.type, H, H, proj, H);
            for (size_t i = 0; i < T * H; ++i) x[i] += proj[i];
            free(bcx); free(yc);
            goto ffn;
        }
        ggo_matmul_exact(xn, n_tok, H, l->attn_q.data, l->attn_q.type, qd, H, q, qd);
        ggo_matmul_exact(xn, n_tok, H, l->attn_k.data, l->attn_k.type, kvd, H, k, kvd);
        ggo_matmul_exact(xn, n_tok, H, l->attn_v.data, l->attn_v.type, kvd, H, v, kvd);
        for (int t = 0; t < n_tok; ++t) {                         /* main.cpp:3274-3284 */
            if (l->bq) for (int j = 0; j < qd; ++j) q[(size_t)t * qd + j] += l->bq[j];
            if (l->bk) for (int j = 0; j < kvd; ++j) k[(size_t)t * kvd + j] += l->bk[j];
            if (l->bv) for (int j = 0; j < kvd; ++j) v[(size_t)t * kvd + j] += l->bv[j];
        }
        for (int t = 0; t < n_tok; ++t) {                         /* main.cpp:3289-3312 */
            if (m->lfm2) {                                        /* main.cpp:2756-2761: the backend's rms_norm, in place */
                if (l->q_norm) for (int h = 0; h < m->n_head; ++h) { float* p = q + (size_t)t * qd + (size_t)h * hd; ggo_rms_norm(p, p, hd, m->rms_eps, l->q_norm); }
                if (l->k_norm) for (int h = 0; h < m->n_kv; ++h) { float* p = k + (size_t)t * kvd + (size_t)h * hd; ggo_rms_norm(p, p, hd, m->rms_eps, l->k_norm); }
                continue;
            }
            if (l->q_norm) for (int h = 0; h < m->n_head; ++h) ggo_rms_norm_head_f64(q + (size_t)t * qd + (size_t)h * hd, hd, m->rms_eps, l->q_norm);
            if (l->k_norm) for (int h = 0; h < m->n_kv; ++h) ggo_rms_norm_head_f64(k + (size_t)t * kvd + (size_t)h * hd, hd, m->rms_eps, l->k_norm);
        }
        for (int t = 0; t < n_tok; ++t) {                         /* main.cpp:3314-3351 */
            const float* c = m->rope_cos + (size_t)(pos + t) * (hd / 2);
            const float* s = m->rope_sin + (size_t)(pos + t) * (hd / 2);
            if (m->lfm2 && m->cpu_rope) {                         /* main.cpp:2762-2763 on the CPU backend */
                memcpy(qr + (size_t)t * qd, q + (size_t)t * qd, sizeof(float) * qd);
                memcpy(kr + (size_t)t * kvd, k + (size_t)t * kvd, sizeof(float) * kvd);
                for (int h = 0; h < m->n_head; ++h) ggo_rope_cpu_ref(qr + (size_t)t * qd + (size_t)h * hd, hd, pos + t, 1.0f, hd);
                for (int h = 0; h < m->n_kv; ++h) ggo_rope_cpu_ref(kr + (size_t)t * kvd + (size_t)h * hd, hd, pos + t, 1.0f, hd);
                continue;
            }
            ggo_rope_apply(qr + (size_t)t * qd, q + (size_t)t * qd, m->n_head, hd, hd, c, s, m->rope_neox);
            ggo_rope_apply(kr + (size_t)t * kvd, k + (size_t)t * kvd, m->n_kv, hd, hd, c, s, m->rope_neox);
        }
        /* KV write, src/runtime/kv_cache.cpp:76-104 */
        float* kc = m->kcache + (size_t)L * m->ctx * kvd;
        float* vc = m->vcache + (size_t)L * m->ctx * kvd;
        memcpy(kc + (size_t)pos * kvd, kr, sizeof(float) * T * kvd);
        memcpy(vc + (size_t)pos * kvd, v, sizeof(float) * T * kvd);
        /* GQA expand, main.cpp:3364-3383 */
        for (int h = 0; h < m->n_head; ++h)
            for (int64_t j = 0; j < ctx_len; ++j) {
                memcpy(kexp + ((size_t)h * ctx_len + j) * hd, kc + (size_t)j * kvd + (size_t)(h / grp) * hd, sizeof(float) * hd);
                memcpy(vexp + ((size_t)h * ctx_len + j) * hd, vc + (size_t)j * kvd + (size_t)(h / grp) * hd, sizeof(float) * hd);
            }
        for (int t = 0; t < n_tok; ++t)                           /* main.cpp:3393-3410 */
            ggo_flash_attn(qr + (size_t)t * qd, kexp, vexp, att + (size_t)t * qd, m->n_head, hd, ctx_len, pos + t);
        ggo_matmul_exact(att, n_tok, qd, l->attn_o.data, l->attn_o.type, H, qd, proj, H);
        for (size_t i = 0; i < T * H; ++i) x[i] += proj[i];
    ffn:
        for (int t = 0; t < n_tok; ++t) ggo_rms_norm(x + (size_t)t * H, xn + (size_t)t * H, H, m->rms_eps, l->ffn_norm);
        ggo_matmul_exact(xn, n_tok, H, l->ffn_gate.data, l->ffn_gate.type, F, H, g, F);
        ggo_matmul_exact(xn, n_tok, H, l->ffn_up.data, l->ffn_up.type, F, H, u, F);
        for (int t = 0; t < n_tok; ++t) {                         /* main.cpp:3461-3479 */
            ggo_silu(g + (size_t)t * F, g + (size_t)t * F, F);
            for (int i = 0; i < F; ++i) g[(size_t)t * F + i] *= u[(size_t)t * F + i];
        }
        ggo_matmul_exact(g, n_tok, F, l->ffn_down.data, l->ffn_down.type, H, F, proj, H);
        for (size_t i = 0; i < T * H; ++i) x[i] += proj[i];
    }
    for (int t = 0; t < n_tok; ++t) ggo_rms_norm(x + (size_t)t * H, xn + (size_t)t * H, H, m->rms_eps, m->output_norm);
    if (hidden_out) memcpy(hidden_out, xn, sizeof(float) * T * H);
    if (logits) ggo_matmul_exact(xn + (T - 1) * H, 1, H, m->output.data, m->output.type, m->vocab, H, logits, m->vocab);
    free(x); free(xn); free(q); free(k); free(v); free(qr); free(kr); free(att); free(proj); free(g); free(u);
    free(kexp); free(vexp);
    return 0;
}

/* Read access to the oracle KV cache row (layer, position): [n_kv][hd]. */
GGO_API const float* ggo_model_kv(const ggo_model* m, int layer, int pos, int want_v) {
    const size_t kvd = (size_t)m->n_kv * m->head_dim;
    return (want_v ? m->vcache : m->kcache) + ((size_t)layer * m->ctx + pos) * kvd;
}

/* ---- qwen35 / qwen35moe forward: src/cli/main.cpp:2859-3232 -------------------------------------
 * One token per call, as the reference runs this architecture (no prompt batching, main.cpp:2327).
 * Per layer: attn_norm -> Gated DeltaNet mixer (layers that have ssm_conv1d, :2900-3034, restated in
 * ggo_deltanet_step) or gated full attention (:3035-3105) -> residual -> post_attention_norm ->
 * MoE FFN (:3110-3193, restated in ggo_moe_ffn) -> residual; then output_norm and logits (:3504-3512,
 * :3593-3598).  Every matmul is the exact path (M == 1 under GGNPU_FP32_MATMUL, :1379-1388), F32
 * weights included (ssm_alpha / ssm_beta).
 * Parity of this block (and through it of ggo_moe_ffn and ggo_deltanet_step) is pinned by the
 * unmodified reference CLI's top-10 logits and greedy stream on a synthetic qwen35moe GGUF
 * (tests/golden/ref_cli.npz, written by tests/golden/make_golden.py). */

typedef struct {
    int is_ssm;
    const float *attn_norm, *post_norm;
    /* DeltaNet layers */
    ggo_weight qkv, zgate, alpha, beta, ssm_out;
    const float *conv_w, *ssm_a, *dt_bias, *ssm_norm;
    float *conv_state, *rec_state;
    /* full-attention layers */
    ggo_weight q, k, v, o;
    const float *q_norm, *k_norm;
    float *k_store, *v_store;                   /* [ctx][n_kv * head_dim], K after norm + RoPE (main.cpp:3070-3071) */
    /* MoE FFN */
    const float* router;
    ggo_weight gate_exps, up_exps, down_exps, sh_gate, sh_up, sh_down;
    const float* sh_gate_inp;
} ggo_q35_layer;

typedef struct {
    int n_layer, hidden, n_head, n_kv, head_dim, rope_dim, conv_k, sk, n_vhead, n_khead, n_expert, top_k, eff, vocab, ctx;
    float rms_eps, rope_base;
    ggo_weight tok_embd, output;
    const float* output_norm;
    ggo_q35_layer* layers;
} ggo_q35_model;

GGO_API ggo_q35_model* ggo_q35_new(int n_layer, int hidden, int n_head, int n_kv, int head_dim, int rope_dim, int conv_k,
                                   int sk, int n_vhead, int n_khead, int n_expert, int top_k, int eff, int vocab, int ctx,
                                   float rms_eps, float rope_base) {
    ggo_q35_model* m = (ggo_q35_model*)calloc(1, sizeof(ggo_q35_model));
    if (!m) return NULL;
    m->n_layer = n_layer; m->hidden = hidden; m->n_head = n_head; m->n_kv = n_kv; m->head_dim = head_dim; m->rope_dim = rope_dim;
    m->conv_k = conv_k; m->sk = sk; m->n_vhead = n_vhead; m->n_khead = n_khead; m->n_expert = n_expert; m->top_k = top_k;
    m->eff = eff; m->vocab = vocab; m->ctx = ctx; m->rms_eps = rms_eps; m->rope_base = rope_base;
    m->layers = (ggo_q35_layer*)calloc((size_t)n_layer, sizeof(ggo_q35_layer));
    return m;
}

GGO_API void ggo_q35_free(ggo_q35_model* m) {
    if (!m) return;
    for (int l = 0; l < m->n_layer; ++l) {
        free(m->layers[l].conv_state); free(m->layers[l].rec_state); free(m->layers[l].k_store); free(m->layers[l].v_store);
    }
    free(m->layers); free(m);
}

GGO_API void ggo_q35_set_globals(ggo_q35_model* m, const uint8_t* tok_embd, uint32_t tok_type, const uint8_t* output,
                                 uint32_t out_type, const float* output_norm) {
    m->tok_embd.data = tok_embd; m->tok_embd.type = tok_type;
    m->output.data = output ? output : tok_embd; m->output.type = output ? out_type : tok_type;   /* main.cpp:2065-2067 */
    m->output_norm = output_norm;
}

/* A layer is a DeltaNet layer iff it has ssm_conv1d.weight (main.cpp:2207-2213). */
GGO_API void ggo_q35_set_kind(ggo_q35_model* m, int layer, int is_ssm) {
    ggo_q35_layer* l = &m->layers[layer];
    l->is_ssm = is_ssm;
    const size_t conv_dim = (size_t)2 * m->n_khead * m->sk + (size_t)m->n_vhead * m->sk;
    if (is_ssm) {
        l->conv_state = (float*)calloc((size_t)(m->conv_k - 1) * conv_dim + 1, sizeof(float));
        l->rec_state = (float*)calloc((size_t)m->n_vhead * m->sk * m->sk, sizeof(float));
    } else {
        l->k_store = (float*)calloc((size_t)m->ctx * m->n_kv * m->head_dim, sizeof(float));
        l->v_store = (float*)calloc((size_t)m->ctx * m->n_kv * m->head_dim, sizeof(float));
    }
}

/* which: 0 attn_qkv, 1 attn_gate, 2 ssm_alpha, 3 ssm_beta, 4 ssm_out, 5 attn_q, 6 attn_k, 7 attn_v, 8 attn_output,
 *        9 ffn_gate_exps, 10 ffn_up_exps, 11 ffn_down_exps, 12 ffn_gate_shexp, 13 ffn_up_shexp, 14 ffn_down_shexp */
GGO_API void ggo_q35_set_weight(ggo_q35_model* m, int layer, int which, const uint8_t* data, uint32_t type) {
    ggo_q35_layer* l = &m->layers[layer];
    ggo_weight* w[15] = {&l->qkv, &l->zgate, &l->alpha, &l->beta, &l->ssm_out, &l->q, &l->k, &l->v, &l->o,
                         &l->gate_exps, &l->up_exps, &l->down_exps, &l->sh_gate, &l->sh_up, &l->sh_down};
    w[which]->data = data; w[which]->type = type;
}

/* which: 0 attn_norm, 1 post_attention_norm, 2 ssm_conv1d, 3 ssm_a, 4 ssm_dt.bias, 5 ssm_norm, 6 attn_q_norm,
 *        7 attn_k_norm, 8 ffn_gate_inp (router), 9 ffn_gate_inp_shexp */
GGO_API void ggo_q35_set_vec(ggo_q35_model* m, int layer, int which, const float* v) {
    ggo_q35_layer* l = &m->layers[layer];
    const float** p[10] = {&l->attn_norm, &l->post_norm, &l->conv_w, &l->ssm_a, &l->dt_bias, &l->ssm_norm, &l->q_norm,
                           &l->k_norm, &l->router, &l->sh_gate_inp};
    *p[which] = v;
}

/* src/cli/main.cpp:896-901 (host_rmsnorm): sum of squares in float. */
static void q35_host_rmsnorm(float* dst, const float* src, int n, const float* w, float eps) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += src[i] * src[i];
    const float r = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; ++i) dst[i] = src[i] * r * (w ? w[i] : 1.0f);
}

/* src/cli/main.cpp:906-920 (rope_neox_partial): theta = pos * base^(-2i/rope_dim) in float, pairs (i, i + rope_dim/2). */
static void q35_rope_neox_partial(float* vec, int n_heads, int head_dim, int rope_dim, int64_t pos, float base) {
    const int half = rope_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        float* p = vec + (size_t)h * head_dim;
        for (int i = 0; i < half; ++i) {
            const float theta = (float)pos * powf(base, -2.0f * (float)i / (float)rope_dim);
            const float c = cosf(theta), s = sinf(theta);
            const float x0 = p[i], x1 = p[i + half];
            p[i] = x0 * c - x1 * s;
            p[i + half] = x0 * s + x1 * c;
        }
    }
}

/* The cos / sin rows the device path uploads, computed exactly as q35_rope_neox_partial does. */
GGO_API void ggo_q35_rope_table(int64_t max_pos, int rope_dim, float base, float* cos_out, float* sin_out) {
    const int half = rope_dim / 2;
    for (int64_t p = 0; p < max_pos; ++p)
        for (int i = 0; i < half; ++i) {
            const float theta = (float)p * powf(base, -2.0f * (float)i / (float)rope_dim);
            cos_out[p * half + i] = cosf(theta);
            sin_out[p * half + i] = sinf(theta);
        }
}

/* One token at position pos.  logits (optional) [vocab]; hidden_out (optional) the final-normed row. */
GGO_API int ggo_q35_forward(ggo_q35_model* m, int32_t token, int pos, float* logits, float* hidden_out) {
    const int H = m->hidden, Hd = m->head_dim, nQ = m->n_head, nKV = m->n_kv, qdim = nQ * Hd, kvdim = nKV * Hd;
    const int sk = m->sk, nVH = m->n_vhead, nKH = m->n_khead, key_dim = nKH * sk, value_dim = nVH * sk, conv_dim = 2 * key_dim + value_dim;
    if (pos < 0 || pos >= m->ctx) return -1;
    int rc = 0;
    float* x = (float*)malloc(sizeof(float) * (size_t)H);
    float* xn = (float*)malloc(sizeof(float) * (size_t)H);
    float* mixed = (float*)malloc(sizeof(float) * (size_t)conv_dim);
    float* zgate = (float*)malloc(sizeof(float) * (size_t)value_dim);
    float* araw = (float*)malloc(sizeof(float) * (size_t)nVH);
    float* braw = (float*)malloc(sizeof(float) * (size_t)nVH);
    float* o_all = (float*)malloc(sizeof(float) * (size_t)value_dim);
    float* proj = (float*)malloc(sizeof(float) * (size_t)H);
    float* qg = (float*)malloc(sizeof(float) * (size_t)2 * qdim);
    float* q = (float*)malloc(sizeof(float) * (size_t)qdim);
    float* fgate = (float*)malloc(sizeof(float) * (size_t)qdim);
    float* kbuf = (float*)malloc(sizeof(float) * (size_t)kvdim);
    float* vbuf = (float*)malloc(sizeof(float) * (size_t)kvdim);
    float* attn_in = (float*)malloc(sizeof(float) * (size_t)qdim);
    const int64_t ctx_len = (int64_t)pos + 1;
    float* kexp = (float*)malloc(sizeof(float) * (size_t)nQ * ctx_len * Hd);
    float* vexp = (float*)malloc(sizeof(float) * (size_t)nQ * ctx_len * Hd);
    int32_t sel_ids[64]; float sel_w[65];

    ggo_dequant_row(m->tok_embd.type, m->tok_embd.data, token, H, x);               /* main.cpp:2367-2375 */
    for (int L = 0; L < m->n_layer && rc == 0; ++L) {
        ggo_q35_layer* l = &m->layers[L];
        ggo_rms_norm(x, xn, H, m->rms_eps, l->attn_norm);                            /* :2896 */
        if (l->is_ssm) {
            rc |= ggo_matmul_exact(xn, 1, H, l->qkv.data, l->qkv.type, conv_dim, H, mixed, conv_dim);      /* :2916-2923 */
            rc |= ggo_matmul_exact(xn, 1, H, l->zgate.data, l->zgate.type, value_dim, H, zgate, value_dim);
            rc |= ggo_matmul_exact(xn, 1, H, l->alpha.data, l->alpha.type, nVH, H, araw, nVH);
            rc |= ggo_matmul_exact(xn, 1, H, l->beta.data, l->beta.type, nVH, H, braw, nVH);
            rc |= ggo_deltanet_step(mixed, zgate, araw, braw, l->conv_w, l->ssm_a, l->dt_bias, l->ssm_norm, l->conv_state,
                                    l->rec_state, o_all, nKH, nVH, sk, m->conv_k, m->rms_eps);             /* :2925-3024 */
            rc |= ggo_matmul_exact(o_all, 1, value_dim, l->ssm_out.data, l->ssm_out.type, H, value_dim, proj, H);   /* :3028 */
            for (int i = 0; i < H; ++i) x[i] += proj[i];                             /* :3033 */
        } else {
            rc |= ggo_matmul_exact(xn, 1, H, l->q.data, l->q.type, 2 * qdim, H, qg, 2 * qdim);             /* :3047-3052 */
            rc |= ggo_matmul_exact(xn, 1, H, l->k.data, l->k.type, kvdim, H, kbuf, kvdim);
            rc |= ggo_matmul_exact(xn, 1, H, l->v.data, l->v.type, kvdim, H, vbuf, kvdim);
            for (int h = 0; h < nQ; ++h) {                                            /* :3056-3060 */
                memcpy(q + (size_t)h * Hd, qg + (size_t)h * 2 * Hd, sizeof(float) * Hd);
                memcpy(fgate + (size_t)h * Hd, qg + (size_t)h * 2 * Hd + Hd, sizeof(float) * Hd);
            }
            for (int h = 0; h < nQ; ++h) q35_host_rmsnorm(q + (size_t)h * Hd, q + (size_t)h * Hd, Hd, l->q_norm, m->rms_eps);      /* :3063-3066 */
            for (int h = 0; h < nKV; ++h) q35_host_rmsnorm(kbuf + (size_t)h * Hd, kbuf + (size_t)h * Hd, Hd, l->k_norm, m->rms_eps);
            q35_rope_neox_partial(q, nQ, Hd, m->rope_dim, pos, m->rope_base);        /* :3067-3068 */
            q35_rope_neox_partial(kbuf, nKV, Hd, m->rope_dim, pos, m->rope_base);
            memcpy(l->k_store + (size_t)pos * kvdim, kbuf, sizeof(float) * kvdim);   /* :3070-3071 */
            memcpy(l->v_store + (size_t)pos * kvdim, vbuf, sizeof(float) * kvdim);
            const int group = nQ / nKV;                                               /* :3073-3086 */
            for (int h = 0; h < nQ; ++h)
                for (int64_t j = 0; j < ctx_len; ++j) {
                    memcpy(kexp + ((size_t)h * ctx_len + j) * Hd, l->k_store + ((size_t)j * nKV + h / group) * Hd, sizeof(float) * Hd);
                    memcpy(vexp + ((size_t)h * ctx_len + j) * Hd, l->v_store + ((size_t)j * nKV + h / group) * Hd, sizeof(float) * Hd);
                }
            rc |= ggo_flash_attn(q, kexp, vexp, attn_in, nQ, Hd, ctx_len, pos);      /* :3088-3096 */
            for (int i = 0; i < qdim; ++i) attn_in[i] *= 1.0f / (1.0f + expf(-fgate[i]));                   /* :3098 */
            rc |= ggo_matmul_exact(attn_in, 1, qdim, l->o.data, l->o.type, H, qdim, proj, H);               /* :3100 */
            for (int i = 0; i < H; ++i) x[i] += proj[i];                             /* :3104 */
        }
        ggo_rms_norm(x, xn, H, m->rms_eps, l->post_norm);                            /* :3109 */
        rc |= ggo_moe_ffn(xn, H, l->router, m->n_expert, m->top_k, m->eff, l->gate_exps.data, l->up_exps.data, l->gate_exps.type,
                          l->down_exps.data, l->down_exps.type, l->sh_gate.data, l->sh_up.data, l->sh_gate.type, l->sh_down.data,
                          l->sh_down.type, m->eff, l->sh_gate_inp, proj, sel_ids, sel_w);                  /* :3110-3192 */
        for (int i = 0; i < H; ++i) x[i] += proj[i];                                 /* :3193 */
    }
    ggo_rms_norm(x, xn, H, m->rms_eps, m->output_norm);                              /* :3504-3512 */
    if (hidden_out) memcpy(hidden_out, xn, sizeof(float) * (size_t)H);
    if (logits && rc == 0) rc |= ggo_matmul_exact(xn, 1, H, m->output.data, m->output.type, m->vocab, H, logits, m->vocab);
    free(x); free(xn); free(mixed); free(zgate); free(araw); free(braw); free(o_all); free(proj); free(qg); free(q); free(fgate);
    free(kbuf); free(vbuf); free(attn_in); free(kexp); free(vexp);
    return rc;
}

/* Read access for tests: the K or V row [n_kv][head_dim] a full-attention layer stored at `pos`; the recurrent state
 * [n_vhead][sk][sk] of a DeltaNet layer. */
GGO_API const float* ggo_q35_kv(const ggo_q35_model* m, int layer, int pos, int want_v) {
    const ggo_q35_layer* l = &m->layers[layer];
    if (l->is_ssm) return NULL;
    return (want_v ? l->v_store : l->k_store) + (size_t)pos * m->n_kv * m->head_dim;
}
GGO_API const float* ggo_q35_rec_state(const ggo_q35_model* m, int layer) { return m->layers[layer].rec_state; }
