// Dequant-fused GEMV for decode (M <= a few rows): y[M][N] = x[M][K] * W[N][K]^T with W in
// the packed stream layout of ggb_formats.cuh.  Replaces the M==1 path of mul_mat_weight
// (src/cli/main.cpp:1379-1388) and CpuRefBackend::mul_mat_q (src/backends/cpu_ref/cpu_ref.cpp:25-137).
//
// Shape of the kernel (HBM-bound; every weight byte is read exactly once):
//   * the activation rows are staged once per CTA into shared memory (optionally RMS-normalised
//     on the way: the fused form of src/backends/cpu_ref/cpu_ref.cpp:139-156), in a bank-swizzled
//     order so that the 16-byte reads below are conflict free for every format;
//   * a warp owns RW consecutive weight rows; lane u owns "unit" u, u+32, ... of each row, a unit
//     being the weights covered by one 16-byte load of the quant stream (32 or 64 weights);
//     consecutive lanes read consecutive 16-byte words, so every warp load is one or more full
//     128-byte lines;
//   * the lane keeps the unit's activations in registers and reuses them for its RW rows, so
//     shared-memory traffic is 4/RW bytes per weight;
//   * products are accumulated in fp32 on integer quant values, the block scales are applied per
//     sub-block (d*sc*sum(x*q) - dmin*m*sum(x)), which differs from dequantise-then-dot only by
//     fp32 summation order.
#include <stdlib.h>

#include "ggb_internal.h"

namespace ggb {

// ---- shared-memory swizzle -------------------------------------------------------------------
// float4 index k4 -> k4 ^ m(k4 >> 3): permutes inside aligned groups of 8 float4 (128 bytes).
// The three mask bits are chosen so that the 8 lanes of a quarter warp hit 8 different 16-byte
// bank groups for the access pattern of every format (see the per-format unit maps below).
__device__ __forceinline__ int swz_mask(int k4) {
    const int b3 = (k4 >> 3) & 1, b4 = (k4 >> 4) & 1, b5 = (k4 >> 5) & 1, b6 = (k4 >> 6) & 1;
    return (b3 ^ b4 ^ b6) | (b5 << 1) | (b3 << 2);
}
__device__ __forceinline__ int swz4(int k4) { return k4 ^ swz_mask(k4); }

// 16 consecutive activations x[k0 .. k0+15], k0 a multiple of 16.
__device__ __forceinline__ void load_run16(const float4* __restrict__ xs, int k0, float (&x)[16]) {
    const int base = swz4(k0 >> 2);          // bits 0,1 of k0>>2 are zero, so ^i enumerates the run
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 v = xs[base ^ i];
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
}
__device__ __forceinline__ void load_run8(const float4* __restrict__ xs, int k0, float (&x)[8]) {
    const int base = swz4(k0 >> 2);          // k0 multiple of 8
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float4 v = xs[base ^ i];
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
}
__device__ __forceinline__ float sum16(const float (&x)[16]) {
    float s0 = (x[0] + x[1]) + (x[2] + x[3]), s1 = (x[4] + x[5]) + (x[6] + x[7]);
    float s2 = (x[8] + x[9]) + (x[10] + x[11]), s3 = (x[12] + x[13]) + (x[14] + x[15]);
    return (s0 + s1) + (s2 + s3);
}

// byte i of w as an exact float: one byte-permute builds 2^23 + b in the mantissa.
__device__ __forceinline__ float bytef(uint32_t w, int i) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 + i)) - 8388608.0f;
}
// sum_{l<16} x[l] * byte_l(q) for a 16-byte vector of small unsigned values
__device__ __forceinline__ float dot16_bytes(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, const float (&x)[16]) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) s = fmaf(x[i], bytef(w0, i), s);
#pragma unroll
    for (int i = 0; i < 4; ++i) s = fmaf(x[4 + i], bytef(w1, i), s);
#pragma unroll
    for (int i = 0; i < 4; ++i) s = fmaf(x[8 + i], bytef(w2, i), s);
#pragma unroll
    for (int i = 0; i < 4; ++i) s = fmaf(x[12 + i], bytef(w3, i), s);
    return s;
}
__device__ __forceinline__ float dot16_lo(const uint4& q, const float (&x)[16]) {
    return dot16_bytes(q.x & 0x0F0F0F0Fu, q.y & 0x0F0F0F0Fu, q.z & 0x0F0F0F0Fu, q.w & 0x0F0F0F0Fu, x);
}
__device__ __forceinline__ float dot16_hi(const uint4& q, const float (&x)[16]) {
    return dot16_bytes((q.x >> 4) & 0x0F0F0F0Fu, (q.y >> 4) & 0x0F0F0F0Fu, (q.z >> 4) & 0x0F0F0F0Fu,
                       (q.w >> 4) & 0x0F0F0F0Fu, x);
}
__device__ __forceinline__ uint4 ldg16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float ldg_f16(const uint8_t* p) {
    return f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p)));
}
__device__ __forceinline__ uint32_t word_byte(uint32_t w, int i) { return (w >> (8 * i)) & 0xFFu; }

// ---- per-format units --------------------------------------------------------------------------
// Every format provides:
//   UNIT           weights per unit
//   struct Raw     what one lane loads from HBM for one (row, unit)
//   struct X       the unit's activations (and their sub-block sums where the format has mins)
//   load(w, rb, u) rb = row * blocks-per-row
//   load_x(xs, u)
//   dot(raw, x)    contribution of this unit to the row's dot product

struct FQ4K {
    static constexpr int UNIT = 32;
    struct Raw { uint4 q; uint4 h; };
    struct X { float lo[16], hi[16], slo, shi; };
    // unit u: block b = u>>3, t8 = u&7, group j = t8>>1, half hf = t8&1:
    //   low nibbles -> values 64j + 16hf + l (sub-block 2j), high nibbles -> +32 (sub-block 2j+1)
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        if (w.layout == 0) {
            r.q = ldg16(w.s[1] + (rb * 8 + u) * 16);
            r.h = ldg16(w.s[0] + (rb + (u >> 3)) * 16);
        } else {
            // row-group-major layout: the unit's four words sit in four consecutive lane slots
            const int64_t blk = rb + (u >> 3);
            const uint32_t* p = reinterpret_cast<const uint32_t*>(w.s[1] + q4k_qs_off(1, w.nb, blk, (u & 7) * 16));
            r.q = make_uint4(__ldg(p), __ldg(p + 4), __ldg(p + 8), __ldg(p + 12));
            r.h = ldg16(w.s[0] + q4k_hdr_off(1, w.nb, blk));
        }
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        const int k0 = (u >> 3) * 256 + ((u & 7) >> 1) * 64 + (u & 1) * 16;
        load_run16(xs, k0, x.lo); load_run16(xs, k0 + 32, x.hi);
        x.slo = sum16(x.lo); x.shi = sum16(x.hi);
    }
    __device__ static void scales(const uint4& h, int j, float& d, float& dmin, int& sc0, int& m0, int& sc1, int& m1) {
        d = f16_bits_to_f32(static_cast<uint16_t>(h.x & 0xFFFF));
        dmin = f16_bits_to_f32(static_cast<uint16_t>(h.x >> 16));
        // 12 scale bytes live in h.y, h.z, h.w; pairs 2j and 2j+1
        if (j < 2) {
            sc0 = word_byte(h.y, 2 * j) & 63; m0 = word_byte(h.z, 2 * j) & 63;
            sc1 = word_byte(h.y, 2 * j + 1) & 63; m1 = word_byte(h.z, 2 * j + 1) & 63;
        } else {
            const int p = 2 * j - 4;
            sc0 = (word_byte(h.w, p) & 15) | ((word_byte(h.y, p) >> 6) << 4);
            m0 = (word_byte(h.w, p) >> 4) | ((word_byte(h.z, p) >> 6) << 4);
            sc1 = (word_byte(h.w, p + 1) & 15) | ((word_byte(h.y, p + 1) >> 6) << 4);
            m1 = (word_byte(h.w, p + 1) >> 4) | ((word_byte(h.z, p + 1) >> 6) << 4);
        }
    }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        float d, dmin; int sc0, m0, sc1, m1;
        scales(r.h, (u & 7) >> 1, d, dmin, sc0, m0, sc1, m1);
        const float s0 = dot16_lo(r.q, x.lo), s1 = dot16_hi(r.q, x.hi);
        return d * (static_cast<float>(sc0) * s0 + static_cast<float>(sc1) * s1) -
               dmin * (static_cast<float>(m0) * x.slo + static_cast<float>(m1) * x.shi);
    }
};

struct FQ5K {
    static constexpr int UNIT = 32;
    struct Raw { uint4 q; uint4 h; uint4 qh; };
    typedef FQ4K::X X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        r.q = ldg16(w.s[2] + (rb * 8 + u) * 16);
        r.h = ldg16(w.s[0] + (rb + (u >> 3)) * 16);
        r.qh = ldg16(w.s[1] + (rb + (u >> 3)) * 32 + (u & 1) * 16);
    }
    __device__ static void load_x(const float4* xs, int u, X& x) { FQ4K::load_x(xs, u, x); }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        const int j = (u & 7) >> 1;
        float d, dmin; int sc0, m0, sc1, m1;
        FQ4K::scales(r.h, j, d, dmin, sc0, m0, sc1, m1);
        // fifth bit: bit 2j (low run) / 2j+1 (high run) of each qh byte -> +16
        const uint32_t k1 = 0x01010101u;
        const float s0 = dot16_bytes((r.q.x & 0x0F0F0F0Fu) | (((r.qh.x >> (2 * j)) & k1) << 4),
                                     (r.q.y & 0x0F0F0F0Fu) | (((r.qh.y >> (2 * j)) & k1) << 4),
                                     (r.q.z & 0x0F0F0F0Fu) | (((r.qh.z >> (2 * j)) & k1) << 4),
                                     (r.q.w & 0x0F0F0F0Fu) | (((r.qh.w >> (2 * j)) & k1) << 4), x.lo);
        const float s1 = dot16_bytes(((r.q.x >> 4) & 0x0F0F0F0Fu) | (((r.qh.x >> (2 * j + 1)) & k1) << 4),
                                     ((r.q.y >> 4) & 0x0F0F0F0Fu) | (((r.qh.y >> (2 * j + 1)) & k1) << 4),
                                     ((r.q.z >> 4) & 0x0F0F0F0Fu) | (((r.qh.z >> (2 * j + 1)) & k1) << 4),
                                     ((r.q.w >> 4) & 0x0F0F0F0Fu) | (((r.qh.w >> (2 * j + 1)) & k1) << 4), x.hi);
        return d * (static_cast<float>(sc0) * s0 + static_cast<float>(sc1) * s1) -
               dmin * (static_cast<float>(m0) * x.slo + static_cast<float>(m1) * x.shi);
    }
};

struct FQ6K {
    static constexpr int UNIT = 32;
    struct Raw { uint4 ql; uint4 qh; float d; int sc_lo, sc_hi; };
    typedef FQ4K::X X;
    // unit u: block b = u>>3, t8 = u&7 = 4hf + 2p + c: 16 bytes ql[64hf + 32p + 16c ..],
    //   low nibbles -> values 128hf + 32p + 16c + l, high nibbles -> +64; qh bytes qh[32hf + 16c ..]
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        const int64_t blk = rb + (u >> 3);
        const int t8 = u & 7, hf = t8 >> 2, p = (t8 >> 1) & 1, c = t8 & 1;
        const int64_t slot = q6k_row_slot(w.layout, w.nb, blk);
        if (w.layout == 0) {
            r.ql = ldg16(w.s[0] + (rb * 8 + u) * 16);
            r.qh = ldg16(w.s[1] + blk * 64 + hf * 32 + c * 16);
        } else {
            // row-group-major layout: the four words of each 16-byte run sit in four consecutive lane slots
            const uint32_t* pl = reinterpret_cast<const uint32_t*>(w.s[0] + q6k_ql_off(1, w.nb, blk, 64 * hf + 32 * p + 16 * c));
            const uint32_t* ph = reinterpret_cast<const uint32_t*>(w.s[1] + q6k_qh_off(1, w.nb, blk, 32 * hf + 16 * c));
            r.ql = make_uint4(__ldg(pl), __ldg(pl + 4), __ldg(pl + 8), __ldg(pl + 12));
            r.qh = make_uint4(__ldg(ph), __ldg(ph + 4), __ldg(ph + 8), __ldg(ph + 12));
        }
        const int8_t* sc = reinterpret_cast<const int8_t*>(w.s[2] + slot * 16 + 8 * hf + 2 * p + c);
        r.sc_lo = __ldg(sc); r.sc_hi = __ldg(sc + 4);
        r.d = ldg_f16(w.s[3] + slot * 2);
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        const int t8 = u & 7;
        const int k0 = (u >> 3) * 256 + (t8 >> 2) * 128 + ((t8 >> 1) & 1) * 32 + (t8 & 1) * 16;
        load_run16(xs, k0, x.lo); load_run16(xs, k0 + 64, x.hi);
        x.slo = sum16(x.lo); x.shi = sum16(x.hi);
    }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        const int p = ((u & 7) >> 1) & 1;
        const uint32_t k3 = 0x03030303u, kf = 0x0F0F0F0Fu;
        const int s_lo = 2 * p, s_hi = 2 * p + 4;
        const float s0 = dot16_bytes((r.ql.x & kf) | (((r.qh.x >> s_lo) & k3) << 4), (r.ql.y & kf) | (((r.qh.y >> s_lo) & k3) << 4),
                                     (r.ql.z & kf) | (((r.qh.z >> s_lo) & k3) << 4), (r.ql.w & kf) | (((r.qh.w >> s_lo) & k3) << 4), x.lo);
        const float s1 = dot16_bytes(((r.ql.x >> 4) & kf) | (((r.qh.x >> s_hi) & k3) << 4), ((r.ql.y >> 4) & kf) | (((r.qh.y >> s_hi) & k3) << 4),
                                     ((r.ql.z >> 4) & kf) | (((r.qh.z >> s_hi) & k3) << 4), ((r.ql.w >> 4) & kf) | (((r.qh.w >> s_hi) & k3) << 4), x.hi);
        return r.d * (static_cast<float>(r.sc_lo) * (s0 - 32.0f * x.slo) + static_cast<float>(r.sc_hi) * (s1 - 32.0f * x.shi));
    }
};

// Q4_0, Q4_1, IQ4_NL: one 32-value block per unit; low nibbles -> values 0..15, high -> 16..31.
template <uint32_t TYPE>
struct FQ4Small {
    static constexpr int UNIT = 32;
    struct Raw { uint4 q; float d, m; };
    typedef FQ4K::X X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        r.q = ldg16(w.s[1] + (rb + u) * 16);
        if (TYPE == T_Q4_1) { r.d = ldg_f16(w.s[0] + (rb + u) * 4); r.m = ldg_f16(w.s[0] + (rb + u) * 4 + 2); }
        else { r.d = ldg_f16(w.s[0] + (rb + u) * 2); r.m = 0.0f; }
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        load_run16(xs, u * 32, x.lo); load_run16(xs, u * 32 + 16, x.hi);
        x.slo = sum16(x.lo); x.shi = sum16(x.hi);
    }
    __device__ static float dot(const Raw& r, const X& x, int) {
        if (TYPE == T_IQ4_NL) {
            float s = 0.0f;
            const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t b = (qw[i >> 2] >> (8 * (i & 3))) & 0xFFu;
                s = fmaf(x.lo[i], static_cast<float>(kIq4Codebook[b & 15]), s);
                s = fmaf(x.hi[i], static_cast<float>(kIq4Codebook[b >> 4]), s);
            }
            return r.d * s;
        }
        const float s = dot16_lo(r.q, x.lo) + dot16_hi(r.q, x.hi);
        if (TYPE == T_Q4_0) return r.d * (s - 8.0f * (x.slo + x.shi));
        return r.d * s + r.m * (x.slo + x.shi);
    }
};

struct FIQ4XS {
    static constexpr int UNIT = 32;
    struct Raw { uint4 q; uint2 h; };
    typedef FQ4K::X X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        r.q = ldg16(w.s[1] + (rb * 8 + u) * 16);
        r.h = __ldg(reinterpret_cast<const uint2*>(w.s[0] + (rb + (u >> 3)) * 8));
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        load_run16(xs, u * 32, x.lo); load_run16(xs, u * 32 + 16, x.hi);
        x.slo = 0.0f; x.shi = 0.0f;
    }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        const int ib = u & 7;
        const float d = f16_bits_to_f32(static_cast<uint16_t>(r.h.x & 0xFFFF));
        const uint32_t sh = r.h.x >> 16;
        const int ls = static_cast<int>((word_byte(r.h.y, ib >> 1) >> (4 * (ib & 1))) & 15) | static_cast<int>(((sh >> (2 * ib)) & 3) << 4);
        float s = 0.0f;
        const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t b = (qw[i >> 2] >> (8 * (i & 3))) & 0xFFu;
            s = fmaf(x.lo[i], static_cast<float>(kIq4Codebook[b & 15]), s);
            s = fmaf(x.hi[i], static_cast<float>(kIq4Codebook[b >> 4]), s);
        }
        return d * static_cast<float>(ls - 32) * s;
    }
};

#ifdef GGB_HAVE_IQ_GRIDS
// Grid-coded formats: a unit is one 32-value sub-block, decoded eight values at a time through the
// codebook (iq_decode8).  Correct for every one of them; not tuned (none is in a benchmark configuration).
template <uint32_t TYPE>
struct FIQGrid {
    static constexpr int UNIT = 32;
    struct Raw { const uint8_t* p; };
    typedef FQ4K::X X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        r.p = w.s[0] + (rb + (u >> 3)) * format_info(TYPE).block_bytes;
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        load_run16(xs, u * 32, x.lo); load_run16(xs, u * 32 + 16, x.hi);
        x.slo = 0.0f; x.shi = 0.0f;
    }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        float s = 0.0f, v[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            iq_decode8<TYPE>(r.p, (u & 7) * 4 + g, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(g < 2 ? x.lo[8 * g + i] : x.hi[8 * (g - 2) + i], v[i], s);
        }
        return s;
    }
};
#endif

struct FQ80 {
    static constexpr int UNIT = 32;
    struct Raw { uint4 q0, q1; float d; };
    typedef FQ4K::X X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        r.q0 = ldg16(w.s[1] + (rb + u) * 32);
        r.q1 = ldg16(w.s[1] + (rb + u) * 32 + 16);
        r.d = ldg_f16(w.s[0] + (rb + u) * 2);
    }
    __device__ static void load_x(const float4* xs, int u, X& x) {
        load_run16(xs, u * 32, x.lo); load_run16(xs, u * 32 + 16, x.hi);
        x.slo = sum16(x.lo); x.shi = sum16(x.hi);
    }
    __device__ static float dot(const Raw& r, const X& x, int) {
        // int8 q -> unsigned q+128 by flipping the sign bit, bias removed through the sums
        const uint32_t f = 0x80808080u;
        const float s = dot16_bytes(r.q0.x ^ f, r.q0.y ^ f, r.q0.z ^ f, r.q0.w ^ f, x.lo) +
                        dot16_bytes(r.q1.x ^ f, r.q1.y ^ f, r.q1.z ^ f, r.q1.w ^ f, x.hi);
        return r.d * (s - 128.0f * (x.slo + x.shi));
    }
};

// Q2_K / Q3_K: a unit is 16 bytes of qs = 64 values: (half hf, odd) of block b, four 2-bit planes
// sh = 0..3 -> sub-block 8hf + 2sh + odd, values 128hf + 32sh + 16odd + l.
struct X64 { float r[4][16]; float s[4]; };
__device__ __forceinline__ void load_x64(const float4* xs, int u, X64& x) {
    const int k0 = (u >> 2) * 256 + ((u >> 1) & 1) * 128 + (u & 1) * 16;
#pragma unroll
    for (int sh = 0; sh < 4; ++sh) { load_run16(xs, k0 + 32 * sh, x.r[sh]); x.s[sh] = sum16(x.r[sh]); }
}

struct FQ2K {
    static constexpr int UNIT = 64;
    struct Raw { uint4 q; uint2 sc; float d, dmin; };
    typedef X64 X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        const int64_t blk = rb + (u >> 2);
        r.q = ldg16(w.s[1] + (rb * 4 + u) * 16);
        r.sc = __ldg(reinterpret_cast<const uint2*>(w.s[0] + blk * 16 + ((u >> 1) & 1) * 8));
        r.d = ldg_f16(w.s[2] + blk * 4); r.dmin = ldg_f16(w.s[2] + blk * 4 + 2);
    }
    __device__ static void load_x(const float4* xs, int u, X& x) { load_x64(xs, u, x); }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        const int odd = u & 1;
        const uint32_t k3 = 0x03030303u;
        float acc_d = 0.0f, acc_m = 0.0f;
#pragma unroll
        for (int sh = 0; sh < 4; ++sh) {
            const uint32_t sbyte = word_byte(sh < 2 ? r.sc.x : r.sc.y, 2 * (sh & 1) + odd);
            const float s = dot16_bytes((r.q.x >> (2 * sh)) & k3, (r.q.y >> (2 * sh)) & k3, (r.q.z >> (2 * sh)) & k3,
                                        (r.q.w >> (2 * sh)) & k3, x.r[sh]);
            acc_d = fmaf(static_cast<float>(sbyte & 15), s, acc_d);
            acc_m = fmaf(static_cast<float>(sbyte >> 4), x.s[sh], acc_m);
        }
        return r.d * acc_d - r.dmin * acc_m;
    }
};

struct FQ3K {
    static constexpr int UNIT = 64;
    struct Raw { uint4 q; uint4 hm; uint32_t s0, s1, s2; float d; };
    typedef X64 X;
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        const int64_t blk = rb + (u >> 2);
        r.q = ldg16(w.s[1] + (rb * 4 + u) * 16);
        r.hm = ldg16(w.s[0] + blk * 32 + (u & 1) * 16);
        const uint32_t* sp = reinterpret_cast<const uint32_t*>(w.s[2] + blk * 12);
        r.s0 = __ldg(sp); r.s1 = __ldg(sp + 1); r.s2 = __ldg(sp + 2);
        r.d = ldg_f16(w.s[3] + blk * 2);
    }
    __device__ static void load_x(const float4* xs, int u, X& x) { load_x64(xs, u, x); }
    __device__ static float dot(const Raw& r, const X& x, int u) {
        const int odd = u & 1, hf = (u >> 1) & 1;
        const uint32_t k3 = 0x03030303u, k1 = 0x01010101u;
        float acc = 0.0f;
#pragma unroll
        for (int sh = 0; sh < 4; ++sh) {
            const int sb = 8 * hf + 2 * sh + odd;
            const uint32_t lo_src = (sb & 4) ? r.s1 : r.s0;                 // bytes 0..7 hold the low nibbles
            const int lo = (sb < 8) ? (word_byte(lo_src, sb & 3) & 15) : (word_byte(lo_src, sb & 3) >> 4);
            const int hi = (word_byte(r.s2, sb & 3) >> (2 * (sb >> 2))) & 3;
            const int bit = 4 * hf + sh;
            // value = q2 - (hbit ? 0 : 4) = (q2 + 4*hbit) - 4
            const float s = dot16_bytes(((r.q.x >> (2 * sh)) & k3) | (((r.hm.x >> bit) & k1) << 2), ((r.q.y >> (2 * sh)) & k3) | (((r.hm.y >> bit) & k1) << 2),
                                        ((r.q.z >> (2 * sh)) & k3) | (((r.hm.z >> bit) & k1) << 2), ((r.q.w >> (2 * sh)) & k3) | (((r.hm.w >> bit) & k1) << 2), x.r[sh]);
            acc = fmaf(static_cast<float>((lo | (hi << 4)) - 32), s - 4.0f * x.s[sh], acc);
        }
        return r.d * acc;
    }
};

// F16 / BF16: a unit is 16 bytes = 8 weights.  F32: a unit is 32 bytes = 8 weights.
template <uint32_t TYPE>
struct FPlain {
    static constexpr int UNIT = 8;
    struct Raw { uint4 a, b; };
    struct X { float v[8]; };
    __device__ static void load(const PackedW& w, int64_t rb, int u, Raw& r) {
        if (TYPE == T_F32) { r.a = ldg16(w.s[0] + (rb + u * 8) * 4); r.b = ldg16(w.s[0] + (rb + u * 8) * 4 + 16); }
        else { r.a = ldg16(w.s[0] + (rb + u * 8) * 2); r.b = make_uint4(0, 0, 0, 0); }
    }
    __device__ static void load_x(const float4* xs, int u, X& x) { load_run8(xs, u * 8, x.v); }
    __device__ static float dot(const Raw& r, const X& x, int) {
        float wv[8];
        if (TYPE == T_F32) {
            wv[0] = __uint_as_float(r.a.x); wv[1] = __uint_as_float(r.a.y); wv[2] = __uint_as_float(r.a.z); wv[3] = __uint_as_float(r.a.w);
            wv[4] = __uint_as_float(r.b.x); wv[5] = __uint_as_float(r.b.y); wv[6] = __uint_as_float(r.b.z); wv[7] = __uint_as_float(r.b.w);
        } else {
            const uint32_t q[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (TYPE == T_BF16) { wv[2 * i] = __uint_as_float(q[i] << 16); wv[2 * i + 1] = __uint_as_float(q[i] & 0xFFFF0000u); }
                else { wv[2 * i] = f16_bits_to_f32(static_cast<uint16_t>(q[i] & 0xFFFF)); wv[2 * i + 1] = f16_bits_to_f32(static_cast<uint16_t>(q[i] >> 16)); }
            }
        }
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(x.v[i], wv[i], s);
        return s;
    }
};

// ---- the kernel --------------------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Stage MT activation rows into swizzled shared memory; with gamma != nullptr each row is first
// RMS-normalised: v = sum(x^2)/K + eps, y = x * (1/sqrt(v)) * gamma.
template <int MT>
__device__ void stage_x(const GemvArgs& a, int m0, float4* xs, float* red) {
    const int K4 = a.w.K >> 2;
    const int tid = threadIdx.x, nt = blockDim.x;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int row = min(m0 + m, a.M - 1);
        const float4* src = reinterpret_cast<const float4*>(a.x + static_cast<size_t>(row) * a.lda);
        float inv = 1.0f;
        if (a.gamma) {
            float ss = 0.0f;
            for (int i = tid; i < K4; i += nt) { const float4 v = __ldg(src + i); ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
            ss = warp_sum(ss);
            __syncthreads();
            if ((tid & 31) == 0) red[tid >> 5] = ss;
            __syncthreads();
            float tot = 0.0f;
            for (int i = 0; i < (nt >> 5); ++i) tot += red[i];
            inv = 1.0f / sqrtf(tot / static_cast<float>(a.w.K) + a.eps);
        }
        float4* dst = xs + static_cast<size_t>(m) * K4;
        for (int i = tid; i < K4; i += nt) {
            float4 v = __ldg(src + i);
            if (a.gamma) {
                const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + i);
                v.x = v.x * inv * g.x; v.y = v.y * inv * g.y; v.z = v.z * inv * g.z; v.w = v.w * inv * g.w;
            }
            dst[swz4(i)] = v;
        }
    }
    __syncthreads();
}

template <class F, int MT, int RW, bool DUAL>
__global__ void __launch_bounds__(128) gemv_kernel(const GemvArgs a, const int m0) {
    extern __shared__ float4 xs[];
    __shared__ float red[32];
    stage_x<MT>(a, m0, xs, red);
    const int K4 = a.w.K >> 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
    const int units = a.w.K / F::UNIT;
    const int64_t N = a.w.N;
    const int64_t groups = (N + RW - 1) / RW;
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * wpc + warp; g < groups; g += static_cast<int64_t>(gridDim.x) * wpc) {
        const int64_t r0 = g * RW;
        float acc[RW][MT], acc2[DUAL ? RW : 1][MT];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) { acc[r][m] = 0.0f; if constexpr (DUAL) acc2[r][m] = 0.0f; }
        for (int u = lane; u < units; u += 32) {
            typename F::Raw raw[RW], raw2[DUAL ? RW : 1];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int64_t rb = min(r0 + r, N - 1) * a.w.nb;
                F::load(a.w, rb, u, raw[r]);
                if constexpr (DUAL) F::load(a.w2, rb, u, raw2[r]);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                typename F::X x;
                F::load_x(xs + static_cast<size_t>(m) * K4, u, x);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    acc[r][m] += F::dot(raw[r], x, u);
                    if constexpr (DUAL) acc2[r][m] += F::dot(raw2[r], x, u);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                float v = warp_sum(acc[r][m]);
                float v2 = 0.0f;
                if constexpr (DUAL) v2 = warp_sum(acc2[r][m]);
                const int64_t n = r0 + r;
                if (lane == 0 && n < N && m0 + m < a.M) {
                    const size_t o = static_cast<size_t>(m0 + m) * a.ldc + n;
                    if (DUAL) v = (v / (1.0f + expf(-v))) * v2;                 // silu(gate) * up
                    else if (a.epi == EPI_ADD_BIAS) v += __ldg(a.bias + n);
                    else if (a.epi == EPI_RESIDUAL) v += a.resid[o];
                    a.y[o] = v;
                }
            }
    }
}

template <class F, int MT, int RW, bool DUAL>
static cudaError_t launch_one(Context* c, const GemvArgs& a, int m0, cudaStream_t s) {
    const size_t smem = static_cast<size_t>(MT) * a.w.K * sizeof(float);
    auto kern = gemv_kernel<F, MT, RW, DUAL>;
    {   // raised on first need, outside any capture
        const cudaError_t e = ensure_dynamic_smem(c, kern, smem);
        if (e != cudaSuccess) return e;
    }
    const int64_t groups = (a.w.N + RW - 1) / RW;
    const int wpc = 4;
    int64_t ctas = (groups + wpc - 1) / wpc;
    const int64_t cap = static_cast<int64_t>(c->sm_count) * 8;
    if (ctas > cap) ctas = cap;
    kern<<<static_cast<int>(ctas), wpc * 32, smem, s>>>(a, m0);
    c->launches++;
    return cudaGetLastError();
}

template <class F, bool DUAL>
static int launch_fmt(Context* c, const GemvArgs& a, cudaStream_t s) {
    if (a.w.K % F::UNIT || a.w.K % 32) return set_status(c, GGB_INVALID_PARAM, "gemv: K must be a multiple of 32 and of the format's unit");
    const bool big = a.w.N >= 8192;
    cudaError_t e = cudaSuccess;
    int m0 = 0;
    // rows of x go through in tiles of 4, 2 or 1 (shared memory holds MT * K floats)
    while (m0 < a.M && e == cudaSuccess) {
        const int left = a.M - m0;
        const size_t per_row = static_cast<size_t>(a.w.K) * sizeof(float);
        if (left >= 4 && 4 * per_row <= 160 * 1024) { e = launch_one<F, 4, 2, DUAL>(c, a, m0, s); m0 += 4; }
        else if (left >= 2 && 2 * per_row <= 160 * 1024) { e = launch_one<F, 2, 2, DUAL>(c, a, m0, s); m0 += 2; }
        else {
            if (per_row > 200 * 1024) return set_status(c, GGB_INVALID_PARAM, "gemv: K too large for shared memory");
            e = (big && !DUAL) ? launch_one<F, 1, 4, DUAL>(c, a, m0, s) : launch_one<F, 1, 2, DUAL>(c, a, m0, s);
            m0 += 1;
        }
    }
    return cuda_status(c, e, "gemv launch");
}

template <bool DUAL>
static int dispatch(Context* c, const GemvArgs& a, cudaStream_t s) {
    switch (a.w.type) {
    case T_Q4_K: return launch_fmt<FQ4K, DUAL>(c, a, s);
    case T_Q5_K: return launch_fmt<FQ5K, DUAL>(c, a, s);
    case T_Q6_K: return launch_fmt<FQ6K, DUAL>(c, a, s);
    case T_Q4_0: return launch_fmt<FQ4Small<T_Q4_0>, DUAL>(c, a, s);
    case T_Q4_1: return launch_fmt<FQ4Small<T_Q4_1>, DUAL>(c, a, s);
    case T_IQ4_NL: return launch_fmt<FQ4Small<T_IQ4_NL>, DUAL>(c, a, s);
    case T_IQ4_XS: return launch_fmt<FIQ4XS, DUAL>(c, a, s);
#ifdef GGB_HAVE_IQ_GRIDS
    case T_IQ2_XXS: return launch_fmt<FIQGrid<T_IQ2_XXS>, DUAL>(c, a, s);
    case T_IQ2_XS: return launch_fmt<FIQGrid<T_IQ2_XS>, DUAL>(c, a, s);
    case T_IQ2_S: return launch_fmt<FIQGrid<T_IQ2_S>, DUAL>(c, a, s);
    case T_IQ3_XXS: return launch_fmt<FIQGrid<T_IQ3_XXS>, DUAL>(c, a, s);
    case T_IQ3_S: return launch_fmt<FIQGrid<T_IQ3_S>, DUAL>(c, a, s);
    case T_IQ1_S: return launch_fmt<FIQGrid<T_IQ1_S>, DUAL>(c, a, s);
    case T_IQ1_M: return launch_fmt<FIQGrid<T_IQ1_M>, DUAL>(c, a, s);
#endif
    case T_Q8_0: return launch_fmt<FQ80, DUAL>(c, a, s);
    case T_Q2_K: return launch_fmt<FQ2K, DUAL>(c, a, s);
    case T_Q3_K: return launch_fmt<FQ3K, DUAL>(c, a, s);
    case T_F32: return launch_fmt<FPlain<T_F32>, DUAL>(c, a, s);
    case T_F16: return launch_fmt<FPlain<T_F16>, DUAL>(c, a, s);
    case T_BF16: return launch_fmt<FPlain<T_BF16>, DUAL>(c, a, s);
    default: return set_status(c, GGB_INVALID_PARAM, "gemv: unsupported weight type");
    }
}

// Grow the workspace for split-K / K-slice partial sums (never inside a stream capture: callers run one eager pass first).
static int ensure_ws(Context* c, size_t floats, cudaStream_t s) {
    if (floats <= c->d_ws_floats) return GGB_OK;
    cudaStreamSynchronize(s);
    if (c->d_ws) cudaFree(c->d_ws);
    c->d_ws = nullptr; c->d_ws_floats = 0;
    if (cuda_status(c, cudaMalloc(&c->d_ws, floats * sizeof(float)), "cudaMalloc(partial sums)") != GGB_OK) return c->last_status;
    c->d_ws_floats = floats;
    return GGB_OK;
}

// The same for the int8-limb image of the activations (multi-row GEMVs).
static int ensure_limbs(Context* c, size_t bytes, cudaStream_t s) {
    if (bytes <= c->d_limbs_bytes) return GGB_OK;
    c->limbs_x = nullptr;
    cudaStreamSynchronize(s);
    if (c->d_limbs) cudaFree(c->d_limbs);
    c->d_limbs = nullptr; c->d_limbs_bytes = 0;
    if (cuda_status(c, cudaMalloc(&c->d_limbs, bytes), "cudaMalloc(activation limbs)") != GGB_OK) return c->last_status;
    c->d_limbs_bytes = bytes;
    return GGB_OK;
}

int launch_gemv(Context* c, const GemvArgs& a, cudaStream_t s) {
    c->gemv_calls++;
    if ((!a.x && !a.attn_partial && !a.x_img) || (!a.y && !a.y_img) || a.M <= 0 || a.w.N <= 0 || a.w.K <= 0) return set_status(c, GGB_INVALID_PARAM, "gemv: bad arguments");
    if (a.attn_partial && (a.w.layout != 1 || a.M != 1)) return set_status(c, GGB_INVALID_PARAM, "gemv: attention-merge input needs the tensor-core layout and M == 1");
    if (a.x && ((reinterpret_cast<uintptr_t>(a.x) & 15) || (a.lda & 3))) return set_status(c, GGB_INVALID_PARAM, "gemv: x must be 16-byte aligned with lda % 4 == 0");
    if (a.epi == EPI_SWIGLU && (a.w2.type != a.w.type || a.w2.N != a.w.N || a.w2.K != a.w.K))
        return set_status(c, GGB_INVALID_PARAM, "gemv: gate/up mismatch");
    if (c->use_tc && a.M >= c->tc_min_m && (a.x || a.x_img) && !a.n_cat && !a.attn_partial) {
        const size_t need = a.x_img ? 0 : gemm_tc_xb_elems(a);
        if (need > c->d_xb_elems) {
            cudaStreamSynchronize(s);
            if (c->d_xb) cudaFree(c->d_xb);
            c->d_xb = nullptr; c->d_xb_elems = 0;
            if (cuda_status(c, cudaMalloc(&c->d_xb, need * 2), "cudaMalloc(fp16 activations)") != GGB_OK) return c->last_status;
            c->d_xb_elems = need;
        }
        if (ensure_ws(c, gemm_tc_ws_floats(a), s) != GGB_OK) return c->last_status;
        const int st = launch_gemm_tc(c, a, c->d_xb, c->d_xb_elems, c->d_ws, c->d_ws_floats, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (a.x_img || a.y_img) return set_status(c, GGB_INVALID_PARAM, "gemv: tile-image operands need the tensor-core GEMM");
    if (a.w.layout == 1 && a.M >= 3 && a.M <= 16) {
        // up to 16 activation rows in one pass over the weights
        if (ensure_ws(c, gemv_mma_rows_ws_floats(a), s) != GGB_OK) return c->last_status;
        if (ensure_limbs(c, gemv_mma_rows_limbs_bytes(a.M, a.w.K), s) != GGB_OK) return c->last_status;
        const int st = launch_gemv_mma_rows(c, a, c->d_ws, c->d_ws_floats, c->d_limbs, c->d_limbs_bytes, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (a.w.layout == 1) {
        // tensor-core kernel, two activation rows per pass (each pass streams the weights once)
        int st = GGB_OK;
        for (int m0 = 0; m0 < a.M && st == GGB_OK; m0 += 2) {
            GemvArgs sub = a;
            sub.M = std::min(2, a.M - m0);
            sub.x = a.x + static_cast<size_t>(m0) * a.lda;
            sub.y = a.y + static_cast<size_t>(m0) * a.ldc;
            if (a.resid) sub.resid = a.resid + static_cast<size_t>(m0) * a.ldc;
            st = launch_gemv_mma(c, sub, s);
            if (st == GGB_NOT_FOUND && m0 == 0) break;
        }
        if (st != GGB_NOT_FOUND) return st;
    }
    if (a.attn_partial || a.sel || a.xscale)
        return set_status(c, GGB_INVALID_PARAM, "gemv: attention-merge input, routed experts and scaled activations need the tensor-core kernel (Q4_K / Q6_K)");
    static const bool stream_mma_m1 = getenv("GGB_NO_STREAM_MMA") == nullptr;
    if (c->use_mma && stream_mma_m1 && a.M <= 2 && a.w.layout == 0 && a.w.K % 256 == 0 && (a.w.type == T_Q8_0 || a.w.type == T_Q4_0)) {
        // One or two rows of Q8_0 / Q4_0 on the int8 tensor cores (the activations are converted in the kernel's prologue).
        // Against the dp4a kernel below at M = 1: Q4_0 5.7-8.6 us against 5.8-9.0, Q8_0 6.3-10.4 against 5.9-10.3 per matrix
        // but 1.50 against 1.60 ms for the Qwen2.5-1.5B-shape decode step; the IQ4 formats (codebook look-ups per fragment)
        // are slower here (12.7 against 8.6 us) and stay on the dp4a kernel.
        const int st = launch_gemv_mma_stream(c, a, c->d_ws, c->d_ws_floats, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (c->use_tma && a.M == 1) {
        const int st = launch_gemv_tma(c, a, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (c->use_mma && a.M >= 3 && a.M <= 16 && a.w.layout == 0 && a.w.K % 256 == 0 && !a.n_cat &&
        (a.w.type == T_Q8_0 || a.w.type == T_Q4_0 || a.w.type == T_IQ4_NL || a.w.type == T_IQ4_XS)) {
        // 3..16 rows of a 32-block format on the int8 tensor cores, straight from the stream layout
        if (ensure_ws(c, gemv_mma_stream_ws_floats(a), s) != GGB_OK) return c->last_status;
        if (ensure_limbs(c, gemv_mma_rows_limbs_bytes(a.M, a.w.K), s) != GGB_OK) return c->last_status;
        const int st = launch_gemv_mma_stream(c, a, c->d_ws, c->d_ws_floats, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (c->use_tma && a.M >= 3 && a.M <= 16 && a.w.layout == 0 && a.w.K % 256 == 0 && !a.n_cat && a.w.type != T_Q8_0) {
        // 3..16 rows of a stream-layout matrix: the weights once per chunk of rows, exact int8-limb activations.
        // Measured at M = 16 against the general kernel below: IQ4_XS 31-116 us against 90-342, Q4_0 23-85 against 35-128;
        // Q8_0 (twice the dp4a per weight byte pair) 29-111 against 35-128 but slower on wide matrices (90 against 74 us
        // at 8192 x 2048), so it stays on the general kernel.
        if (ensure_limbs(c, gemv_mma_rows_limbs_bytes(a.M, a.w.K), s) != GGB_OK) return c->last_status;
        const int st = launch_gemv_tma_rows(c, a, s);
        if (st != GGB_NOT_FOUND) return st;
    }
    if (a.n_cat) {
        // no kernel took the stack: one launch per matrix
        GemvArgs one = a;
        one.n_cat = 0;
        int st = launch_gemv(c, one, s);
        for (int i = 0; i < a.n_cat && st == GGB_OK; ++i) {
            one.w = a.cat_w[i]; one.y = a.cat_y[i]; one.bias = a.cat_bias[i]; one.ldc = a.cat_ldc[i];
            st = launch_gemv(c, one, s);
        }
        return st;
    }
    if (a.epi == EPI_SWIGLU) return dispatch<true>(c, a, s);
    return dispatch<false>(c, a, s);
}

}  // namespace ggb
