// The body of the split-KV paged attention for one (KV head, context split, token): shared by the stand-alone
// kernel (ggb_attn.cu) and by the attention phase of the persistent decode-step kernel (ggb_decode_step.cu).
#pragma once
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#include "ggb_attn.h"

namespace ggb {

// Loads of activations: COHERENT reads through L2 only (ld.global.cg), for callers in which another CTA of the
// SAME launch wrote the value a moment ago (L1 is not coherent between SMs).
template <bool COHERENT>
__device__ __forceinline__ float ldx(const float* p) { return COHERENT ? __ldcg(p) : *p; }

__device__ __forceinline__ float attn_wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Shared memory the body needs, in bytes.
constexpr size_t attn_tile_smem(int HD) {
    return sizeof(uint32_t) * (64 * (HD / 2) + 64 * (HD / 2 + 1)) + sizeof(float) * (8 * HD + 8 * 64 + 24 + 12) + 2 * 2 * HD + 16;
}

// 128 threads (tid 0..127) run it together; sync() is a barrier over exactly those threads.  Keys are processed in
// chunks of 64: the chunk's K and V rows are first copied into shared memory with every 16-byte load in flight at
// once, then scores, an online softmax and P*V run out of shared memory in fp32.  With a.fuse (single-token decode)
// the body also rotates q and the new key, and the split that contains pos stores the new key and value.
template <int HD, bool COHERENT, bool HSPLIT = false, class Sync>
__device__ __forceinline__ void attn_tile_body(const AttnPagedArgs& a, const int hx, const int split, const int t, const int tid,
                                               uint32_t* sm_u, Sync sync) {
    constexpr int KW = HD / 2;           // 32-bit words (bf16 pairs) per K or V row
    constexpr int KS = KW + 1;           // padded K row stride: thread-per-key reads hit distinct banks
    constexpr int TK = 64;               // keys per chunk
    constexpr int NP = (8 * KW + 127) / 128;   // (head, dim pair) items per thread in P*V
    const int lane = tid & 31, warp = tid >> 5;
    // HSPLIT: hx = KV head * head_split + part, the query heads that share a KV head are dealt to several CTAs (models
    // with one or two KV heads would otherwise fill a fraction of the SMs).  It is a template parameter because the
    // general form, compiled into the one-CTA-per-KV-head kernel, made that kernel slower (a 16-sequence step of the
    // 8B shape: 12.4 ms against 10.9) although it computes the same values there.
    const int hs = HSPLIT ? max(a.head_split, 1) : 1;
    const int h = HSPLIT ? hx / hs : hx, hpart = HSPLIT ? hx - h * hs : 0;
    const int G = HSPLIT ? (a.n_head / a.n_kv) / hs : a.n_head / a.n_kv;      // query heads of this CTA
    const size_t head0 = HSPLIT ? static_cast<size_t>(h) * (a.n_head / a.n_kv) + static_cast<size_t>(hpart) * G
                                : static_cast<size_t>(h) * G;                 // the first of them
    // Fused step: the values the rotation below needs (the G query heads and the new key) do not depend
    // on the position, so their loads are issued before the position is looked at; the position's own
    // round trip to memory then overlaps theirs instead of preceding it.
    constexpr int NQ = HD <= 128 ? (9 * (HD / 2) + 127) / 128 : 0;       // rotation items per thread, G <= 8
    float qpre0[NQ > 0 ? NQ : 1], qpre1[NQ > 0 ? NQ : 1];
    if (NQ > 0 && a.fuse) {
        const float* qb = a.q + (static_cast<size_t>(t) * a.n_head + head0) * HD;
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int idx = tid + 128 * u, hh = idx / (HD / 2), i = idx - hh * (HD / 2);
            if (hh <= G) {
                const int i0 = a.neox ? i : 2 * i, i1 = a.neox ? i + HD / 2 : 2 * i + 1;
                const float* src = hh < G ? qb + hh * HD : a.k_new + (static_cast<size_t>(t) * a.n_kv + h) * HD;
                qpre0[u] = ldx<COHERENT>(src + i0); qpre1[u] = ldx<COHERENT>(src + i1);
            }
        }
    }
    const int pos = a.seq_pos ? a.seq_pos[t] : (a.d_pos ? a.d_pos[0] : a.pos0) + t;
    const int32_t* const bt = a.block_table + static_cast<size_t>(t) * a.seq_table_stride;
    const int keys_per_split = a.pages_per_split * a.page;
    const int j_begin = split * keys_per_split;
    const int j_end = min(j_begin + keys_per_split, pos + 1);
    if (j_begin > pos) return;           // no visible key in this split (the merge skips it too)

    uint32_t* Vt = sm_u;                                   // [TK][KW]   (16-byte aligned rows)
    uint32_t* Kt = Vt + TK * KW;                           // [TK][KS]
    float* qs = reinterpret_cast<float*>(Kt + TK * KS);    // [G][HD], already multiplied by 1/sqrt(HD)
    float* S = qs + 8 * HD;                                // [8][TK] scores, then probabilities
    float* mrun = S + 8 * TK;                              // [8] running max, [8] running sum, [8] rescale
    float* lrun = mrun + 8;
    float* corr = lrun + 8;
    float* hinv = corr + 8;                                // [9] per-head norm factors (q heads, then k)
    __nv_bfloat16* fresh = reinterpret_cast<__nv_bfloat16*>(hinv + 12);   // [2][HD] new key and value
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    const float* q = a.q + (static_cast<size_t>(t) * a.n_head + head0) * HD;
    const bool has_new = a.fuse && pos >= j_begin && pos < j_begin + keys_per_split;
    const int half = HD >> 1;

    // The first chunk's K and V rows are requested now, into registers, so that their memory latency
    // overlaps the q / new-key preparation below (head_dim <= 128; larger heads load in the loop).
    constexpr int NPF = HD <= 128 ? HD / 16 : 0;
    uint4 kpre[NPF > 0 ? NPF : 1], vpre[NPF > 0 ? NPF : 1];
    // chunk [j0, j0 + n) of K and V into registers (16 bytes per thread and item, all loads in flight at once)
    auto prefetch = [&](int j0, int n) {
#pragma unroll
        for (int u = 0; u < NPF; ++u) {
            const int i = tid + 128 * u;
            const int row = i / (HD / 8), part = i - row * (HD / 8);
            if (row < n) {
                const int j = j0 + row;
                const int page = bt[j / a.page], slot = j % a.page;
                const size_t o = ((static_cast<size_t>(page) * a.n_kv + h) * a.page + slot) * HD + part * 8;
                kpre[u] = *reinterpret_cast<const uint4*>(a.k_cache + o);
                vpre[u] = *reinterpret_cast<const uint4*>(a.v_cache + o);
            }
        }
    };
    if (NPF > 0) prefetch(j_begin, min(TK, j_end - j_begin));
    if (tid < 8) { mrun[tid] = -INFINITY; lrun[tid] = 0.0f; }
    if (a.fuse) {
        // optional per-head RMS norm of q and k before the rotation, sum of squares in double
        // (src/cli/main.cpp:3294-3299)
        for (int hh = warp; hh < G + 1; hh += 4) {
            const float* nw = hh < G ? a.q_norm : a.k_norm;
            float inv = 1.0f;
            if (nw) {
                const float* src = hh < G ? q + hh * HD : a.k_new + (static_cast<size_t>(t) * a.n_kv + h) * HD;
                double ss = 0.0;
                for (int i = lane; i < HD; i += 32) { const float sv = ldx<COHERENT>(src + i); ss += static_cast<double>(sv) * sv; }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                inv = 1.0f / sqrtf(static_cast<float>(ss / HD) + a.eps);
            }
            if (lane == 0) hinv[hh] = inv;
        }
        sync();
        const float* cs = a.cos_tab + static_cast<size_t>(pos) * half;
        const float* sn = a.sin_tab + static_cast<size_t>(pos) * half;
        auto rotate = [&](int idx, float v0, float v1) {
            const int hh = idx / half, i = idx - hh * half;
            const int i0 = a.neox ? i : 2 * i, i1 = a.neox ? i + half : 2 * i + 1;
            const bool is_q = hh < G;
            const float* nw = is_q ? a.q_norm : a.k_norm;
            if (nw) { v0 = v0 * hinv[hh] * nw[i0]; v1 = v1 * hinv[hh] * nw[i1]; }
            const float r0 = v0 * cs[i] - v1 * sn[i], r1 = v0 * sn[i] + v1 * cs[i];
            if (is_q) { qs[hh * HD + i0] = r0 * scale; qs[hh * HD + i1] = r1 * scale; }
            else { fresh[i0] = __float2bfloat16_rn(r0); fresh[i1] = __float2bfloat16_rn(r1); }
        };
        const int n_items = (G + (has_new ? 1 : 0)) * half;
        if (NQ > 0) {
#pragma unroll
            for (int u = 0; u < NQ; ++u)
                if (tid + 128 * u < n_items) rotate(tid + 128 * u, qpre0[u], qpre1[u]);
        } else {
            for (int idx = tid; idx < n_items; idx += 128) {
                const int hh = idx / half, i = idx - hh * half;
                const int i0 = a.neox ? i : 2 * i, i1 = a.neox ? i + half : 2 * i + 1;
                const float* src = hh < G ? q + hh * HD : a.k_new + (static_cast<size_t>(t) * a.n_kv + h) * HD;
                rotate(idx, ldx<COHERENT>(src + i0), ldx<COHERENT>(src + i1));
            }
        }
        if (has_new) for (int i = tid; i < HD; i += 128) fresh[HD + i] = __float2bfloat16_rn(ldx<COHERENT>(a.v_new + (static_cast<size_t>(t) * a.n_kv + h) * HD + i));
        sync();
        if (has_new && hpart == 0) {     // K is cached after RoPE, V raw (src/cli/main.cpp:3354-3356)
            const int page = bt[pos / a.page], slot = pos % a.page;
            const size_t o = ((static_cast<size_t>(page) * a.n_kv + h) * a.page + slot) * HD;
            for (int i = tid; i < HD; i += 128) { a.k_cache_w[o + i] = fresh[i]; a.v_cache_w[o + i] = fresh[HD + i]; }
        }
    } else {
        for (int i = tid; i < G * HD; i += 128) qs[i] = ldx<COHERENT>(q + i) * scale;
    }

    float acc[NP][2];
#pragma unroll
    for (int p = 0; p < NP; ++p) { acc[p][0] = 0.0f; acc[p][1] = 0.0f; }

    for (int jc = j_begin; jc < j_end; jc += TK) {
        const int nk = min(TK, j_end - jc);
        sync();                                   // previous chunk fully consumed
        if (NPF > 0) {
#pragma unroll
            for (int u = 0; u < NPF; ++u) {
                const int i = tid + 128 * u;
                const int row = i / (HD / 8), part = i - row * (HD / 8);
                if (row < nk) {
                    uint32_t* kd = Kt + row * KS + part * 4;
                    kd[0] = kpre[u].x; kd[1] = kpre[u].y; kd[2] = kpre[u].z; kd[3] = kpre[u].w;
                    *reinterpret_cast<uint4*>(Vt + row * KW + part * 4) = vpre[u];
                }
            }
            // the next chunk's rows are requested now and arrive while this chunk is scored and summed
            if (jc + TK < j_end) prefetch(jc + TK, min(TK, j_end - jc - TK));
        } else
        for (int i = tid; i < nk * (HD / 8); i += 128) {
            const int row = i / (HD / 8), part = i - row * (HD / 8);
            const int j = jc + row;
            const int page = bt[j / a.page], slot = j % a.page;
            const size_t o = ((static_cast<size_t>(page) * a.n_kv + h) * a.page + slot) * HD + part * 8;
            const uint4 kv = *reinterpret_cast<const uint4*>(a.k_cache + o);
            const uint4 vv = *reinterpret_cast<const uint4*>(a.v_cache + o);
            uint32_t* kd = Kt + row * KS + part * 4;
            kd[0] = kv.x; kd[1] = kv.y; kd[2] = kv.z; kd[3] = kv.w;
            *reinterpret_cast<uint4*>(Vt + row * KW + part * 4) = vv;
        }
        if (has_new && pos >= jc && pos < jc + nk) {       // the new token's row comes from shared memory
            sync();
            const uint32_t* fk = reinterpret_cast<const uint32_t*>(fresh);
            for (int w = tid; w < KW; w += 128) { Kt[(pos - jc) * KS + w] = fk[w]; Vt[(pos - jc) * KW + w] = fk[KW + w]; }
        }
        sync();
        {   // scores: thread = (key, head parity); heads hg, hg+2, hg+4, hg+6 share each K word
            const int key = tid & 63, hg = tid >> 6;
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
            if (key < nk) {
                const uint32_t* kr = Kt + key * KS;
#pragma unroll 8
                for (int w = 0; w < KW; ++w) {
                    const uint32_t kw = kr[w];
                    const float k0 = __uint_as_float(kw << 16), k1 = __uint_as_float(kw & 0xFFFF0000u);
                    const float2 q0 = *reinterpret_cast<const float2*>(qs + hg * HD + 2 * w);
                    s0 = fmaf(q0.x, k0, fmaf(q0.y, k1, s0));
                    if (G > 2) { const float2 q1 = *reinterpret_cast<const float2*>(qs + (hg + 2) * HD + 2 * w); s1 = fmaf(q1.x, k0, fmaf(q1.y, k1, s1)); }
                    if (G > 4) { const float2 q2 = *reinterpret_cast<const float2*>(qs + (hg + 4) * HD + 2 * w); s2 = fmaf(q2.x, k0, fmaf(q2.y, k1, s2)); }
                    if (G > 6) { const float2 q3 = *reinterpret_cast<const float2*>(qs + (hg + 6) * HD + 2 * w); s3 = fmaf(q3.x, k0, fmaf(q3.y, k1, s3)); }
                }
            } else { s0 = s1 = s2 = s3 = -INFINITY; }
            if (hg < G) S[hg * TK + key] = s0;
            if (hg + 2 < G) S[(hg + 2) * TK + key] = s1;
            if (hg + 4 < G) S[(hg + 4) * TK + key] = s2;
            if (hg + 6 < G) S[(hg + 6) * TK + key] = s3;
        }
        sync();
        for (int hh = warp; hh < G; hh += 4) {             // online softmax, one warp per head
            const float v0 = S[hh * TK + lane], v1 = S[hh * TK + lane + 32];
            float mx = fmaxf(v0, v1);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
            const float mo = mrun[hh], mn = fmaxf(mo, mx);
            const float p0 = expf(v0 - mn), p1 = expf(v1 - mn);
            const float sum = attn_wsum(p0 + p1);
            S[hh * TK + lane] = p0; S[hh * TK + lane + 32] = p1;
            if (lane == 0) { const float c = expf(mo - mn); corr[hh] = c; lrun[hh] = lrun[hh] * c + sum; mrun[hh] = mn; }
        }
        sync();
#pragma unroll
        for (int p = 0; p < NP; ++p) {                     // acc = acc * corr + P V
            const int idx = tid + 128 * p;
            if (idx < G * KW) {
                const int gq = idx / KW, w = idx - gq * KW;
                const float c = corr[gq];
                float a0 = acc[p][0] * c, a1 = acc[p][1] * c;
                const float* pr = S + gq * TK;
                // two partial sums per output and eight keys per pass: the shared-memory loads of a pass are
                // all in flight before the first multiply-add needs one
                float b0 = 0.0f, b1 = 0.0f;
                int j = 0;
                for (; j + 8 <= nk; j += 8) {
                    uint32_t vw[8];
                    float pj[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) { vw[u] = Vt[(j + u) * KW + w]; pj[u] = pr[j + u]; }
#pragma unroll
                    for (int u = 0; u < 8; u += 2) {
                        a0 = fmaf(pj[u], __uint_as_float(vw[u] << 16), a0);
                        a1 = fmaf(pj[u], __uint_as_float(vw[u] & 0xFFFF0000u), a1);
                        b0 = fmaf(pj[u + 1], __uint_as_float(vw[u + 1] << 16), b0);
                        b1 = fmaf(pj[u + 1], __uint_as_float(vw[u + 1] & 0xFFFF0000u), b1);
                    }
                }
                for (; j < nk; ++j) {
                    const uint32_t v1 = Vt[j * KW + w];
                    const float p1 = pr[j];
                    a0 = fmaf(p1, __uint_as_float(v1 << 16), a0);
                    a1 = fmaf(p1, __uint_as_float(v1 & 0xFFFF0000u), a1);
                }
                acc[p][0] = a0 + b0; acc[p][1] = a1 + b1;
            }
        }
    }
    float* part = a.partial + ((static_cast<size_t>(t) * a.n_head + head0) * a.n_splits + split) * (HD + 2);
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        const int idx = tid + 128 * p;
        if (idx < G * KW) {
            const int gq = idx / KW, w = idx - gq * KW;
            float* pg = part + static_cast<size_t>(gq) * a.n_splits * (HD + 2);
            pg[2 + 2 * w] = acc[p][0]; pg[3 + 2 * w] = acc[p][1];
            if (w == 0) { pg[0] = mrun[gq]; pg[1] = lrun[gq]; }
        }
    }
    if (!a.merge_ticket) return;
    // ---- the last CTA of this (token, KV head) merges the splits ----
    // Every CTA publishes its partials (fence), then takes a ticket; the one that takes the last ticket sees all partials
    // (it reads them past L1) and owns the merge.  No CTA waits for another.
    const int n_active = min(a.n_splits, pos / keys_per_split + 1);
    if (n_active < a.merge_min_splits) return;                      // few splits: the consumer merges them in its prologue
    int* flag = reinterpret_cast<int*>(corr);                       // corr[] is free now
    __threadfence();
    sync();
    if (tid == 0) {
        int* ticket = a.merge_ticket + static_cast<size_t>(t) * a.n_kv + h;
        const int got = atomicAdd(ticket, 1);
        const int last = got == n_active - 1;
        if (last) *ticket = 0;                                      // every CTA of this (token, head) has taken its ticket
        flag[0] = last;
    }
    sync();
    if (!flag[0]) return;
    __threadfence();
    const float* base = a.partial + (static_cast<size_t>(t) * a.n_head + head0) * a.n_splits * (HD + 2);
    float* wts = reinterpret_cast<float*>(Kt);                      // [G][128]: exp(max_s - max) per head and split (n_splits <= 128;
    float* lsm = wts + 8 * 128;                                     // [G][128]: the splits' sums       the K tile is free now)
    for (int i = tid; i < G * n_active; i += 128) {                 // every split's (max, sum) by its own thread: independent loads
        const int gq = i / n_active, s2 = i - gq * n_active;
        const float* ps = base + (static_cast<size_t>(gq) * a.n_splits + s2) * (HD + 2);
        wts[gq * 128 + s2] = __ldcg(ps);
        lsm[gq * 128 + s2] = __ldcg(ps + 1);
    }
    sync();
    if (tid < G) {
        float mx = -INFINITY;
        for (int s2 = 0; s2 < n_active; ++s2) mx = fmaxf(mx, wts[tid * 128 + s2]);
        float lsum = 0.0f;
        for (int s2 = 0; s2 < n_active; ++s2) {
            const float wv = expf(wts[tid * 128 + s2] - mx);
            wts[tid * 128 + s2] = wv;
            lsum += lsm[tid * 128 + s2] * wv;
        }
        mrun[tid] = 1.0f / lsum;
    }
    sync();
    for (int idx = tid; idx < G * HD; idx += 128) {
        const int gq = idx / HD, d = idx - gq * HD;
        const float* pg = base + static_cast<size_t>(gq) * a.n_splits * (HD + 2) + 2 + d;
        float o = 0.0f;
        int s2 = 0;
        for (; s2 + 8 <= n_active; s2 += 8) {                       // eight loads in flight
            float pv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) pv[u] = __ldcg(pg + static_cast<size_t>(s2 + u) * (HD + 2));
#pragma unroll
            for (int u = 0; u < 8; ++u) o += pv[u] * wts[gq * 128 + s2 + u];
        }
        for (; s2 < n_active; ++s2) o += __ldcg(pg + static_cast<size_t>(s2) * (HD + 2)) * wts[gq * 128 + s2];
        a.out[(static_cast<size_t>(t) * a.n_head + head0 + gq) * HD + d] = o * mrun[gq];
    }
}

}  // namespace ggb
