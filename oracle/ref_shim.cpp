// ref_shim.cpp -- C entry points over the UNMODIFIED reference sources, so that
// Python tests can call the reference's own functions and pin the C restatement
// (ggb_oracle.c) to them bit for bit.  TEST INFRASTRUCTURE ONLY.
//
// It is compiled together with the reference's .cpp files where they lie (see
// oracle/Makefile, REF=<path to the ggnpu tree>); nothing from the reference is
// copied into this repository.  The CLI translation unit is pulled in with
// `main` renamed so its file-local helpers (dequant_tensor_row, RopeCache,
// compute_logits) become callable.
#define main ggnpu_reference_cli_main
#include "src/cli/main.cpp"
#undef main

#include "quant/iq4_nl.h"
#include "quant/iq4_xs.h"
#include "quant/kquant.h"
#include "quant/q4_0.h"
#include "quant/q4_1.h"
#include "quant/q8_0.h"

namespace ggnpu {
// The reference CLI only links when an NPU factory exists.  This one hands back
// the reference's own CPU backend, so every operator call made by the CLI lands
// in src/backends/cpu_ref/cpu_ref.cpp.
std::shared_ptr<Backend> create_amd_xdna_backend(int) { return create_cpu_ref_backend(); }
}  // namespace ggnpu

using namespace ggnpu;

static std::shared_ptr<Backend>& cpu_backend() {
    static std::shared_ptr<Backend> b = create_cpu_ref_backend();
    return b;
}

extern "C" {

int ref_cli_main(int argc, char** argv) { return ggnpu_reference_cli_main(argc, argv); }

int ref_block_elems(uint32_t t) { return static_cast<int>(ggml_blck_size(static_cast<GgmlType>(t))); }
int ref_block_bytes(uint32_t t) { return static_cast<int>(ggml_type_size(static_cast<GgmlType>(t))); }

float ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
float ref_kquant_fp16_to_f32(uint16_t h) { return fp16_to_f32(h); }
float ref_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
uint16_t ref_f32_to_bf16(float f) { return f32_to_bf16(f); }

int ref_dequant_block(uint32_t type, const uint8_t* blk, float* out) {
    switch (static_cast<GgmlType>(type)) {
    case GgmlType::Q4_0: dequant_q4_0_block(blk, out); return 0;
    case GgmlType::Q4_1: dequant_q4_1_block(blk, out); return 0;
    case GgmlType::Q8_0: dequant_q8_0_block(blk, out); return 0;
    case GgmlType::Q2_K: dequant_q2_k_block(blk, out); return 0;
    case GgmlType::Q3_K: dequant_q3_k_block(blk, out); return 0;
    case GgmlType::Q4_K: dequant_q4_k_block(blk, out); return 0;
    case GgmlType::Q5_K: dequant_q5_k_block(blk, out); return 0;
    case GgmlType::Q6_K: dequant_q6_k_block(blk, out); return 0;
    case GgmlType::IQ4_NL: dequant_iq4_nl_block(blk, out); return 0;
    case GgmlType::IQ4_XS: dequant_iq4_xs_block(blk, out); return 0;
    case GgmlType::IQ2_XXS: dequant_iq2_xxs_block(blk, out); return 0;
    case GgmlType::IQ2_XS: dequant_iq2_xs_block(blk, out); return 0;
    case GgmlType::IQ2_S: dequant_iq2_s_block(blk, out); return 0;
    case GgmlType::IQ3_XXS: dequant_iq3_xxs_block(blk, out); return 0;
    case GgmlType::IQ3_S: dequant_iq3_s_block(blk, out); return 0;
    case GgmlType::IQ1_S: dequant_iq1_s_block(blk, out); return 0;
    case GgmlType::IQ1_M: dequant_iq1_m_block(blk, out); return 0;
    default: return -1;
    }
}

// The CLI's row decoder (file-local in src/cli/main.cpp).
void ref_dequant_tensor_row(uint32_t type, const uint8_t* data, int row, int K, float* out) {
    TensorView tv;
    tv.type = static_cast<GgmlType>(type);
    tv.data = data;
    dequant_tensor_row(&tv, row, out, K);
}

// The CLI's exact matmul: dequant_tensor_row + running fp32 dot, per row of A.
void ref_matmul_exact(const float* A, int M, int lda, const uint8_t* W, uint32_t type, int N, int K,
                      float* C, int ldc) {
    TensorView tv;
    tv.type = static_cast<GgmlType>(type);
    tv.data = W;
    std::vector<float> wr(static_cast<size_t>(K));
    for (int n = 0; n < N; n++) {
        dequant_tensor_row(&tv, n, wr.data(), K);
        for (int m = 0; m < M; m++) {
            const float* a = A + static_cast<size_t>(m) * lda;
            float acc = 0.0f;
            for (int k = 0; k < K; k++) acc += a[k] * wr[static_cast<size_t>(k)];
            C[static_cast<size_t>(m) * ldc + n] = acc;
        }
    }
}

void ref_rope_table(int64_t max_pos, int n_dims, float scale, float base, const float* ff, int n_ff,
                    float* cos_out, float* sin_out) {
    RopeCache rc;
    std::vector<float> f(ff, ff + (ff ? n_ff : 0));
    rc.build(max_pos, n_dims, scale, base, f);
    std::memcpy(cos_out, rc.cos.data(), rc.cos.size() * sizeof(float));
    std::memcpy(sin_out, rc.sin.data(), rc.sin.size() * sizeof(float));
}

int ref_mul_mat_q(const float* A, const void* B, float* C, int M, int N, int K, uint32_t type) {
    MulMatParams p{};
    p.A = A; p.B = B; p.C = C; p.M = M; p.N = N; p.K = K; p.lda = K; p.ldb = K; p.ldc = N;
    p.n_batches = 1; p.B_type = static_cast<GgmlType>(type);
    return static_cast<int>(cpu_backend()->mul_mat_q(p));
}

int ref_rms_norm(const float* in, float* out, int n, float eps, const float* w) {
    RmsNormParams p{}; p.input = in; p.output = out; p.size = n; p.eps = eps; p.weight = w;
    return static_cast<int>(cpu_backend()->rms_norm(p));
}

int ref_rope(float* data, int n_dims, int64_t offset, float freq_scale, float freq_base, int64_t rope_dims) {
    RopeParams p{}; p.data = data; p.n_dims = n_dims; p.offset = offset; p.freq_scale = freq_scale;
    p.freq_base = freq_base; p.rope_dims = rope_dims;
    return static_cast<int>(cpu_backend()->rope(p));
}

int ref_softmax(const float* in, float* out, int rows, int cols) {
    SoftmaxParams p{}; p.input = in; p.output = out; p.rows = rows; p.cols = cols;
    return static_cast<int>(cpu_backend()->softmax(p));
}

int ref_silu(const float* in, float* out, int n) {
    SiluParams p{}; p.input = in; p.output = out; p.size = n;
    return static_cast<int>(cpu_backend()->silu(p));
}

int ref_gelu(const float* in, float* out, int n) {
    GeluParams p{}; p.input = in; p.output = out; p.size = n;
    return static_cast<int>(cpu_backend()->gelu(p));
}

int ref_flash_attn(const float* Q, const float* K, const float* V, float* out, int n_head, int head_dim,
                   int64_t ctx_len, int64_t query_pos) {
    AttnParams p{}; p.Q = Q; p.K = K; p.V = V; p.output = out; p.batch_size = 1; p.n_head = n_head;
    p.head_dim = head_dim; p.ctx_len = ctx_len; p.query_pos = query_pos; p.freq_factors = nullptr;
    return static_cast<int>(cpu_backend()->flash_attn(p));
}

int ref_argmax(const float* logits, int n) {
    std::vector<float> v(logits, logits + n);
    uint64_t seed = 0;
    return sample_token(v, 0.0f, seed);
}

}  // extern "C"
