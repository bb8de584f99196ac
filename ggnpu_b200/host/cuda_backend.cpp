// ggnpu::Backend implemented on libggb200.so -- the C++ side of the drop-in.
//
// This file is written to be compiled INSIDE the ggnpu tree (it includes ggnpu's own
// include/ggnpu/backend.h) next to src/backends/amd_xdna/, and linked with -lggb200.  It adds one
// factory, create_cuda_b200_backend(int), with the shape of create_amd_xdna_backend
// (include/ggnpu/backend.h:162-165).  With -DGGB_ALIAS_XDNA_FACTORY it also defines
// create_amd_xdna_backend itself, so the unmodified CLI (src/cli/main.cpp:1031,1127,1445), built with
// GGNPU_HAS_NPU_BACKEND, runs on the GPU without a source change.
//
// Behaviour carried over from the NPU backend (src/backends/amd_xdna/amd_xdna.cpp):
//   * every operator completes before it returns; sync() only drains the stream (:2036-2039);
//   * a failed construction yields a backend whose is_available() is false (:448-458, :2041-2043);
//   * no exception leaves a method; errors are Status codes with a sticky last_error().
// name() is "cuda_b200": the CLI then passes raw GGUF blocks as MulMatParams::B
// (src/cli/main.cpp:1430-1432) instead of the NPU's int8 re-quantisation.
#include <memory>
#include <string>

#include "backend.h"
#include "ggb200.h"

namespace ggnpu {

namespace {

Status to_status(int s) {
    switch (s) {
    case GGB_OK: return Status::OK;
    case GGB_NOT_FOUND: return Status::NOT_FOUND;
    case GGB_INVALID_PARAM: return Status::INVALID_PARAM;
    case GGB_UNAVAILABLE: return Status::NPU_UNAVAILABLE;
    case GGB_OUT_OF_MEMORY: return Status::OUT_OF_MEMORY;
    default: return Status::ERROR;
    }
}

class CudaB200Backend final : public Backend {
public:
    explicit CudaB200Backend(int device) { create_status_ = ggb_create(device, &h_); }
    ~CudaB200Backend() override { ggb_destroy(h_); }

    Status mul_mat_q(const MulMatParams& p) override {
        ggb_mul_mat_params q{};
        q.A = p.A; q.B = p.B; q.C = p.C; q.M = p.M; q.N = p.N; q.K = p.K;
        q.lda = p.lda; q.ldb = p.ldb; q.ldc = p.ldc; q.n_batches = p.n_batches;
        q.scales = p.scales; q.n_weight_scales = p.n_weight_scales;
        q.B_type = static_cast<uint32_t>(p.B_type);
        return call(ggb_mul_mat_q(h_, &q));
    }
    Status rms_norm(const RmsNormParams& p) override {
        ggb_rms_norm_params q{p.input, p.output, p.size, p.eps, p.weight};
        return call(ggb_rms_norm(h_, &q));
    }
    Status rope(const RopeParams& p) override {
        ggb_rope_params q{p.data, p.n_dims, p.offset, p.freq_scale, p.freq_base, p.rope_dims, p.cos_table, p.sin_table,
                          static_cast<uint8_t>(p.neox_split_half)};
        return call(ggb_rope(h_, &q));
    }
    Status rope_batched(const RopeBatchedParams& p) override {
        ggb_rope_batched_params q{p.data, p.n_heads, p.n_dims, p.offset, p.freq_scale, p.freq_base, p.rope_dims,
                                  p.cos_table, p.sin_table, static_cast<uint8_t>(p.neox_split_half)};
        return call(ggb_rope_batched(h_, &q));
    }
    Status matmul_bf16(const float* A, const float* B, float* C, int M, int N, int K) override {
        return call(ggb_matmul_bf16(h_, A, B, C, M, N, K));
    }
    Status softmax(const SoftmaxParams& p) override {
        ggb_softmax_params q{p.input, p.output, p.rows, p.cols};
        return call(ggb_softmax(h_, &q));
    }
    Status silu(const SiluParams& p) override {
        ggb_unary_params q{p.input, p.output, p.size};
        return call(ggb_silu(h_, &q));
    }
    Status gelu(const GeluParams& p) override {
        ggb_unary_params q{p.input, p.output, p.size};
        return call(ggb_gelu(h_, &q));
    }
    Status flash_attn(const AttnParams& p) override {
        ggb_attn_params q{p.Q, p.K, p.V, p.output, p.batch_size, p.n_head, p.head_dim, p.ctx_len, p.query_pos, p.freq_factors};
        return call(ggb_flash_attn(h_, &q));
    }
    void sync() override { if (h_) ggb_sync(h_); }
    bool is_available() const override { return h_ != nullptr && create_status_ == GGB_OK; }
    std::string name() const override { return "cuda_b200"; }
    Status last_error() const override { return last_; }

private:
    Status call(int rc) {
        if (!h_) return last_ = Status::NPU_UNAVAILABLE;
        const Status s = to_status(rc);
        if (s != Status::OK) last_ = s;
        return s;
    }
    ggb_handle h_ = nullptr;
    int create_status_ = GGB_UNAVAILABLE;
    Status last_ = Status::OK;
};

}  // namespace

std::shared_ptr<Backend> create_cuda_b200_backend(int device_id) {
    return std::make_shared<CudaB200Backend>(device_id);
}

#ifdef GGB_ALIAS_XDNA_FACTORY
std::shared_ptr<Backend> create_amd_xdna_backend(int device_id) { return create_cuda_b200_backend(device_id); }
#endif

}  // namespace ggnpu
