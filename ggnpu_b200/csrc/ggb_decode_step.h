// Argument blocks of the persistent decode-step kernel (ggb_decode_step.cu).
#pragma once
#include <stdint.h>

#include "ggb_attn.h"
#include "ggb_formats.cuh"

namespace ggb {

struct Context;

// One packed Q4_K / Q6_K matrix (row-group-major layout) and where its product goes.
struct StepMat {
    const uint8_t* s[4];      // the format's streams (ggb_formats.cuh)
    uint32_t type;
    int nb;                   // 256-blocks per row
    int64_t N;                // rows
    float* y;                 // output vector (the residual stream itself for the projections that add to it)
};

// Work split of one GEMV phase; the same for every layer.
struct StepShape {
    int K, nb;
    int groups;               // row groups of 16 over the stacked matrices (gate/up pair: of one matrix)
    int nmat;                 // 2: gate/up pair (both matrices of a row group go to the same team); else 1
    int ncat;                 // matrices stacked along N (q, k, v share the input row)
    int g_start[3];           // first row group of stacked matrix i
    int ws, log_ws;           // warps per row group (1, 2, 4 or 8) and its log2
    int sb4, sb6;             // 256-blocks per tile for Q4_K / Q6_K matrices
    int spr4, spr6;           // tiles per (row group, matrix) = ceil(nb / sb)
    int g_begin, n_rg;        // this CTA's range of row groups (filled in by each CTA at kernel start)
};

enum : int { kPhaseQkv = 0, kPhaseO = 1, kPhaseGateUp = 2, kPhaseDown = 3, kPhaseLogits = 4, kPhaseCount = 5 };

struct StepLayer {
    StepMat q, k, v, o, gate, up, down;
    const float *attn_norm, *ffn_norm;
    __nv_bfloat16 *k_cache, *v_cache;     // this layer's pages
};

struct StepArgs {
    const StepLayer* layers;  // device array
    int n_layer;
    StepMat out;              // logits matrix
    const float* out_norm;
    StepShape shape[kPhaseCount];
    const float* x;           // residual stream (the embedding row on entry)
    const float* act;         // SwiGLU output
    AttnPagedArgs attn;       // attention arguments without the per-layer cache pointers (fuse = 1)
    float eps;
    int k_max;                // largest K of any phase
    int n_cta;
    int P;                    // ring stages per consumer warp           (set by launch_decode_step)
    int fixed_bytes;          // shared memory after the rings           (set by launch_decode_step)
    unsigned* bar;            // grid barrier counter (device)
    int* err;
};

bool step_mat_ok(const PackedW& w);
StepMat step_mat(const PackedW& w, float* y);
void step_shape_init(StepShape& sh, int K, int64_t n0, int64_t n1, int64_t n2, bool dual, int n_cta);
// GGB_NOT_FOUND: the shapes do not fit the kernel's shared memory
int launch_decode_step(Context* c, StepArgs& a, int head_dim, cudaStream_t s);

}  // namespace ggb
