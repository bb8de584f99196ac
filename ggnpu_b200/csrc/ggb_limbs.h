// The int8-limb image of up to 16 activation rows: written once per call by rows_prep_kernel (ggb_gemv_mma_rows.cu),
// bulk-copied by the CTAs of the multi-row GEMV kernels (tensor-core layout: ggb_gemv_mma_rows.cu; stream layout:
// ggb_gemv_tma.cu).  x[m][k] * gamma[k] ~= xs[m][k / 256] * (l1 + l2 / 128 + l3 / 16384), |l| <= 127.
#pragma once
#include <stddef.h>
#include <cuda_runtime.h>

#include "ggb_internal.h"

namespace ggb {

//   planes int8 [M][3][K] (limbs l1, l2, l3) | asum float [M][K / 32] (sums of x * gamma over runs of 32)
//   | asum16 float [M][K / 16] | xs float [M][K / 256] (block scales) | inv_s float [16] (RMS factors; 1 without gamma)
struct LimbImage {
    size_t planes, asum, asum16, xs, inv_s, bytes;
    __host__ __device__ LimbImage(int M, int K) {
        planes = 0;
        asum = static_cast<size_t>(3) * M * K;
        asum16 = asum + sizeof(float) * static_cast<size_t>(M) * (K >> 5);
        xs = asum16 + sizeof(float) * static_cast<size_t>(M) * (K >> 4);
        inv_s = (xs + sizeof(float) * static_cast<size_t>(M) * (K >> 8) + 15) & ~static_cast<size_t>(15);
        bytes = inv_s + 64;
    }
};

// Make c->d_limbs hold the image of g's activations (g.M rows, K = g.w.K): launches rows_prep_kernel unless g.limbs_reuse
// is set and the very previous launch_gemv call left the image of the same source there.  The buffer must already be
// large enough (launch_gemv grows it outside stream capture).  K % 256 == 0, x 16-byte aligned, lda % 4 == 0.
int limb_image_prepare(Context* c, const GemvArgs& g, cudaStream_t s);

}  // namespace ggb
