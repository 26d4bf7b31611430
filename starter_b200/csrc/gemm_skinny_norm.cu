// The weight-streaming product of the RMSNorm of its activation rows (kernel: gemm_skinny.cuh, NORM), up to 16 rows.
// Reference: engine/kernels/gemm.py:29-56,60-112 (the norm-prologue variant of its skinny product).
#include "gemm_skinny.cuh"

extern "C" {

// C = rmsnorm(A; gamma, eps) * W^T (with gate_up: swiglu of it).  A [M, K] bfloat16, gamma [K] bfloat16; the other
// arguments as sb_gemm_skinny.  stats: what the product that wrote A left as its stats_out ([M][ceil(K / 16)]), or
// null: every block then reads all of A's rows once more for their statistics.
int sb_gemm_skinny_normed(const void* A, const void* gamma, float eps, const float* stats, const void* W, void* C, int M,
                          int n_out, int K, int n_splits, int k_per_split, int gate_up, int out_f32, int tiled, int warps,
                          int accumulate, float* stats_out, float* partial, int* counters, cudaStream_t stream) {
    if (gamma == nullptr) return (int)cudaErrorInvalidValue;
    return skinny_launch<true, 2>(A, W, C, M, n_out, K, n_splits, k_per_split, gate_up, out_f32, tiled, warps, accumulate,
                                  SbSkinnyNorm{(const __nv_bfloat16*)gamma, eps, stats, (K + GS_ROWS - 1) / GS_ROWS},
                                  stats_out, partial, counters, stream);
}

}  // extern "C"
SB_TIMELINE_SETTER(skinny_norm)
