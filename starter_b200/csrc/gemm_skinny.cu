// Entry points of the weight-streaming product without a norm (kernel and layout: gemm_skinny.cuh) and the
// tile-major copy of a weight matrix that it reads.
#include "gemm_skinny.cuh"

// dst element index -> (half, row tile, turn, row in tile, column in turn); 8 elements (16 bytes) per thread.
__global__ void tile_matrix_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int rows, int K,
                                   int halves, long long total) {
    const int kt_n = (K + GS_KWARP - 1) / GS_KWARP, rt_n = (rows + GS_ROWS - 1) / GS_ROWS;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += (long long)gridDim.x * blockDim.x * 8) {
        const int col = (int)(i % GS_KWARP);
        const int r_in = (int)((i / GS_KWARP) % GS_ROWS);
        const long long tile = i / (GS_ROWS * GS_KWARP);
        const int kt = (int)(tile % kt_n);
        const int rt = (int)((tile / kt_n) % rt_n);
        const int half = (int)(tile / ((long long)kt_n * rt_n));
        const int row = rt * GS_ROWS + r_in, k = kt * GS_KWARP + col;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows && k < K) v = *reinterpret_cast<const uint4*>(src + ((long long)half * rows + row) * K + k);   // K % 8 == 0
        *reinterpret_cast<uint4*>(dst + i) = v;
    }
}

extern "C" {

// Scratch for n_splits > 1: partial sums (floats) and one counter per row block (ints, zero before
// the first launch; the kernel leaves them zero).
long long sb_gemm_skinny_scratch_floats(int M, int n_out, int n_splits, int gate_up) {
    const int nt = (M + 7) / 8;
    const long long blocks = (n_out + GS_ROWS - 1) / GS_ROWS;
    return n_splits > 1 ? blocks * n_splits * (gate_up ? 2 : 1) * GS_ROWS * 8 * nt : 0;
}

// A [M, K], W [n_out, K] (or [2 * n_out, K] with gate_up), C [M, n_out] bfloat16 or float.
// Takes M <= 32 and K a multiple of 8; k_per_split a multiple of 128.  tiled: W is the tile-major copy (see
// gemm_skinny.cuh).  accumulate: C += product (bfloat16 C only).  stats_out (or null): [M][ceil(n_out / 16)] floats,
// the sums of squares of each block's 16 columns of every row of C as it now stands.
int sb_gemm_skinny(const void* A, const void* W, void* C, int M, int n_out, int K, int n_splits, int k_per_split,
                   int gate_up, int out_f32, int tiled, int warps, int accumulate, float* stats_out, float* partial,
                   int* counters, cudaStream_t stream) {
    return skinny_launch<false, 4>(A, W, C, M, n_out, K, n_splits, k_per_split, gate_up, out_f32, tiled, warps, accumulate,
                                   SbSkinnyNorm{nullptr, 0.f, nullptr, 0}, stats_out, partial, counters, stream);
}

// The tile-major copy of a row-major matrix for the kernel above.  src [halves * rows, K] bfloat16 row-major; dst
// holds halves * ceil(rows / 16) * ceil(K / 128) tiles of 16 x 128 (sb_tile_matrix_elements of them in all).
long long sb_tile_matrix_elements(int rows, int K, int halves) {
    return (long long)halves * ((rows + GS_ROWS - 1) / GS_ROWS) * ((K + GS_KWARP - 1) / GS_KWARP) * (GS_ROWS * GS_KWARP);
}

int sb_tile_matrix(const void* src, void* dst, int rows, int K, int halves, cudaStream_t stream) {
    if (rows <= 0 || K <= 0 || halves < 1) return (int)cudaErrorInvalidValue;
    const long long total = sb_tile_matrix_elements(rows, K, halves);
    const int blocks = (int)((total / 8 + 255) / 256 < 65535 * 16 ? (total / 8 + 255) / 256 : 65535 * 16);
    tile_matrix_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, rows, K, halves, total);
    SB_LAUNCH_CHECK();
}

}  // extern "C"

SB_TIMELINE_SETTER(skinny)
