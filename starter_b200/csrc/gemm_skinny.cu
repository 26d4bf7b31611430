// Weight-streaming matrix product for a handful of rows (decode): C[M,N] = A[M,K] * W[N,K]^T,
// bfloat16 in, 32-bit accumulate, M <= 32.
//
// Reference: engine/kernels/gemm.py:60-112 (one M tile, persistent grid over N tiles and K
// splits, 32-bit partial sums reduced afterwards) and :212-256 (CUDA-core GEMV for M <= 4).
// The work is bound by reading W once, so the kernel is built around that stream:
//  * the tensor cores see W as the 16-row operand of mma.sync m16n8k16 and the M activation
//    rows as the 8-column operand, so no lane is wasted on padding rows of A;
//  * a lane reads 16 contiguous bytes of a weight row at a time.  The instruction only needs
//    both operands to agree on which k sits where, so the k indices inside a block of 32 are
//    assigned to lanes in the order of those 16-byte reads, and the activations are read the
//    same way;
//  * a block owns 16 weight rows and one slice of K; its 8 warps walk the slice in turns of
//    128 columns each and meet in shared memory at the end;
//  * with 2 to 8 K slices per row block, the slices' blocks form a thread-block cluster and add their sums
//    through one another's shared memory; with more, partial sums go to scratch memory and the last
//    block to arrive adds them (an atomic counter per row block).  Either way the output is written once.
// Optional fusions: the SwiGLU epilogue for a fused [gate; up] matrix (engine/kernels/gemm.py:
// 116-168: both halves rounded to bfloat16, silu in 32-bit rounded, product rounded).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define GS_WARPS 8
#define GS_ROWS 16          // weight rows per block
#define GS_KWARP 128        // columns one warp covers per turn (4 blocks of 32)
#define GS_KTURN (GS_WARPS * GS_KWARP)
#define GS_MAX_CLUSTER 8    // K slices that meet through the cluster's shared memory

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned int a0, unsigned int a1, unsigned int a2,
                                               unsigned int a3, unsigned int b0, unsigned int b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
    // engine/kernels/gemm.py:116-121
    const float gb = __bfloat162float(__float2bfloat16_rn(g)), ub = __bfloat162float(__float2bfloat16_rn(u));
    const float s = __bfloat162float(__float2bfloat16_rn(gb / (1.0f + expf(-gb))));
    return s * ub;
}

// NT: activation tiles of 8 rows (M <= 8 * NT).  GATE_UP: W is [2 * n_out, K], gate rows first; the first half of
// the warps takes the gate rows of the block, the second half the matching up rows, and the output is swiglu(gate, up).
// TILED: W is the tile-major copy that sb_tile_matrix makes: [row tile of 16][turn of 128 columns][16 rows][128
// columns], rows and columns zero-padded to whole tiles (with GATE_UP: the gate half's tiles, then the up half's).
// What a warp reads in one turn is then one contiguous piece of 4 KB instead of sixteen pieces of 256 bytes a row
// apart, which memory serves faster (measured on the 4B shapes: the decode step 3.7% shorter at batch 8, 6.8% at batch 1).
template <int NT, bool GATE_UP, bool TILED, int WARPS, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 8 ? 4 : 8) / (NT > 2 ? 2 : 1))   // 64 registers; 128 from 17 rows on
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, void* __restrict__ C,
                   int M, int n_out, int K, int k_per_split, int n_splits, int out_f32,
                   float* __restrict__ partial, int* __restrict__ counters) {
    constexpr int GROUPS = GATE_UP ? 2 : 1;              // row groups the warps are divided into
    constexpr int WPG = WARPS / GROUPS;                  // warps per group, sharing K among them
    __shared__ float red[WARPS][GS_ROWS][8 * NT + 1];
    __shared__ int s_is_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int group = warp / WPG, wk = warp % WPG;
    const int n0 = blockIdx.x * GS_ROWS;
    const int split = blockIdx.y;
    const int k_begin = split * k_per_split, k_end = min(K, k_begin + k_per_split);
    const long long row_lo = (long long)group * n_out + n0 + g, row_hi = row_lo + 8;
    const bool ok_lo = n0 + g < n_out, ok_hi = n0 + g + 8 < n_out;
    const __nv_bfloat16* w_lo = W + row_lo * K;
    const __nv_bfloat16* w_hi = W + row_hi * K;
    // TILED: this lane's place in the first turn of the block's row tile (see the layout at the top of the file)
    const __nv_bfloat16* w_tile = W + ((long long)group * gridDim.x + blockIdx.x) * ((K + GS_KWARP - 1) / GS_KWARP) * (GS_ROWS * GS_KWARP) +
                                  g * GS_KWARP + c * 8;

    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // The weights of the next turn are requested before the current turn is multiplied, so that a
    // warp always has a turn's worth of loads (4 KB) in flight behind the one it works on.
    auto load_w = [&](uint4 (&lo)[4], uint4 (&hi)[4], int kt) {
        if (TILED) {   // whole turns exist, zero-padded: no edges; the turn is 4 KB in one piece
            const __nv_bfloat16* wt = w_tile + (long long)(kt / GS_KWARP) * (GS_ROWS * GS_KWARP);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                lo[u] = load_stream(wt + u * 32);
                hi[u] = load_stream(wt + 8 * GS_KWARP + u * 32);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k = kt + u * 32 + c * 8;
                const bool ok = k < k_end;
                lo[u] = ok && ok_lo ? load_stream(w_lo + k) : zero;
                hi[u] = ok && ok_hi ? load_stream(w_hi + k) : zero;
            }
        }
    };
    auto turn = [&](const uint4 (&lo)[4], const uint4 (&hi)[4], int kt) {
        uint4 x[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k = kt + u * 32 + c * 8;
                const int m = t * 8 + g;
                x[t][u] = (k < k_end && m < M) ? __ldg(reinterpret_cast<const uint4*>(A + (long long)m * K + k)) : zero;
            }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                mma_bf16_16816(acc[t], lo[u].x, hi[u].x, lo[u].y, hi[u].y, x[t][u].x, x[t][u].y);
                mma_bf16_16816(acc[t], lo[u].z, hi[u].z, lo[u].w, hi[u].w, x[t][u].z, x[t][u].w);
            }
    };
    constexpr int STRIDE = WPG * GS_KWARP;
    int kt = k_begin + wk * GS_KWARP;
    sb_stamp(2, 0);
    // The weights do not depend on the kernel before this one: a turn's weights are requested
    // before the wait for that kernel (which matters in the first turn only), the activations after it.
#pragma unroll 1
    for (; kt < k_end; kt += STRIDE) {
        uint4 lo[4], hi[4];
        load_w(lo, hi, kt);
        pdl_wait();
        turn(lo, hi, kt);
    }
    pdl_wait();   // a warp without a turn of its own waits too, before anything is written

    sb_stamp(2, 1);
    pdl_launch_dependents();   // the weights are read; the next kernel may start fetching its own
    // Warps meet: red[warp][weight row][activation row].
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        red[warp][g][t * 8 + c * 2] = acc[t][0];
        red[warp][g][t * 8 + c * 2 + 1] = acc[t][1];
        red[warp][g + 8][t * 8 + c * 2] = acc[t][2];
        red[warp][g + 8][t * 8 + c * 2 + 1] = acc[t][3];
    }
    __syncthreads();

    // Element e of the block's output: weight row r (and group), activation row m.
    constexpr int ELEMS = GROUPS * GS_ROWS * 8 * NT;
    const long long part_block = (long long)ELEMS;
    float* my_part = partial + ((long long)blockIdx.x * n_splits + split) * part_block;
    for (int e = tid; e < ELEMS; e += WARPS * 32) {
        const int grp = e / (GS_ROWS * 8 * NT), r = (e / (8 * NT)) % GS_ROWS, m = e % (8 * NT);
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WPG; ++w) v += red[grp * WPG + w][r][m];
        if (n_splits > 1 && !CLUSTER) {
            my_part[e] = v;
        } else {
            red[grp * WPG][r][m] = v;  // keep the block's sums for the epilogue (or for the cluster)
        }
    }
    if (CLUSTER) {
        // The blocks of this row block's K slices are one cluster (rank = slice).  Each finishes an equal share of
        // the outputs from the sums in all the blocks' shared memory, added in the order of the slices.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        constexpr int OUTS = GS_ROWS * 8 * NT;
        const int share = (OUTS + n_splits - 1) / n_splits;
        const int e_end = min(OUTS, (split + 1) * share);
        for (int e = split * share + tid; e < e_end; e += WARPS * 32) {
            const int r = e % GS_ROWS, m = e / GS_ROWS;
            if (m >= M || n0 + r >= n_out) continue;
            float v = 0.f, v2 = 0.f;
            for (int c = 0; c < n_splits; ++c) {
                v += *cluster.map_shared_rank(&red[0][r][m], c);
                if (GATE_UP) v2 += *cluster.map_shared_rank(&red[WPG][r][m], c);
            }
            if (GATE_UP) v = silu_mul_bf16(v, v2);
            const long long o = (long long)m * n_out + n0 + r;
            if (out_f32)
                reinterpret_cast<float*>(C)[o] = v;
            else
                reinterpret_cast<__nv_bfloat16*>(C)[o] = __float2bfloat16_rn(v);
        }
        cluster.sync();   // nobody leaves while its sums are still being read
        sb_stamp(2, 2);
        return;
    }
    if (n_splits > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) s_is_last = atomicAdd(&counters[blockIdx.x], 1) == n_splits - 1;
        __syncthreads();
        if (!s_is_last) return;
        __threadfence();
        const float* parts = partial + (long long)blockIdx.x * n_splits * part_block;
        for (int e = tid; e < ELEMS; e += WARPS * 32) {
            const int grp = e / (GS_ROWS * 8 * NT), r = (e / (8 * NT)) % GS_ROWS, m = e % (8 * NT);
            float v = 0.f;
            for (int s = 0; s < n_splits; ++s) v += __ldcg(parts + s * part_block + e);
            red[grp * WPG][r][m] = v;
        }
        if (tid == 0) counters[blockIdx.x] = 0;
    }
    __syncthreads();

    // Epilogue: one output element per (weight row r, activation row m); consecutive threads take
    // consecutive r so that a row of C is written in runs of 16.
    for (int e = tid; e < GS_ROWS * 8 * NT; e += WARPS * 32) {
        const int r = e % GS_ROWS, m = e / GS_ROWS;
        if (m >= M || n0 + r >= n_out) continue;
        float v = red[0][r][m];
        if (GATE_UP) v = silu_mul_bf16(v, red[WPG][r][m]);
        const long long o = (long long)m * n_out + n0 + r;
        if (out_f32)
            reinterpret_cast<float*>(C)[o] = v;
        else
            reinterpret_cast<__nv_bfloat16*>(C)[o] = __float2bfloat16_rn(v);
    }
    sb_stamp(2, 2);
}

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
// Takes M <= 32 and K a multiple of 8; k_per_split a multiple of 128.  tiled: W is the tile-major copy (see above).
int sb_gemm_skinny(const void* A, const void* W, void* C, int M, int n_out, int K, int n_splits, int k_per_split,
                   int gate_up, int out_f32, int tiled, int warps, float* partial, int* counters, cudaStream_t stream) {
    if (M <= 0 || n_out <= 0) return 0;
    if (M > 32 || (K & 7) || n_splits < 1 || n_splits > 65535 || (k_per_split % GS_KWARP) ||
        (long long)k_per_split * n_splits < K || (warps != 4 && warps != 8))
        return (int)cudaErrorInvalidValue;
    dim3 grid((n_out + GS_ROWS - 1) / GS_ROWS, n_splits);
    const int cluster_reduce = n_splits >= 2 && n_splits <= GS_MAX_CLUSTER;
    dim3 cluster(1, cluster_reduce ? n_splits : 1, 1);
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
#define SB_SKINNY3(NT, GU, TL, CL)                                                                                     \
    do {                                                                                                               \
        if (warps == 4)                                                                                                \
            sb_launch_cluster(gemm_skinny_kernel<NT, GU, TL, 4, CL>, grid, 128, cluster, 0, stream, a, w, C, M, n_out, K, \
                              k_per_split, n_splits, out_f32, partial, counters);                                      \
        else                                                                                                           \
            sb_launch_cluster(gemm_skinny_kernel<NT, GU, TL, 8, CL>, grid, 256, cluster, 0, stream, a, w, C, M, n_out, K, \
                              k_per_split, n_splits, out_f32, partial, counters);                                      \
    } while (0)
#define SB_SKINNY2(NT, GU, TL)                                                  \
    do {                                                                        \
        if (cluster_reduce) SB_SKINNY3(NT, GU, TL, true); else SB_SKINNY3(NT, GU, TL, false); \
    } while (0)
#define SB_SKINNY(NT, GU)                                                       \
    do {                                                                        \
        if (tiled) SB_SKINNY2(NT, GU, true); else SB_SKINNY2(NT, GU, false);    \
    } while (0)
    if (M <= 8) {
        if (gate_up) SB_SKINNY(1, true); else SB_SKINNY(1, false);
    } else if (M <= 16) {
        if (gate_up) SB_SKINNY(2, true); else SB_SKINNY(2, false);
    } else if (M <= 24) {
        if (gate_up) SB_SKINNY(3, true); else SB_SKINNY(3, false);
    } else {
        if (gate_up) SB_SKINNY(4, true); else SB_SKINNY(4, false);
    }
#undef SB_SKINNY
#undef SB_SKINNY2
#undef SB_SKINNY3
    SB_LAUNCH_CHECK();
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
