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
// Optional fusions:
//  * the SwiGLU epilogue for a fused [gate; up] matrix (engine/kernels/gemm.py:116-168: both halves rounded to
//    bfloat16, silu in 32-bit rounded, product rounded);
//  * NORM, the RMSNorm of the activation rows in the prologue (engine/kernels/gemm.py:29-56: every block takes the
//    statistics of the whole rows it multiplies and norms its pieces on the fly, bf16(w * bf16(x * rstd)), so the
//    normed rows are never written).  Reading whole rows in every block costs more than the norm kernel it saves
//    (measured: 2.80 -> 2.99 ms a decode step at batch 8), so the statistics come from the product that wrote the
//    rows where there is one (below); a warp per row adds them in a fixed order, so a row's result does not depend
//    on the other rows of the batch;
//  * accumulate, an epilogue that adds the product to what C holds (32-bit sum of two bfloat16 values, rounded once:
//    the residual sum of engine/kernels/add_rmsnorm.py:21-24, taken here by the thread that owns the element).  With
//    it a block can leave the sum of squares of its 16 columns of every new row (stats_out [rows][row blocks]), which
//    is what the next product's NORM reads instead of the rows.
// With both, a pre-norm layer's branch is its products and nothing else: no norm kernel, no pass over the residual.
#pragma once
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
// What NORM needs: the norm's weight (bfloat16 [K]) and eps; and, if the rows were written by a product that left
// their statistics, those: stats[m * n_stats + i] is the sum of squares of piece i of row m (else nullptr: every
// block reads the rows themselves).
struct SbSkinnyNorm {
    const __nv_bfloat16* gamma;
    float eps;
    const float* stats;
    int n_stats;
};

// Stores one output and returns what C now holds there.
__device__ __forceinline__ float skinny_store(void* C, long long o, float v, int out_f32, int accumulate) {
    if (out_f32) {
        reinterpret_cast<float*>(C)[o] = v;
        return v;
    }
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(C);
    __nv_bfloat16 r = __float2bfloat16_rn(v);
    if (accumulate) r = __float2bfloat16_rn(__fadd_rn(__bfloat162float(c[o]), __bfloat162float(r)));
    c[o] = r;
    return __bfloat162float(r);
}

// The 16 lanes of a half-warp hold the 16 columns of one output row: their squares added in a fixed tree, left by
// the first of them.  Every lane of the half-warp must call it.
__device__ __forceinline__ void skinny_leave_stats(float* stats_out, float stored, bool row_ok, int m, int r) {
    float sq = stored * stored;
    const unsigned int half = 0xffffu << (threadIdx.x & 16);
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) sq += __shfl_xor_sync(half, sq, off);
    if (r == 0 && row_ok) stats_out[(long long)m * gridDim.x + blockIdx.x] = sq;
}

// Eight packed bfloat16 activations -> bf16(gamma * bf16(x * rstd)), pair by pair.  The product of two bfloat16
// values is exact in 32-bit, so the packed multiply with one rounding equals the 32-bit multiply rounded.
__device__ __forceinline__ uint4 normed8(uint4 x, uint4 gamma, float rstd) {
    uint4 out;
    const unsigned int* xi = reinterpret_cast<const unsigned int*>(&x);
    const __nv_bfloat162* gi = reinterpret_cast<const __nv_bfloat162*>(&gamma);
    __nv_bfloat162* oi = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float lo = __uint_as_float(xi[e] << 16), hi = __uint_as_float(xi[e] & 0xffff0000u);
        oi[e] = __hmul2_rn(__floats2bfloat162_rn(__fmul_rn(lo, rstd), __fmul_rn(hi, rstd)), gi[e]);
    }
    return out;
}

template <int NT, bool GATE_UP, bool TILED, int WARPS, bool CLUSTER, bool NORM>
__global__ void __launch_bounds__(WARPS * 32, (WARPS == 8 ? 4 : 8) / (NT > 2 ? 2 : 1))   // 64 registers; 128 from 17 rows on
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ W, void* __restrict__ C,
                   int M, int n_out, int K, int k_per_split, int n_splits, int out_f32, int accumulate, SbSkinnyNorm norm,
                   float* __restrict__ stats_out, float* __restrict__ partial, int* __restrict__ counters) {
    constexpr int GROUPS = GATE_UP ? 2 : 1;              // row groups the warps are divided into
    constexpr int WPG = WARPS / GROUPS;                  // warps per group, sharing K among them
    __shared__ float red[WARPS][GS_ROWS][8 * NT + 1];
    __shared__ int s_is_last;
    __shared__ float rstd_s[NORM ? 8 * NT : 1];
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
    float rstd[NT];   // NORM: of this lane's activation rows
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
        for (int u = 0; u < 4; ++u) {
            if (NORM) {   // the norm's weights for these columns come from L1 after the block's first turn
                const int k = kt + u * 32 + c * 8;
                const uint4 gm = k < k_end ? __ldg(reinterpret_cast<const uint4*>(norm.gamma + k)) : zero;
#pragma unroll
                for (int t = 0; t < NT; ++t) x[t][u] = normed8(x[t][u], gm, rstd[t]);
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                mma_bf16_16816(acc[t], lo[u].x, hi[u].x, lo[u].y, hi[u].y, x[t][u].x, x[t][u].y);
                mma_bf16_16816(acc[t], lo[u].z, hi[u].z, lo[u].w, hi[u].w, x[t][u].z, x[t][u].w);
            }
        }
    };
    constexpr int STRIDE = WPG * GS_KWARP;
    int kt = k_begin + wk * GS_KWARP;
    sb_stamp(2, 0);
    // The weights do not depend on the kernel before this one: a turn's weights are requested
    // before the wait for that kernel (which matters in the first turn only), the activations after it.
    if (NORM) {
        // The first turn's weights are on their way while the rows' statistics are taken: a warp per row, a lane
        // every 32nd piece, the lanes' sums added in a fixed tree.
        uint4 lo[4], hi[4];
        const bool has_turn = kt < k_end;
        if (has_turn) load_w(lo, hi, kt);
        pdl_wait();
        for (int m = warp; m < M; m += WARPS) {
            float ss = 0.f;
            if (norm.stats != nullptr) {
                for (int i = lane; i < norm.n_stats; i += 32) ss += __ldcg(norm.stats + (long long)m * norm.n_stats + i);
            } else {
                const __nv_bfloat16* row = A + (long long)m * K;
                for (int k = lane * 8; k < K; k += 256) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + k));
                    const unsigned int* vi = reinterpret_cast<const unsigned int*>(&v);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = __uint_as_float(vi[e] << 16), b = __uint_as_float(vi[e] & 0xffff0000u);
                        ss = fmaf(a, a, ss);
                        ss = fmaf(b, b, ss);
                    }
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            if (lane == 0) rstd_s[m] = 1.0f / sqrtf(ss / (float)K + norm.eps);
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < NT; ++t) rstd[t] = t * 8 + g < M ? rstd_s[t * 8 + g] : 0.f;
        if (has_turn) {
            turn(lo, hi, kt);
            kt += STRIDE;
        }
    }
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
        const int share = (8 * NT + n_splits - 1) / n_splits * GS_ROWS;   // whole activation rows
        const int e_end = min(OUTS, (split + 1) * share);
        for (int e = split * share + tid; e < e_end; e += WARPS * 32) {   // the lanes of a half-warp stay together
            const int r = e % GS_ROWS, m = e / GS_ROWS;
            float stored = 0.f;
            if (m < M && n0 + r < n_out) {
                float v = 0.f, v2 = 0.f;
                for (int c = 0; c < n_splits; ++c) {
                    v += *cluster.map_shared_rank(&red[0][r][m], c);
                    if (GATE_UP) v2 += *cluster.map_shared_rank(&red[WPG][r][m], c);
                }
                if (GATE_UP) v = silu_mul_bf16(v, v2);
                stored = skinny_store(C, (long long)m * n_out + n0 + r, v, out_f32, accumulate);
            }
            if (stats_out != nullptr) skinny_leave_stats(stats_out, stored, m < M, m, r);
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
        float stored = 0.f;
        if (m < M && n0 + r < n_out) {
            float v = red[0][r][m];
            if (GATE_UP) v = silu_mul_bf16(v, red[WPG][r][m]);
            stored = skinny_store(C, (long long)m * n_out + n0 + r, v, out_f32, accumulate);
        }
        if (stats_out != nullptr) skinny_leave_stats(stats_out, stored, m < M, m, r);
    }
    sb_stamp(2, 2);
}


// One launch: picks the instantiation for the rows, the layout and the way the K slices meet.  M <= 8 * MAX_NT.
template <bool NORM, int MAX_NT>
static int skinny_launch(const void* A, const void* W, void* C, int M, int n_out, int K, int n_splits, int k_per_split,
                         int gate_up, int out_f32, int tiled, int warps, int accumulate, SbSkinnyNorm norm, float* stats_out,
                         float* partial, int* counters, cudaStream_t stream) {
    if (M <= 0 || n_out <= 0) return 0;
    if (M > 8 * MAX_NT || (K & 7) || n_splits < 1 || n_splits > 65535 || (k_per_split % GS_KWARP) ||
        (long long)k_per_split * n_splits < K || (warps != 4 && warps != 8) || (accumulate && out_f32) ||
        (stats_out != nullptr && out_f32) || (norm.stats != nullptr && norm.n_stats != (K + GS_ROWS - 1) / GS_ROWS))
        return (int)cudaErrorInvalidValue;
    dim3 grid((n_out + GS_ROWS - 1) / GS_ROWS, n_splits);
    const int cluster_reduce = n_splits >= 2 && n_splits <= GS_MAX_CLUSTER;
    dim3 cluster(1, cluster_reduce ? n_splits : 1, 1);
    const __nv_bfloat16* a = (const __nv_bfloat16*)A;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
#define SB_SKINNY3(NT, GU, TL, CL)                                                                                     \
    do {                                                                                                               \
        if (warps == 4)                                                                                                \
            sb_launch_cluster(gemm_skinny_kernel<NT, GU, TL, 4, CL, NORM>, grid, 128, cluster, 0, stream, a, w, C, M, n_out, K, \
                              k_per_split, n_splits, out_f32, accumulate, norm, stats_out, partial, counters);         \
        else                                                                                                           \
            sb_launch_cluster(gemm_skinny_kernel<NT, GU, TL, 8, CL, NORM>, grid, 256, cluster, 0, stream, a, w, C, M, n_out, K, \
                              k_per_split, n_splits, out_f32, accumulate, norm, stats_out, partial, counters);         \
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
    } else if (M <= 16 || MAX_NT <= 2) {
        if (gate_up) SB_SKINNY(2, true); else SB_SKINNY(2, false);
    } else if (M <= 24) {
        if (gate_up) SB_SKINNY((MAX_NT > 2 ? 3 : 2), true); else SB_SKINNY((MAX_NT > 2 ? 3 : 2), false);
    } else {
        if (gate_up) SB_SKINNY((MAX_NT > 2 ? 4 : 2), true); else SB_SKINNY((MAX_NT > 2 ? 4 : 2), false);
    }
#undef SB_SKINNY
#undef SB_SKINNY2
#undef SB_SKINNY3
    SB_LAUNCH_CHECK();
}
