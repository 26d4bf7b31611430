// Weight-streaming matrix product for decode on the Blackwell tensor cores:
//   C[M, N] = A[M, K] * W[N, K]^T  (optionally swiglu over a fused [gate; up] W), M <= 64,
// bfloat16 in, 32-bit accumulate in tensor memory, operands brought in by TMA.
//
// Reference: engine/kernels/gemm.py:60-181 (persistent grid over tiles and K splits so that the
// weights stream through all SMs in whole waves, 32-bit partial sums, SwiGLU epilogue with the
// roundings of :116-121).  The step is bound by reading W once, so:
//  * W is the 128-row operand of tcgen05.mma (cta_group::1, kind::f16) and the M activation rows,
//    padded by TMA's zero fill to 16/32/64, are the N operand: no tensor-core row is spent on padding;
//  * both operands arrive by cp.async.bulk.tensor (128-byte swizzle) into a ring of stages, so a
//    block keeps 140-200 KB of loads in flight with one producer thread and no registers;
//  * the work is cut into units of (128-row tile of W, 64-column block of K) and every block gets
//    the same number of consecutive units, whatever the shape: no wave is left partly filled.  A tile
//    whose units fall to several blocks is finished by the last of them to arrive (partial sums in
//    scratch memory, one counter per tile);
//  * accumulators are double-buffered in tensor memory: the four epilogue warps drain one tile
//    (tcgen05.ld) while the MMA thread already works on the next.
// One block per SM: warp 0 = TMA producer, warp 1 = MMA issuer and tensor-memory owner, warps 2-5 =
// epilogue.  Every wait on an mbarrier gives up after a bounded time, raises SB_STATUS_TIMEOUT in the
// status word, and the block leaves through its normal teardown (tensor memory freed).
#include <cuda.h>
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "tc_utils.cuh"

#define ST_BM 128               // rows of W per tile
#define ST_BK 64                // columns of K per stage: 128 bytes, one swizzle span
#define ST_THREADS 192

__device__ __forceinline__ float silu_mul_rounded(float g, float u) {
    // engine/kernels/gemm.py:116-121
    const float gb = __bfloat162float(__float2bfloat16_rn(g)), ub = __bfloat162float(__float2bfloat16_rn(u));
    const float s = __bfloat162float(__float2bfloat16_rn(gb / (1.0f + expf(-gb))));
    return s * ub;
}

// ---- the kernel ---------------------------------------------------------------------------------

struct StreamArgs {
    void* C;             // [M, n_out] bfloat16 or float
    float* partial;      // scratch: [tile][max_parts][128][acc_cols] floats
    int* counters;       // one per tile, zero before the first launch; the kernel leaves them zero
    int* status;
    int M, n_out, K;
    int n_tiles, k_blocks, max_parts;
    int out_f32;
#ifdef SB_TIMELINE
    long long* timeline;  // tuning builds only: [block][16] globaltimer stamps of the block's milestones
#endif
};

#ifdef SB_TIMELINE
__device__ __forceinline__ void stamp(const StreamArgs& args, int slot) {
    if (args.timeline) {
        long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        args.timeline[blockIdx.x * 16 + slot] = t;
    }
}
#else
#define stamp(args, slot) ((void)0)
#endif

// Units [u0, u1) of block c out of P, with U units in all.
__device__ __forceinline__ long long unit_begin(long long c, long long U, long long P) { return c * U / P; }
__device__ __forceinline__ int block_of_unit(long long x, long long U, long long P) {
    long long c = x * P / U;
    while (c + 1 < P && unit_begin(c + 1, U, P) <= x) ++c;
    while (c > 0 && unit_begin(c, U, P) > x) --c;
    return (int)c;
}

// BN: activation rows per MMA (16, 32 or 64); GATE_UP: W is [gate; up], two accumulators per tile.
template <int BN, bool GATE_UP, int STAGES>
__global__ void __launch_bounds__(ST_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_a, StreamArgs args) {
    constexpr int A_BYTES = ST_BM * ST_BK * 2;          // one tile of W per stage (two with GATE_UP)
    constexpr int B_BYTES = BN * ST_BK * 2;
    constexpr int N_A = GATE_UP ? 2 : 1;
    constexpr int ACC_COLS = N_A * BN;                  // columns of tensor memory per accumulator buffer
    constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_s = smem;                                   // [STAGES][N_A][128][64]
    unsigned char* b_s = smem + STAGES * N_A * A_BYTES;          // [STAGES][BN][64]
    uint64_t* bars = (uint64_t*)(b_s + STAGES * B_BYTES);
    uint64_t* full = bars;                  // [STAGES]  TMA -> MMA
    uint64_t* empty = bars + STAGES;        // [STAGES]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES; // [2]       MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;     // [2]       epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* last_flag = (int*)(tmem_slot + 2);
    int* wait_flag = (int*)(tmem_slot + 3);   // [2]: did the epilogue's wait for an item succeed

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long U = (long long)args.n_tiles * args.k_blocks, P = gridDim.x;
    const long long u0 = unit_begin(blockIdx.x, U, P), u1 = unit_begin(blockIdx.x + 1, U, P);

    if (threadIdx.x == 0) {
        stamp(args, 0);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: one TMA box of W (two with GATE_UP) and one of the activations per unit ----
        // The weights do not depend on the kernel before this one: the first ring of stages is
        // requested before the wait for that kernel, the activations of those stages after it.
        const int pre = (int)min((long long)STAGES, u1 - u0);
        for (int i = 0; i < pre; ++i) {
            const long long u = u0 + i;
            const int tile = (int)(u / args.k_blocks), kb = (int)(u % args.k_blocks);
            mbar_expect_tx(&full[i], N_A * A_BYTES + B_BYTES);
            tma_load_2d(a_s + (i * N_A) * A_BYTES, &map_w, kb * ST_BK, tile * ST_BM, &full[i]);
            if (GATE_UP) tma_load_2d(a_s + (i * N_A + 1) * A_BYTES, &map_w2, kb * ST_BK, tile * ST_BM, &full[i]);
        }
        stamp(args, 1);
        pdl_wait();
        stamp(args, 2);
        for (int i = 0; i < pre; ++i)
            tma_load_2d(b_s + i * B_BYTES, &map_a, (int)((u0 + i) % args.k_blocks) * ST_BK, 0, &full[i]);
        int stage = pre % STAGES;
        uint32_t phase = pre == STAGES ? 1 : 0;
        bool ok = true;
        for (long long u = u0 + pre; u < u1 && ok; ++u) {
            const int tile = (int)(u / args.k_blocks), kb = (int)(u % args.k_blocks);
            ok = mbar_wait<true>(&empty[stage], phase ^ 1, abort_flag, args.status);
            if (!ok) break;
            mbar_expect_tx(&full[stage], N_A * A_BYTES + B_BYTES);
            tma_load_2d(a_s + (stage * N_A) * A_BYTES, &map_w, kb * ST_BK, tile * ST_BM, &full[stage]);
            if (GATE_UP) tma_load_2d(a_s + (stage * N_A + 1) * A_BYTES, &map_w2, kb * ST_BK, tile * ST_BM, &full[stage]);
            tma_load_2d(b_s + stage * B_BYTES, &map_a, kb * ST_BK, 0, &full[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        stamp(args, 3);
        pdl_launch_dependents();   // every load of this block is requested: the next kernel may start fetching
        if (!ok) {
            // Leaving early: give the copies already requested a bounded time to land before the block's
            // shared memory goes away.
            const long long t0 = clock64();
            while (clock64() - t0 < (1ll << 22)) __nanosleep(64);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        pdl_wait();
        const uint32_t idesc = umma_idesc(BN);
        int stage = 0;
        uint32_t phase = 0, acc_phase[2] = {0, 0};
        int item = 0;
        bool ok = true;
        for (long long u = u0; u < u1 && ok; ++item) {
            const int kb0 = (int)(u % args.k_blocks);
            const int n_kb = (int)min((long long)(args.k_blocks - kb0), u1 - u);
            const int buf = item & 1;
            ok = mbar_wait<true>(&acc_empty[buf], acc_phase[buf] ^ 1, abort_flag, args.status);
            if (!ok) break;
            acc_phase[buf] ^= 1;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * ACC_COLS;
            for (int i = 0; i < n_kb && ok; ++i) {
                ok = mbar_wait<true>(&full[stage], phase, abort_flag, args.status);
                if (!ok) break;
                if (item == 0 && i == 0) stamp(args, 5);
                tc_fence_after();
                const uint64_t b_desc = desc_k_major(b_s + stage * B_BYTES);
#pragma unroll
                for (int a = 0; a < N_A; ++a) {
                    const uint64_t a_desc = desc_k_major(a_s + (stage * N_A + a) * A_BYTES);
#pragma unroll
                    for (int k = 0; k < ST_BK / 16; ++k)   // 16 columns = 32 bytes = 2 descriptor units per step
                        tc_mma(d_tmem + a * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&empty[stage]);   // frees the stage when these MMAs have read it
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) tc_commit(&acc_full[buf]);
            u += n_kb;
        }
        stamp(args, 4);
    } else if (warp >= 2) {
        // ---- epilogue: warp w drains lanes 32 * (w % 4) .. + 31 of tensor memory = rows of the tile ----
        pdl_wait();
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        uint32_t acc_phase[2] = {0, 0};
        int item = 0;
        bool ok = true;
        for (long long u = u0; u < u1 && ok; ++item) {
            const int tile = (int)(u / args.k_blocks), kb0 = (int)(u % args.k_blocks);
            const int n_kb = (int)min((long long)(args.k_blocks - kb0), u1 - u);
            const int buf = item & 1;
            const bool whole = n_kb == args.k_blocks;
            // One thread waits and tells the others, so that all four warps go on or all four leave.
            if (threadIdx.x == 64) wait_flag[buf] = mbar_wait<true>(&acc_full[buf], acc_phase[buf], abort_flag, args.status) ? 1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            ok = wait_flag[buf] != 0;
            if (!ok) break;
            if (threadIdx.x == 64) stamp(args, 8);
            acc_phase[buf] ^= 1;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
            const int n_row = tile * ST_BM + row_in_tile;     // output column = row of W
            int first_block = 0, parts = 1;
            if (!whole) {
                first_block = block_of_unit((long long)tile * args.k_blocks, U, P);
                parts = block_of_unit((long long)tile * args.k_blocks + args.k_blocks - 1, U, P) - first_block + 1;
            }
            // Partial sums of a tile: [tile][part][row][column], a thread's columns side by side.
            float* my_part = args.partial +
                (((long long)tile * args.max_parts + (blockIdx.x - first_block)) * ST_BM + row_in_tile) * ACC_COLS;
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= args.M) break;   // columns beyond the activation rows hold zeros nobody reads
                float g[16], up[16];
                tc_ld16(taddr + c0, g);
                if (GATE_UP) tc_ld16(taddr + BN + c0, up);
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c0 + j;
                        if (m < args.M && n_row < args.n_out) {
                            const float v = GATE_UP ? silu_mul_rounded(g[j], up[j]) : g[j];
                            const long long o = (long long)m * args.n_out + n_row;
                            if (args.out_f32) ((float*)args.C)[o] = v;
                            else ((__nv_bfloat16*)args.C)[o] = __float2bfloat16_rn(v);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        if (c0 + j >= args.M) break;
                        *reinterpret_cast<float4*>(my_part + c0 + j) = make_float4(g[j], g[j + 1], g[j + 2], g[j + 3]);
                        if (GATE_UP)
                            *reinterpret_cast<float4*>(my_part + BN + c0 + j) = make_float4(up[j], up[j + 1], up[j + 2], up[j + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);   // the MMA thread may reuse this accumulator
            if (threadIdx.x == 64) stamp(args, 9);
            if (!whole) {
                // The last block to finish its share of this tile adds the shares up, in the order of the
                // blocks, so the sum does not depend on who came last.
                // (The barrier orders the 128 threads' stores before thread 64's fence, and that fence is
                // cumulative: one fence at GPU scope publishes the whole block's share.)
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    __threadfence();
                    *last_flag = atomicAdd(&args.counters[tile], 1) == parts - 1;
                    __threadfence();
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = *last_flag != 0;
                if (threadIdx.x == 64) stamp(args, 10);
                if (last) {
                    const float* base = args.partial + (((long long)tile * args.max_parts) * ST_BM + row_in_tile) * ACC_COLS;
                    const long long part_stride = (long long)ST_BM * ACC_COLS;
                    for (int c0 = 0; c0 < BN && c0 < args.M; c0 += 8) {
                        float gs[8], us[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) gs[j] = us[j] = 0.f;
                        for (int p0 = 0; p0 < parts; p0 += 4) {     // four shares' loads in flight at a time
                            float4 tg[4][2], tu[4][2];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    const bool on = p0 + q < parts && c0 + 4 * h < args.M;
                                    const float* src = base + (p0 + q) * part_stride + c0 + 4 * h;
                                    tg[q][h] = on ? __ldcg(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                    if (GATE_UP)
                                        tu[q][h] = on ? __ldcg(reinterpret_cast<const float4*>(src + BN)) : make_float4(0.f, 0.f, 0.f, 0.f);
                                }
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    gs[4 * h] += tg[q][h].x; gs[4 * h + 1] += tg[q][h].y;
                                    gs[4 * h + 2] += tg[q][h].z; gs[4 * h + 3] += tg[q][h].w;
                                    if (GATE_UP) {
                                        us[4 * h] += tu[q][h].x; us[4 * h + 1] += tu[q][h].y;
                                        us[4 * h + 2] += tu[q][h].z; us[4 * h + 3] += tu[q][h].w;
                                    }
                                }
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int m = c0 + j;
                            if (m < args.M && n_row < args.n_out) {
                                const float v = GATE_UP ? silu_mul_rounded(gs[j], us[j]) : gs[j];
                                const long long o = (long long)m * args.n_out + n_row;
                                if (args.out_f32) ((float*)args.C)[o] = v;
                                else ((__nv_bfloat16*)args.C)[o] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                    if (threadIdx.x == 64) args.counters[tile] = 0;
                }
                if (threadIdx.x == 64) stamp(args, last ? 11 : 12);
                asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is read before the next item writes it
            }
            u += n_kb;
        }
    }
    if (threadIdx.x == 64) stamp(args, 6);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0) stamp(args, 7);
}

// ---- host side ----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A [rows, K] row-major bfloat16 matrix seen as boxes of box_rows x 64 columns, 128-byte swizzle,
// zero fill outside the matrix.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {ST_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN, bool GU, int STAGES>
static int launch_stream(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& ma, StreamArgs args, int grid,
                         cudaStream_t stream) {
    constexpr int N_A = GU ? 2 : 1;
    const int smem = 1024 + STAGES * (N_A * ST_BM * ST_BK * 2 + BN * ST_BK * 2) + (2 * STAGES + 4) * 8 + 32;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<BN, GU, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    sb_launch(gemm_stream_kernel<BN, GU, STAGES>, grid, ST_THREADS, smem, stream, mw, mw2, ma, args);
    return (int)cudaGetLastError();
}

extern "C" {

// Blocks the kernel will run on (one per SM at most) and the most blocks that can share one tile:
// what the caller needs to size the scratch: n_tiles * max_parts * acc_cols * 128 floats and n_tiles ints.
int sb_gemm_stream_plan(int n_out, int K, int n_sms, int* grid, int* n_tiles, int* max_parts) {
    const int tiles = (n_out + ST_BM - 1) / ST_BM, kb = (K + ST_BK - 1) / ST_BK;
    const long long U = (long long)tiles * kb;
    const int g = (int)(U < n_sms ? U : n_sms);
    *grid = g;
    *n_tiles = tiles;
    // a tile of kb units meets blocks that hold at least floor(U / g) units each
    const long long per = U / g;
    *max_parts = (int)((kb + per - 1) / per + 1);
    return 0;
}

// A [M, K], W [n_out, K] (or [2 * n_out, K], gate rows first, with gate_up), C [M, n_out] bfloat16 or float.
// M <= 64, K a multiple of 8.  grid, max_parts from sb_gemm_stream_plan.
#ifdef SB_TIMELINE
static long long* stream_timeline = nullptr;
void sb_gemm_stream_timeline(long long* buffer) { stream_timeline = buffer; }
#endif

int sb_gemm_stream(const void* A, const void* W, void* C, int M, int n_out, int K, int gate_up, int out_f32, int grid,
                   int max_parts, float* partial, int* counters, int* status, cudaStream_t stream) {
    if (M <= 0 || n_out <= 0) return 0;
    if (M > 64 || (K & 7) || (gate_up && M > 32) || grid < 1) return (int)cudaErrorInvalidValue;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, mw2, ma;
    int e = make_map(&mw, W, n_out, K, ST_BM);
    if (e) return e;
    e = make_map(&mw2, gate_up ? (const void*)((const __nv_bfloat16*)W + (long long)n_out * K) : W, n_out, K, ST_BM);
    if (e) return e;
    e = make_map(&ma, A, M, K, bn);
    if (e) return e;
    StreamArgs args;
    args.C = C; args.partial = partial; args.counters = counters; args.status = status;
    args.M = M; args.n_out = n_out; args.K = K;
    args.n_tiles = (n_out + ST_BM - 1) / ST_BM;
    args.k_blocks = (K + ST_BK - 1) / ST_BK;
    args.max_parts = max_parts;
    args.out_f32 = out_f32;
#ifdef SB_TIMELINE
    args.timeline = stream_timeline;
#endif
    if (gate_up) {
        if (bn == 16) return launch_stream<16, true, 6>(mw, mw2, ma, args, grid, stream);
        return launch_stream<32, true, 5>(mw, mw2, ma, args, grid, stream);
    }
    if (bn == 16) return launch_stream<16, false, 10>(mw, mw2, ma, args, grid, stream);
    if (bn == 32) return launch_stream<32, false, 9>(mw, mw2, ma, args, grid, stream);
    return launch_stream<64, false, 8>(mw, mw2, ma, args, grid, stream);
}

}  // extern "C"
