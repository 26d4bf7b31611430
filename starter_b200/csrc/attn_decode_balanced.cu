// Decode attention over the paged cache with the work divided evenly among the blocks.
//
// Same computation and numerics as attn_decode.cu (reference: engine/kernels/attention.py:24-114).
// What differs is who does what.  There, the grid is (sequence, kv head, split) and a block's share
// is fixed by shapes, so with 64 pairs of (sequence, kv head) on 148 SMs some SMs get three blocks and
// some two, and with 512 pairs a second wave runs nearly empty.  Here the unit of work is one cache
// page of one (sequence, kv head); the units of all sequences are laid end to end, the grid is as many
// blocks as the GPU holds at once, and every block takes the same number of consecutive units,
// computed on the device from the sequences' own lengths.  A block's share may cover the end of one
// pair and the start of the next; each piece is a segment.  A pair whose pages fall to several blocks
// is merged by the last of them to arrive, exactly as in attn_decode.cu.  The (pair, block)
// incidences are numbered pair + block, which is unique and dense, so the scratch for the partial
// results holds (pairs + blocks) entries whatever the lengths are.
#include "common.cuh"
#include "mma_utils.cuh"
#include "qk_prep.cuh"

#define AD_WARPS 4
#define AD_STAGES 4
#define AD_KEYS_PER_WARP (SB_PAGE / AD_WARPS)  // 16
#define ADB_MAX_SEQS 1024

// FUSED: q is null and the queries come from the projection's rows: per-head norm, rotary encoding and the store of
// the new key and value happen here (qk_prep.cuh), by the block whose share holds the pair's last page.
template <int D, bool FUSED>
__global__ void __launch_bounds__(AD_WARPS * 32, 1)
attn_decode_balanced_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, SbBatch batch, SbKV kv,
                            int n_heads, float scale_log2, int window, float* __restrict__ partial,
                            int* __restrict__ counters, SbFusedQK fused) {
    constexpr int CH = D / 8;                              // 16-byte chunks per row
    constexpr int SLICE = AD_KEYS_PER_WARP * D * 2;        // bytes of one warp's keys (or values) of a page
    constexpr int NT = D / 8;                              // output n-tiles of 8 columns
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_is_last;
    __shared__ int cum[ADB_MAX_SEQS + 1];                  // units before each sequence
    unsigned char* q_s = smem;                             // [16][D] bfloat16
    unsigned char* pipe = smem + 16 * D * 2;               // [warp][stage][K slice | V slice]

    // The shares are worked out from the lengths, which the kernel before this one does not write, so
    // this part may overlap it; everything after pdl_wait() may read what it wrote.
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = n_heads / kv.n_kv_heads, HKV = kv.n_kv_heads;
    const int B = batch.n_seqs;
    for (int i = tid; i < B; i += AD_WARPS * 32) {
        const int p = batch.lengths[batch.seq_slot[i]];
        const int first = window > 0 ? max(0, p - window + 1) / SB_PAGE : 0;
        cum[i + 1] = (p / SB_PAGE - first + 1) * HKV;
    }
    __syncthreads();
    if (tid == 0) {
        cum[0] = 0;
        for (int i = 0; i < B; ++i) cum[i + 1] += cum[i];
    }
    __syncthreads();
    pdl_wait();
    const int U = cum[B], P = gridDim.x;
    const int quota = (U + P - 1) / P;
    int u = blockIdx.x * quota;
    const int u_end = min(U, u + quota);
    const long long part_stride = D + 2;
    int seq = 0;

    while (u < u_end) {
        while (cum[seq + 1] <= u) ++seq;
        const int pages_seq = (cum[seq + 1] - cum[seq]) / HKV;
        const int kvh = (u - cum[seq]) / pages_seq, page_in_pair = (u - cum[seq]) % pages_seq;
        const int my_pages = min(pages_seq - page_in_pair, u_end - u);
        const int pair = seq * HKV + kvh;
        const int pair_begin = cum[seq] + kvh * pages_seq;
        const int first_block = pair_begin / quota, last_block = (pair_begin + pages_seq - 1) / quota;
        const int parts = last_block - first_block + 1;
        const int slot = batch.seq_slot[seq];
        const int row = batch.cu_q[seq];
        const int pos = batch.lengths[slot];                   // the new token's position; keys 0..pos are visible
        const int lo = window > 0 ? max(0, pos - window + 1) : 0;
        const int p_begin = lo / SB_PAGE + page_in_pair;
        __syncthreads();   // the segment before this one is done with the shared memory

        if (FUSED) {
            // the share that ends with the pair's last page holds the new position: it stores the new key and value
            const bool owns_new = fused.store_kv && page_in_pair + my_pages == pages_seq;
            prepare_group<D, AD_WARPS>(fused, kv, q_s, row, kvh, n_heads, G, pos, owns_new,
                                       owns_new ? kv_offset(kv, slot, pos, kvh) : -1);
        } else {
            // Query heads of this kv head as rows of a 16-row tile, zero beyond G.
            for (int i = tid; i < 16 * CH; i += AD_WARPS * 32) {
                const int r = i / CH, c = i % CH;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (r < G) v = *reinterpret_cast<const uint4*>(q + ((long long)row * n_heads + kvh * G + r) * D + c * 8);
                *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
            }
        }
        __syncthreads();   // the queries are in place; the new key and value are in the cache before their page is copied
        unsigned int qf[D / 16][4];
    #pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
            ldmatrix_x4(qf[ks], q_s + tile_off<D>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

        unsigned char* my_pipe = pipe + warp * (AD_STAGES * 2 * SLICE);
        const __nv_bfloat16* kbase = (const __nv_bfloat16*)kv.k;
        const __nv_bfloat16* vbase = (const __nv_bfloat16*)kv.v;
        const int* table = kv.table + (long long)slot * kv.table_width;

        // The ids of the block's pages, 32 at a time, one per lane: a lookup in the page table costs a trip to
        // L2, and paying it for every page would stall the copies behind it.
        int page_ids = 0;
        auto issue = [&](int i) {  // bring this warp's keys and values of the block's i-th page into stage i % STAGES
            if (i < my_pages) {
                if ((i & 31) == 0) {
                    int lp = p_begin + i + lane;
                    if (kv.ring_pages) lp %= kv.ring_pages;
                    // an unreserved page was flagged when the row was stored; lanes beyond the range read nothing
                    page_ids = i + lane < my_pages ? max(table[lp], 0) : 0;
                }
                const int page = __shfl_sync(0xffffffffu, page_ids, i & 31);
                const long long base = (((long long)page * kv.n_kv_heads + kvh) * SB_PAGE + warp * AD_KEYS_PER_WARP) * D;
                unsigned char* ks = my_pipe + (i % AD_STAGES) * 2 * SLICE;
                unsigned char* vs = ks + SLICE;
    #pragma unroll
                for (int j = lane; j < AD_KEYS_PER_WARP * CH; j += 32) {
                    const int r = j / CH, c = j % CH;
                    cp_async_16(ks + tile_off<D>(r, c), kbase + base + r * D + c * 8);
                    cp_async_16(vs + tile_off<D>(r, c), vbase + base + r * D + c * 8);
                }
            }
            cp_async_commit();
        };

        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float acc[NT][4];
    #pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    #pragma unroll
        for (int i = 0; i < AD_STAGES - 1; ++i) issue(i);
        for (int i = 0; i < my_pages; ++i) {
            issue(i + AD_STAGES - 1);
            cp_async_wait<AD_STAGES - 1>();
            __syncwarp();
            const unsigned char* ks = my_pipe + (i % AD_STAGES) * 2 * SLICE;
            const unsigned char* vs = ks + SLICE;
            // Values of keys that no row of this step may see (beyond the new token, before the window) are stale: they
            // meet a probability of exactly zero, but zero times an infinity or a NaN left by the page's former owner
            // would not be zero.  Such rows exist only in a sequence's last (and, with a window, first) page.
            {
                const int n_base = (p_begin + i) * SB_PAGE + warp * AD_KEYS_PER_WARP;
                if (n_base + AD_KEYS_PER_WARP - 1 > pos || n_base < lo) {
                    for (int j = lane; j < AD_KEYS_PER_WARP * CH; j += 32) {
                        const int r = j / CH, n = n_base + r;
                        if (n > pos || n < lo)
                            *reinterpret_cast<uint4*>(const_cast<unsigned char*>(vs) + tile_off<D>(r, j % CH)) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                }
            }

            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    #pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                unsigned int b[4];
                ldmatrix_x4(b, ks + tile_off<D>((lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
                mma_bf16(s0, qf[kk], b[0], b[1]);
                mma_bf16(s1, qf[kk], b[2], b[3]);
            }
            // keys of this thread's columns: n0 + {0,1} in tile 0, n0 + 8 + {0,1} in tile 1
            const int n0 = (p_begin + i) * SB_PAGE + warp * AD_KEYS_PER_WARP + (lane & 3) * 2;
            const bool v00 = n0 >= lo && n0 <= pos, v01 = n0 + 1 >= lo && n0 + 1 <= pos;
            const bool v10 = n0 + 8 >= lo && n0 + 8 <= pos, v11 = n0 + 9 >= lo && n0 + 9 <= pos;
            float t[2][4];
            t[0][0] = v00 ? s0[0] * scale_log2 : -INFINITY;
            t[0][1] = v01 ? s0[1] * scale_log2 : -INFINITY;
            t[0][2] = v10 ? s1[0] * scale_log2 : -INFINITY;
            t[0][3] = v11 ? s1[1] * scale_log2 : -INFINITY;
            t[1][0] = v00 ? s0[2] * scale_log2 : -INFINITY;
            t[1][1] = v01 ? s0[3] * scale_log2 : -INFINITY;
            t[1][2] = v10 ? s1[2] * scale_log2 : -INFINITY;
            t[1][3] = v11 ? s1[3] * scale_log2 : -INFINITY;
            float alpha[2];
    #pragma unroll
            for (int h = 0; h < 2; ++h) {
                float mx = fmaxf(fmaxf(t[h][0], t[h][1]), fmaxf(t[h][2], t[h][3]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[h], mx);
                const float m_safe = m_new == -INFINITY ? 0.f : m_new;
                alpha[h] = exp2f(m[h] - m_safe);
                float sum = 0.f;
    #pragma unroll
                for (int e = 0; e < 4; ++e) {
                    t[h][e] = fast_exp2(t[h][e] - m_safe);
                    sum += t[h][e];
                }
                l[h] = l[h] * alpha[h] + sum;
                m[h] = m_new;
            }
            unsigned int pf[4];
            pf[0] = pack_bf16(t[0][0], t[0][1]);
            pf[1] = pack_bf16(t[1][0], t[1][1]);
            pf[2] = pack_bf16(t[0][2], t[0][3]);
            pf[3] = pack_bf16(t[1][2], t[1][3]);
    #pragma unroll
            for (int j = 0; j < NT; j += 2) {
                unsigned int b[4];
                ldmatrix_x4_trans(b, vs + tile_off<D>((lane & 7) + ((lane >> 3) & 1) * 8, j + (lane >> 4)));
                acc[j][0] *= alpha[0]; acc[j][1] *= alpha[0]; acc[j][2] *= alpha[1]; acc[j][3] *= alpha[1];
                acc[j + 1][0] *= alpha[0]; acc[j + 1][1] *= alpha[0]; acc[j + 1][2] *= alpha[1]; acc[j + 1][3] *= alpha[1];
                mma_bf16(acc[j], pf, b[0], b[1]);
                mma_bf16(acc[j + 1], pf, b[2], b[3]);
            }
            __syncwarp();
        }
        cp_async_wait<0>();
    #pragma unroll
        for (int h = 0; h < 2; ++h) {
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        }
        __syncthreads();  // every warp is done with the pipeline's memory; it now holds the warps' states

        // Warp states to shared memory: acc [warp][16][D] floats, then m and l [warp][16].
        float* w_acc = reinterpret_cast<float*>(pipe);
        float* w_m = w_acc + AD_WARPS * 16 * D;
        float* w_l = w_m + AD_WARPS * 16;
        {
            const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    #pragma unroll
            for (int j = 0; j < NT; ++j) {
                float* dst = w_acc + (warp * 16 + r0) * D + j * 8 + c0;
                dst[0] = acc[j][0]; dst[1] = acc[j][1];
                dst[8 * D] = acc[j][2]; dst[8 * D + 1] = acc[j][3];
            }
            if ((lane & 3) == 0) {
                w_m[warp * 16 + r0] = m[0]; w_m[warp * 16 + r0 + 8] = m[1];
                w_l[warp * 16 + r0] = l[0]; w_l[warp * 16 + r0 + 8] = l[1];
            }
        }
        __syncthreads();


        // The block's result for this segment: heads of the group, relative to their own maximum.
        float* my_part = partial + (long long)(pair + blockIdx.x) * G * part_stride;
        for (int i = tid; i < G * D; i += AD_WARPS * 32) {
            const int r = i / D, d = i % D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, w_m[w * 16 + r]);
            float o = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) {
                const float mw = w_m[w * 16 + r];
                const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - M);
                o += w_acc[(w * 16 + r) * D + d] * wgt;
                L += w_l[w * 16 + r] * wgt;
            }
            const int head = kvh * G + r;
            if (parts == 1) {
                out[((long long)row * n_heads + head) * D + d] = __float2bfloat16_rn(o / L);
            } else {
                float* p = my_part + r * part_stride;
                p[d] = o;
                if (d == 0) { p[D] = M; p[D + 1] = L; }
            }
        }
        if (parts > 1) {
            // The last block of this pair to get here merges the parts.
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                s_is_last = atomicAdd(&counters[pair], 1) == parts - 1;
                __threadfence();
            }
            __syncthreads();
            if (s_is_last) {
                float* s_w = reinterpret_cast<float*>(pipe);            // [G][parts] exp2(m_p - M), then
                float* s_l = s_w + G * parts;                           // [G][parts] l_p
                const float* base = partial + (long long)(pair + first_block) * G * part_stride;
                for (int i = tid; i < G * parts; i += AD_WARPS * 32) {
                    const int r = i / parts, p = i % parts;
                    const float* src = base + ((long long)p * G + r) * part_stride;
                    s_w[i] = __ldcg(src + D);
                    s_l[i] = __ldcg(src + D + 1);
                }
                __syncthreads();
                for (int r = warp; r < G; r += AD_WARPS) {
                    float M = -INFINITY;
                    for (int p = lane; p < parts; p += 32) M = fmaxf(M, s_w[r * parts + p]);
                    M = warp_max(M);
                    for (int p = lane; p < parts; p += 32) {
                        const float mp = s_w[r * parts + p];
                        s_w[r * parts + p] = mp == -INFINITY ? 0.f : exp2f(mp - M);
                    }
                }
                __syncthreads();
                for (int i = tid; i < G * D; i += AD_WARPS * 32) {
                    const int r = i / D, d = i % D;
                    const float* src = base + (long long)r * part_stride + d;
                    const float* w = s_w + r * parts;
                    const long long step = (long long)G * part_stride;
                    float o = 0.f, L = 0.f;
                    int p = 0;
                    for (; p + 8 <= parts; p += 8) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __ldcg(src + (p + e) * step);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            o += v[e] * w[p + e];
                            L += s_l[r * parts + p + e] * w[p + e];
                        }
                    }
                    for (; p < parts; ++p) {
                        o += __ldcg(src + p * step) * w[p];
                        L += s_l[r * parts + p] * w[p];
                    }
                    out[((long long)row * n_heads + kvh * G + r) * D + d] = __float2bfloat16_rn(o / L);
                }
                if (tid == 0) counters[pair] = 0;  // ready for the next launch
            }
        }
        u += my_pages;
    }
}

template <int D, bool FUSED>
static int launch_balanced(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window, int grid,
                           float* partial, int* counters, SbFusedQK fused, cudaStream_t stream) {
    const int pipe_bytes = AD_WARPS * AD_STAGES * 2 * AD_KEYS_PER_WARP * D * 2;
    const int merge_bytes = (AD_WARPS * 16 * D + 2 * AD_WARPS * 16) * 4;
    // More than half an SM's shared memory is asked for, so that no SM ever holds two of these blocks: the
    // shares are equal only if every block has an SM to itself, also when the grid starts while the kernel
    // before it still holds some SMs.
    const int need = 16 * D * 2 + (pipe_bytes > merge_bytes ? pipe_bytes : merge_bytes);
    const int smem = need > 116 * 1024 ? need : 116 * 1024;
    static bool configured[64] = {};   // the attribute belongs to the kernel as loaded on one device
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_balanced_kernel<D, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    sb_launch(attn_decode_balanced_kernel<D, FUSED>, grid, AD_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
              batch, kv, n_heads, scale * 1.4426950408889634f, window, partial, counters, fused);
    return (int)cudaGetLastError();
}

static bool balanced_shape_ok(const SbBatch& batch, const SbKV& kv, int n_heads, int grid) {
    return kv.n_kv_heads > 0 && n_heads > 0 && batch.n_rows == batch.n_seqs && n_heads % kv.n_kv_heads == 0 &&
           n_heads / kv.n_kv_heads <= 16 && grid >= 1 && grid <= 512 && batch.n_seqs <= ADB_MAX_SEQS &&
           (kv.head_dim == 64 || kv.head_dim == 128);
}

extern "C" {

// One new token per sequence (rows == sequences).  q, out [rows, n_heads * head_dim] bfloat16.
// Takes head_dim 64 or 128, up to 16 query heads per kv head, up to 1024 sequences and up to 512 blocks.
// partial: (n_seqs * n_kv_heads + grid) * (n_heads / n_kv_heads) * (head_dim + 2) floats of scratch;
// counters: n_seqs * n_kv_heads ints, zero before the first launch (the kernel leaves them zero).
int sb_attn_decode_balanced(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                            int grid, float* partial, int* counters, cudaStream_t stream) {
    if (batch.n_seqs <= 0) return 0;
    if (!balanced_shape_ok(batch, kv, n_heads, grid)) return (int)cudaErrorInvalidValue;
    SbFusedQK none = {};
    if (kv.head_dim == 128) return launch_balanced<128, false>(q, out, batch, kv, n_heads, scale, window, grid, partial, counters, none, stream);
    return launch_balanced<64, false>(q, out, batch, kv, n_heads, scale, window, grid, partial, counters, none, stream);
}

// The same with the preparation of q and k inside: qkv is the row of the fused projection; the new key and value
// are stored in the cache by this call.
int sb_attn_decode_balanced_fused(SbFusedQK fused, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                                  int grid, float* partial, int* counters, cudaStream_t stream) {
    if (batch.n_seqs <= 0) return 0;
    if (!balanced_shape_ok(batch, kv, n_heads, grid) || fused.qkv == nullptr || fused.status == nullptr ||
        ((fused.cos_t == nullptr) != (fused.sin_t == nullptr)))
        return (int)cudaErrorInvalidValue;
    if (kv.head_dim == 128) return launch_balanced<128, true>(nullptr, out, batch, kv, n_heads, scale, window, grid, partial, counters, fused, stream);
    return launch_balanced<64, true>(nullptr, out, batch, kv, n_heads, scale, window, grid, partial, counters, fused, stream);
}

}  // extern "C"
