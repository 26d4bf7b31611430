// Decode attention over the paged cache: one new token per sequence, grouped query heads,
// keys split across thread blocks, partial results merged at the end.
//
// Reference: engine/kernels/attention.py:24-114 (split-K flash decoding: all G = heads /
// kv_heads query heads of a key/value head share one program so that keys and values are
// read once per group; scores, maximum, exp and sum in 32-bit; probabilities rounded to
// bfloat16 before they meet V; one division at the end; partial (m, l, acc) triples merged).
//
// Layout of the work.  Grid (sequence, kv head, split).  A block has four warps; warp w owns
// the keys 16w..16w+15 of every cache page (64 keys) in the block's range of pages, brings them
// in with its own cp.async pipeline, and keeps its own running (m, l, acc): softmax states
// merge exactly, so the warps never wait for one another until the end.  The tensor cores
// (mma.sync m16n8k16, bfloat16 in, 32-bit accumulate) see the G query heads as the rows of a
// 16-row tile.  The split count depends on shapes only; the pages are divided among the
// splits on the device from the sequence's own length, so a graph replay stays valid as the
// sequence grows.
//
// Merging the splits.  With 2 to 8 splits the blocks of one (sequence, kv head) form a thread-block
// cluster: each leaves its result in its own shared memory, the cluster meets, and every block
// finishes a share of the output from the others' shared memory (no trip through global memory, no
// atomic).  With more splits each block leaves its partial result in scratch memory and the last one
// to arrive (an atomic counter per sequence and kv head) merges them.
//
// Fused preparation of q and k (FUSED).  The kernel can take the row of the fused q/k/v projection
// instead of finished queries: it then applies the per-head RMSNorm and the rotary encoding to its own
// G query heads (engine/kernels/rope.py:95-144), and the block whose pages hold the new token's
// position does the same for the key head, stores key and value in the cache and reads them back with
// its other keys.  That saves the separate kernel between the projection and the attention.
#include <cooperative_groups.h>

#include "common.cuh"
#include "mma_utils.cuh"
#include "qk_prep.cuh"

namespace cg = cooperative_groups;

#define AD_WARPS 4
#define AD_KEYS_PER_WARP (SB_PAGE / AD_WARPS)  // 16
#define AD_MAX_CLUSTER 8
#define AD_MAX_DEVICES 64     // devices whose per-device set-up this file remembers

template <int D, bool FUSED, int AD_STAGES>
__global__ void __launch_bounds__(AD_WARPS * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, SbBatch batch, SbKV kv,
                   int n_heads, float scale_log2, int window, int n_splits, int cluster_merge, float* __restrict__ partial,
                   int* __restrict__ counters, SbFusedQK fused) {
    constexpr int CH = D / 8;                              // 16-byte chunks per row
    constexpr int SLICE = AD_KEYS_PER_WARP * D * 2;        // bytes of one warp's keys (or values) of a page
    constexpr int NT = D / 8;                              // output n-tiles of 8 columns
    constexpr int LANES = D / 4;                           // lanes that hold a head, four values each
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_is_last;
    unsigned char* q_s = smem;                             // [16][D] bfloat16
    unsigned char* pipe = smem + 16 * D * 2;               // [warp][stage][K slice | V slice]

    // Until pdl_wait() only what the kernel before this one does not write is touched: the batch's description,
    // the lengths, the page table, the norm weights and rotary tables, and pages before the one that holds
    // the new token.  If that kernel releases this one early, the look-ups and first copies below overlap it.
    sb_stamp(4, 0);
    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = n_heads / kv.n_kv_heads;
    const int slot = batch.seq_slot[seq];
    const int row = batch.cu_q[seq];
    const int pos = batch.lengths[slot];                   // the new token's position; keys 0..pos are visible
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_page = lo / SB_PAGE, last_page = pos / SB_PAGE;
    const int n_pages = last_page - first_page + 1;
    const int per_split = (n_pages + n_splits - 1) / n_splits;
    const int p_begin = first_page + split * per_split;
    const int p_end = min(p_begin + per_split, last_page + 1);
    const int my_pages = max(p_end - p_begin, 0);

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

    // Constants of the fused preparation: this lane's four rotary factors and norm weights, and where the
    // new key and value go (only the block whose pages hold the new position stores them).
    const int d0 = lane * 4;
    const bool holds = lane < LANES;
    float rc[4] = {1.f, 1.f, 1.f, 1.f}, rs[4] = {0.f, 0.f, 0.f, 0.f}, wq[4] = {1.f, 1.f, 1.f, 1.f};
    bool owns_new = false;
    long long new_off = -1;
    if (FUSED) {
        if (holds) {
            if (fused.cos_t != nullptr) {
                const int j0 = d0 % (D / 2);
                unpack4(*reinterpret_cast<const uint2*>(fused.cos_t + (long long)pos * (D / 2) + j0), rc);
                unpack4(*reinterpret_cast<const uint2*>(fused.sin_t + (long long)pos * (D / 2) + j0), rs);
            }
            if (fused.q_norm != nullptr) load_norm4(fused.q_norm, fused.norm_f32, d0, wq);
        }
        owns_new = fused.store_kv && p_begin <= last_page && last_page < p_end;
        if (owns_new) new_off = kv_offset(kv, slot, pos, kvh);
    }

    int ahead = 0;
    while (ahead < AD_STAGES - 1 && p_begin + ahead < last_page) issue(ahead++);
    sb_stamp(4, 1);
    pdl_wait();
    sb_stamp(4, 2);

    if (FUSED) {
        // Rows of the query tile beyond the group are zero.
        for (int i = tid; i < 16 * CH; i += AD_WARPS * 32) {
            const int r = i / CH, c = i % CH;
            if (r >= G) *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = make_uint4(0u, 0u, 0u, 0u);
        }
        const int width = (n_heads + (fused.store_kv ? 2 * kv.n_kv_heads : 0)) * D;
        const __nv_bfloat16* qkv_row = fused.qkv + (long long)row * width;
        const int n_jobs = G + (owns_new ? 1 : 0);          // job G: the key head (and the value's copy)
        for (int job = warp; job < n_jobs; job += AD_WARPS) {
            const bool is_q = job < G;
            const __nv_bfloat16* src = qkv_row + (long long)(is_q ? kvh * G + job : n_heads + kvh) * D;
            float y[4] = {0.f, 0.f, 0.f, 0.f};
            if (holds) unpack4(*reinterpret_cast<const uint2*>(src + d0), y);
            const void* wn = is_q ? fused.q_norm : fused.k_norm;
            if (wn != nullptr) {
                float w4[4] = {wq[0], wq[1], wq[2], wq[3]};
                if (!is_q && holds) load_norm4(wn, fused.norm_f32, d0, w4);
                float ss = y[0] * y[0];
                ss = fmaf(y[1], y[1], ss); ss = fmaf(y[2], y[2], ss); ss = fmaf(y[3], y[3], ss);
                ss = warp_sum(ss);
                const float rstd = 1.0f / sqrtf(ss / (float)D + fused.eps);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float n = rnd<__nv_bfloat16>(__fmul_rn(y[e], rstd));
                    y[e] = rnd<__nv_bfloat16>(__fmul_rn(w4[e], n));
                }
            }
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[e] = y[e];
                if (fused.cos_t != nullptr) {   // rotate-half: the partner of d is d +- D/2, held by lane ^ (LANES / 2)
                    const float partner = __shfl_xor_sync(0xffffffffu, y[e], LANES / 2);
                    const float a = rnd<__nv_bfloat16>(__fmul_rn(y[e], rc[e]));
                    const float b = rnd<__nv_bfloat16>(__fmul_rn(lane < LANES / 2 ? -partner : partner, rs[e]));
                    o[e] = __fadd_rn(a, b);
                }
            }
            uint2 res;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
            r2[0] = __floats2bfloat162_rn(o[0], o[1]);
            r2[1] = __floats2bfloat162_rn(o[2], o[3]);
            if (is_q) {
                if (holds) *reinterpret_cast<uint2*>(q_s + tile_off<D>(job, lane >> 1) + (lane & 1) * 8) = res;
            } else if (new_off < 0) {
                if (lane == 0) atomicOr(fused.status, SB_STATUS_NO_PAGE);
            } else if (holds) {
                *reinterpret_cast<uint2*>((__nv_bfloat16*)kv.k + new_off + d0) = res;
                *reinterpret_cast<uint2*>((__nv_bfloat16*)kv.v + new_off + d0) =
                    *reinterpret_cast<const uint2*>(src + (long long)kv.n_kv_heads * D + d0);
            }
        }
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
    for (; ahead < AD_STAGES - 1; ++ahead) issue(ahead);   // the page of the new token, after the wait
    unsigned int qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(qf[ks], q_s + tile_off<D>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

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
    if (FUSED && tid == 0)
        l2_prefetch_share(fused.next_w, fused.next_bytes, ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                          (long long)gridDim.x * gridDim.y * gridDim.z);
    sb_stamp(4, 3);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    __syncthreads();  // every warp is done with the pipeline's memory; it now holds the warps' states

    // Warp states to shared memory: acc [warp][16][D] floats, then m and l [warp][16]; behind them the
    // block's own result for the cluster: o [G][D], m [16], l [16].
    float* w_acc = reinterpret_cast<float*>(pipe);
    float* w_m = w_acc + AD_WARPS * 16 * D;
    float* w_l = w_m + AD_WARPS * 16;
    float* blk_o = w_l + AD_WARPS * 16;
    float* blk_m = blk_o + 16 * D;
    float* blk_l = blk_m + 16;
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

    const long long part_stride = D + 2;
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
        if (n_splits == 1) {
            out[((long long)row * n_heads + head) * D + d] = __float2bfloat16_rn(o / L);
        } else if (cluster_merge) {
            blk_o[i] = o;
            if (d == 0) { blk_m[r] = M; blk_l[r] = L; }
        } else {
            float* p = partial + (((long long)seq * n_heads + head) * n_splits + split) * part_stride;
            p[d] = o;
            if (d == 0) { p[D] = M; p[D + 1] = L; }
        }
    }
    if (n_splits == 1) return;

    if (cluster_merge) {
        // The blocks of this (sequence, kv head) are one cluster, this block's rank in it is its split.  Each
        // finishes an equal share of the G * D outputs from all the blocks' shared memory.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        sb_stamp(4, 4);
        const int share = (G * D + n_splits - 1) / n_splits;
        const int i_end = min(G * D, (split + 1) * share);
        for (int i = split * share + tid; i < i_end; i += AD_WARPS * 32) {
            const int r = i / D, d = i % D;
            float ms[AD_MAX_CLUSTER];
            float M = -INFINITY;
#pragma unroll
            for (int c = 0; c < AD_MAX_CLUSTER; ++c)
                if (c < n_splits) {
                    ms[c] = *cluster.map_shared_rank(blk_m + r, c);
                    M = fmaxf(M, ms[c]);
                }
            float o = 0.f, L = 0.f;
#pragma unroll
            for (int c = 0; c < AD_MAX_CLUSTER; ++c)
                if (c < n_splits) {
                    const float wgt = ms[c] == -INFINITY ? 0.f : exp2f(ms[c] - M);
                    o += *cluster.map_shared_rank(blk_o + i, c) * wgt;
                    L += *cluster.map_shared_rank(blk_l + r, c) * wgt;
                }
            out[((long long)row * n_heads + kvh * G + r) * D + d] = __float2bfloat16_rn(o / L);
        }
        cluster.sync();   // nobody leaves while its shared memory is still being read
        sb_stamp(4, 5);
        return;
    }

    // The last block of this (sequence, kv head) to get here merges the splits.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&counters[seq * kv.n_kv_heads + kvh], 1);
        s_is_last = prev == n_splits - 1;
    }
    __syncthreads();
    sb_stamp(4, 4);
    if (!s_is_last) return;
    __threadfence();
    // Weights of the splits first (each thread fetches other entries, so the loads overlap), then
    // the weighted sums with the loads of several splits in flight at once.
    float* s_w = reinterpret_cast<float*>(pipe);            // [G][n_splits] exp2(m_s - M), then
    float* s_l = s_w + G * n_splits;                        // [G][n_splits] l_s
    const float* base = partial + (long long)seq * n_heads * n_splits * part_stride;
    for (int i = tid; i < G * n_splits; i += AD_WARPS * 32) {
        const int r = i / n_splits, s = i % n_splits;
        const float* p = base + ((long long)(kvh * G + r) * n_splits + s) * part_stride;
        s_w[i] = __ldcg(p + D);
        s_l[i] = __ldcg(p + D + 1);
    }
    __syncthreads();
    for (int r = warp; r < G; r += AD_WARPS) {
        float M = -INFINITY;
        for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, s_w[r * n_splits + s]);
        M = warp_max(M);
        for (int s = lane; s < n_splits; s += 32) {
            const float ms = s_w[r * n_splits + s];
            s_w[r * n_splits + s] = ms == -INFINITY ? 0.f : exp2f(ms - M);
        }
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += AD_WARPS * 32) {
        const int r = i / D, d = i % D;
        const int head = kvh * G + r;
        const float* p = base + (long long)head * n_splits * part_stride + d;
        const float* w = s_w + r * n_splits;
        float o = 0.f, L = 0.f;
        int s = 0;
        for (; s + 8 <= n_splits; s += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __ldcg(p + (s + e) * part_stride);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                o += v[e] * w[s + e];
                L += s_l[r * n_splits + s + e] * w[s + e];
            }
        }
        for (; s < n_splits; ++s) {
            o += __ldcg(p + s * part_stride) * w[s];
            L += s_l[r * n_splits + s] * w[s];
        }
        out[((long long)row * n_heads + head) * D + d] = __float2bfloat16_rn(o / L);
    }
    if (tid == 0) counters[seq * kv.n_kv_heads + kvh] = 0;  // ready for the next launch
    sb_stamp(4, 5);
}

template <int D, bool FUSED, int AD_STAGES>
static int launch_decode_staged(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window, int n_splits,
                         float* partial, int* counters, SbFusedQK fused, cudaStream_t stream) {
    const int pipe_bytes = AD_WARPS * AD_STAGES * 2 * AD_KEYS_PER_WARP * D * 2;
    const int merge_bytes = (AD_WARPS * 16 * D + 2 * AD_WARPS * 16 + 16 * D + 32) * 4;
    const int smem = 16 * D * 2 + (pipe_bytes > merge_bytes ? pipe_bytes : merge_bytes);
    // the attribute belongs to the kernel as loaded on one device: once per device
    static bool configured[AD_MAX_DEVICES] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= AD_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (!configured[device]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, FUSED, AD_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    const int cluster_merge = n_splits >= 2 && n_splits <= AD_MAX_CLUSTER;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(batch.n_seqs, kv.n_kv_heads, n_splits);
    config.blockDim = dim3(AD_WARPS * 32);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (sb_pdl_flag) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (cluster_merge) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = n_splits;
        ++n_attr;
    }
    config.attrs = attr;
    config.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&config, attn_decode_kernel<D, FUSED, AD_STAGES>, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, batch,
                                       kv, n_heads, scale * 1.4426950408889634f, window, n_splits, cluster_merge, partial,
                                       counters, fused);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Pipeline depth per warp: two pages ahead of the one being worked on; three when every block has an SM to
// itself (measured at a context of 4,096: 3.08 against 3.09 ms per step at batch 8 for two against one
// ahead, 396 against 387 tokens a second at batch 1 for three against two; three ahead with blocks that
// share SMs no longer fit two to an SM and lose 10%).
template <int D, bool FUSED>
static int launch_decode(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window, int n_splits,
                         float* partial, int* counters, SbFusedQK fused, cudaStream_t stream) {
    static int sm_counts[AD_MAX_DEVICES] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= AD_MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (sm_counts[device] == 0 &&
        cudaDeviceGetAttribute(&sm_counts[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        sm_counts[device] = 1;
    const int sm_count = sm_counts[device];
    const long long blocks = (long long)batch.n_seqs * kv.n_kv_heads * n_splits;
    if (blocks <= sm_count)
        return launch_decode_staged<D, FUSED, 4>(q, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, fused, stream);
    return launch_decode_staged<D, FUSED, 3>(q, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, fused, stream);
}

// Most splits whose merge fits: the last block of a (sequence, kv head) keeps two floats per (query head of the
// group, split) in the shared memory of its page pipeline (the smallest pipeline: three stages).
static int decode_max_splits(int group, int head_dim) {
    const int pipe_bytes = AD_WARPS * 3 * 2 * AD_KEYS_PER_WARP * head_dim * 2;
    const int merge_bytes = (AD_WARPS * 16 * head_dim + 2 * AD_WARPS * 16 + 16 * head_dim + 32) * 4;
    const int most = (pipe_bytes > merge_bytes ? pipe_bytes : merge_bytes) / (2 * (int)sizeof(float) * (group > 0 ? group : 1));
    return most < 65535 ? most : 65535;
}

static bool decode_shape_ok(const SbBatch& batch, const SbKV& kv, int n_heads, int n_splits) {
    if (kv.n_kv_heads <= 0 || n_heads <= 0 || kv.n_kv_heads > 65535 || (kv.head_dim != 64 && kv.head_dim != 128)) return false;
    if (batch.n_rows != batch.n_seqs || n_heads % kv.n_kv_heads != 0 || n_heads / kv.n_kv_heads > 16) return false;
    return n_splits >= 1 && (n_splits <= AD_MAX_CLUSTER || n_splits <= decode_max_splits(n_heads / kv.n_kv_heads, kv.head_dim));
}

extern "C" {

// Floats of scratch the kernel needs for a batch: partial results [seq][head][split][D + 2]
// (none with up to 8 splits, which merge through shared memory).
long long sb_attn_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
    return n_splits > AD_MAX_CLUSTER ? (long long)n_seqs * n_heads * n_splits * (head_dim + 2) : 0;
}

// Most splits a call may ask for (more would not fit the merge's shared memory and is refused).
int sb_attn_decode_max_splits(int n_heads, int n_kv_heads, int head_dim) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    return decode_max_splits(n_heads / n_kv_heads, head_dim);
}

// One new token per sequence (rows == sequences).  q, out [rows, n_heads * head_dim] bfloat16.
// Takes head_dim 64 or 128 and up to 16 query heads per kv head; anything else is refused.
// partial: scratch of sb_attn_decode_scratch_floats floats; counters: n_seqs * n_kv_heads ints,
// zero before the first launch (the kernel leaves them zero).
int sb_attn_decode(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window, int n_splits,
                   float* partial, int* counters, cudaStream_t stream) {
    if (batch.n_seqs <= 0) return 0;
    if (!decode_shape_ok(batch, kv, n_heads, n_splits)) return (int)cudaErrorInvalidValue;
    SbFusedQK none = {};
    if (kv.head_dim == 128) return launch_decode<128, false>(q, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, none, stream);
    return launch_decode<64, false>(q, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, none, stream);
}

// The same with the preparation of q and k inside (see the top of this file): qkv is the row of the fused
// projection; the new key and value are stored in the cache by this call.
int sb_attn_decode_fused(SbFusedQK fused, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window, int n_splits,
                         float* partial, int* counters, cudaStream_t stream) {
    if (batch.n_seqs <= 0) return 0;
    if (!decode_shape_ok(batch, kv, n_heads, n_splits) || fused.qkv == nullptr || fused.status == nullptr ||
        ((fused.cos_t == nullptr) != (fused.sin_t == nullptr)))
        return (int)cudaErrorInvalidValue;
    if (kv.head_dim == 128) return launch_decode<128, true>(nullptr, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, fused, stream);
    return launch_decode<64, true>(nullptr, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, fused, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// The same kernel for callers that cannot allocate: scratch in a fixed device array.
// Declaration, limits and rules of use: attn_decode_noalloc.h.
#include <stdio.h>

#include "attn_decode_noalloc.h"

// Counters first (ints), then the partial results (floats).  In host code this name is only a
// handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char sb_noalloc_scratch[SB_NOALLOC_MAX_COUNTERS * sizeof(int) +
                                                                  (size_t)SB_NOALLOC_MAX_FLOATS * sizeof(float)];

#define SB_NOALLOC_MAX_DEVICES 64
static void* sb_noalloc_device_ptr[SB_NOALLOC_MAX_DEVICES];
static thread_local char sb_noalloc_message[256];

extern "C" {

const char* sb_attn_decode_noalloc_error(void) { return sb_noalloc_message; }

void* sb_attn_decode_noalloc_scratch(void) {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= SB_NOALLOC_MAX_DEVICES) return nullptr;
    return sb_noalloc_device_ptr[device];
}

int sb_attn_decode_noalloc(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                           int n_splits, cudaStream_t stream) {
    sb_noalloc_message[0] = 0;
    if (batch.n_seqs <= 0) return 0;
    if (kv.n_kv_heads <= 0 || n_heads <= 0 || n_splits < 1) return (int)cudaErrorInvalidValue;
    if (n_splits > AD_MAX_CLUSTER && n_splits > sb_attn_decode_max_splits(n_heads, kv.n_kv_heads, kv.head_dim)) {
        snprintf(sb_noalloc_message, sizeof(sb_noalloc_message),
                 "sb_attn_decode_noalloc: %d splits are more than the %d whose merge fits a block's shared memory "
                 "at %d query heads per kv head", n_splits, sb_attn_decode_max_splits(n_heads, kv.n_kv_heads, kv.head_dim),
                 n_heads / kv.n_kv_heads);
        return SB_NOALLOC_TOO_LARGE;
    }
    const long long counters_needed = (long long)batch.n_seqs * kv.n_kv_heads;
    const long long floats_needed = sb_attn_decode_scratch_floats(batch.n_seqs, n_heads, kv.head_dim, n_splits);
    if (counters_needed > SB_NOALLOC_MAX_COUNTERS || floats_needed > SB_NOALLOC_MAX_FLOATS) {
        snprintf(sb_noalloc_message, sizeof(sb_noalloc_message),
                 "sb_attn_decode_noalloc: the call needs %lld counters and %lld floats of scratch; the fixed array "
                 "holds %d and %d (use sb_attn_decode with scratch of your own, or fewer splits)",
                 counters_needed, floats_needed, SB_NOALLOC_MAX_COUNTERS, SB_NOALLOC_MAX_FLOATS);
        return SB_NOALLOC_TOO_LARGE;
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= SB_NOALLOC_MAX_DEVICES) {
        snprintf(sb_noalloc_message, sizeof(sb_noalloc_message), "sb_attn_decode_noalloc: device %d is beyond the %d this "
                 "entry point keeps addresses for", device, SB_NOALLOC_MAX_DEVICES);
        return SB_NOALLOC_SETUP_FAILED;
    }
    if (sb_noalloc_device_ptr[device] == nullptr) {
        // Set-up, once per device, with that device current: the array's address on this device.
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, sb_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            snprintf(sb_noalloc_message, sizeof(sb_noalloc_message), "sb_attn_decode_noalloc: cudaGetSymbolAddress failed: %s",
                     cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : SB_NOALLOC_SETUP_FAILED;
        }
        sb_noalloc_device_ptr[device] = p;
    }
    int* counters = reinterpret_cast<int*>(sb_noalloc_device_ptr[device]);
    float* partial = reinterpret_cast<float*>(counters + SB_NOALLOC_MAX_COUNTERS);
    // The array keeps the last call's contents: the counters must start at zero.
    e = cudaMemsetAsync(counters, 0, counters_needed * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return sb_attn_decode(q, out, batch, kv, n_heads, scale, window, n_splits, partial, counters, stream);
}

}  // extern "C"

SB_TIMELINE_SETTER(attn_decode)
