// Prefill attention: many new rows per sequence over the paged cache, causal with an optional
// window, grouped query heads, ragged batch.  Flash attention on the warp-level tensor cores.
//
// Reference: the reference calls a library for this step (scaled_dot_product_attention, causal,
// enable_gqa: engine/model.py:268-274) and states its numerics in engine/kernels/attention.py:9-11:
// scores and softmax statistics in 32-bit, probabilities rounded to bfloat16 before they meet V,
// output accumulated in 32-bit and divided once at the end.  The mask follows
// engine/kernels/attention.py:31-33,75: the row at position p sees the keys n <= p (and, with a
// window, p - n < window); positions count from the sequence's length before the step, so the same
// kernel serves a whole prompt, a piece of one appended to a cache, and single tokens.
//
// Layout of the work.  The keys and values of the new rows are already in the cache.  For one
// sequence and one key/value head, the query rows are the pairs (new position, query head of the
// group), position-major, as in the reference's decode kernel (attention.py:46-48).  A block takes
// 64 such rows (four warps of 16) and walks the key pages (64 keys, one cache page each) that any
// of its rows can see, double-buffered through shared memory with cp.async; so one page of keys
// and values is read once for all query heads of the group.
#include "common.cuh"
#include "mma_utils.cuh"

#define AP_WARPS 4
#define AP_ROWS (AP_WARPS * 16)

template <int D>
__global__ void __launch_bounds__(AP_WARPS * 32)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, SbBatch batch, SbKV kv,
                    int n_heads, float scale_log2, int window) {
    constexpr int CH = D / 8;                   // 16-byte chunks per row
    constexpr int TILE = SB_PAGE * D * 2;       // bytes of one page of keys (or values) of one kv head
    constexpr int NT = D / 8;                   // output n-tiles
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                  // [64][D]
    unsigned char* kv_s = smem + AP_ROWS * D * 2;  // [2 stages][K tile | V tile]
    pdl_wait();

    const int seq = blockIdx.z, kvh = blockIdx.x;   // kv head fastest: blocks start longest first across all heads
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = n_heads / kv.n_kv_heads;
    const int slot = batch.seq_slot[seq];
    const int row0 = batch.cu_q[seq];
    const int q_len = batch.cu_q[seq + 1] - row0;
    const int start = batch.lengths[slot];                      // position of the sequence's first new row
    const int total = q_len * G;                                // (position, head) rows of this sequence and kv head
    const int tile = gridDim.y - 1 - blockIdx.y;                // latest rows (most keys) first
    const int t0 = tile * AP_ROWS;
    if (t0 >= total) return;
    const int t_last = min(t0 + AP_ROWS, total) - 1;
    const int pos_min = start + t0 / G, pos_max = start + t_last / G;
    const int lo_min = window > 0 ? max(0, pos_min - window + 1) : 0;
    const int first_page = lo_min / SB_PAGE, last_page = pos_max / SB_PAGE;
    const int n_pages = last_page - first_page + 1;

    // Query rows into shared memory (zero beyond the sequence's rows), then into fragments.
    for (int i = tid; i < AP_ROWS * CH; i += AP_WARPS * 32) {
        const int r = i / CH, c = i % CH;
        const int t = t0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < total)
            v = *reinterpret_cast<const uint4*>(q + ((long long)(row0 + t / G) * n_heads + kvh * G + t % G) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
    }
    __syncthreads();
    unsigned int qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(qf[ks], q_s + tile_off<D>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    const __nv_bfloat16* kbase = (const __nv_bfloat16*)kv.k;
    const __nv_bfloat16* vbase = (const __nv_bfloat16*)kv.v;
    const int* table = kv.table + (long long)slot * kv.table_width;
    // The ids of the block's pages are fetched once, 512 at a time: a lookup in the page table costs a
    // trip to L2, and paying it for every page would stall the copies behind it.
    __shared__ int s_pages[512];
    auto load_ids = [&](int base) {
        for (int j = tid; j < 512 && base + j < n_pages; j += AP_WARPS * 32) {
            int lp = first_page + base + j;
            if (kv.ring_pages) lp %= kv.ring_pages;
            s_pages[j] = max(table[lp], 0);
        }
    };
    load_ids(0);
    __syncthreads();
    auto issue = [&](int i) {
        if (i < n_pages) {
            const int page = s_pages[i & 511];
            const long long base = ((long long)page * kv.n_kv_heads + kvh) * SB_PAGE * D;
            unsigned char* ks = kv_s + (i & 1) * 2 * TILE;
            unsigned char* vs = ks + TILE;
            for (int j = tid; j < SB_PAGE * CH; j += AP_WARPS * 32) {
                const int r = j / CH, c = j % CH;
                cp_async_16(ks + tile_off<D>(r, c), kbase + base + r * D + c * 8);
                cp_async_16(vs + tile_off<D>(r, c), vbase + base + r * D + c * 8);
            }
        }
        cp_async_commit();
    };

    // This thread's two rows: their positions and first visible keys.
    const int tr0 = t0 + warp * 16 + (lane >> 2), tr1 = tr0 + 8;
    const int p0 = tr0 < total ? start + tr0 / G : -1, p1 = tr1 < total ? start + tr1 / G : -1;
    const int lo0 = window > 0 ? max(0, p0 - window + 1) : 0, lo1 = window > 0 ? max(0, p1 - window + 1) : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    issue(0);
    for (int i = 0; i < n_pages; ++i) {
        if (((i + 1) & 511) == 0) {   // the next page's id is in the next batch of ids
            __syncthreads();
            load_ids(i + 1);
            __syncthreads();
        }
        issue(i + 1);
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* ks = kv_s + (i & 1) * 2 * TILE;
        const unsigned char* vs = ks + TILE;
        const int key0 = (first_page + i) * SB_PAGE;
        // Values of keys that no row of this block may see (beyond its last position, before its first window)
        // are stale: they meet probabilities of exactly zero, but zero times an infinity or a NaN left by the
        // page's former owner would not be zero.  Only a block's last (and, with a window, first) page has such rows.
        if (key0 + SB_PAGE - 1 > pos_max || key0 < lo_min) {
            for (int j = tid; j < SB_PAGE * CH; j += AP_WARPS * 32) {
                const int r = j / CH, n = key0 + r;
                if (n > pos_max || n < lo_min)
                    *reinterpret_cast<uint4*>(const_cast<unsigned char*>(vs) + tile_off<D>(r, j % CH)) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();
        }
        // A warp whose rows all lie before this page, or whose windows all lie after it, has nothing here.
        const int w_first = t0 + warp * 16, w_last = min(w_first + 15, total - 1);
        const bool warp_has = w_first < total && key0 <= start + w_last / G &&
                              (window <= 0 || key0 + SB_PAGE - 1 >= start + w_first / G - window + 1);
        if (warp_has) {
            float s[SB_PAGE / 8][4];
#pragma unroll
            for (int nt = 0; nt < SB_PAGE / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int np = 0; np < SB_PAGE / 16; ++np) {
                    unsigned int b[4];
                    ldmatrix_x4(b, ks + tile_off<D>(np * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
                    mma_bf16(s[2 * np], qf[kk], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf[kk], b[2], b[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < SB_PAGE / 8; ++nt) {
                const int n = key0 + nt * 8 + (lane & 3) * 2;
                s[nt][0] = (n <= p0 && n >= lo0) ? s[nt][0] * scale_log2 : -INFINITY;
                s[nt][1] = (n + 1 <= p0 && n + 1 >= lo0) ? s[nt][1] * scale_log2 : -INFINITY;
                s[nt][2] = (n <= p1 && n >= lo1) ? s[nt][2] * scale_log2 : -INFINITY;
                s[nt][3] = (n + 1 <= p1 && n + 1 >= lo1) ? s[nt][3] * scale_log2 : -INFINITY;
                mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
            }
            float alpha[2], m_safe[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m[h], mx[h]);
                m_safe[h] = m_new == -INFINITY ? 0.f : m_new;
                alpha[h] = exp2f(m[h] - m_safe[h]);
                m[h] = m_new;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < SB_PAGE / 8; ++nt) {
                s[nt][0] = fast_exp2(s[nt][0] - m_safe[0]);
                s[nt][1] = fast_exp2(s[nt][1] - m_safe[0]);
                s[nt][2] = fast_exp2(s[nt][2] - m_safe[1]);
                s[nt][3] = fast_exp2(s[nt][3] - m_safe[1]);
                sum[0] += s[nt][0] + s[nt][1];
                sum[1] += s[nt][2] + s[nt][3];
            }
            l[0] = l[0] * alpha[0] + sum[0];
            l[1] = l[1] * alpha[1] + sum[1];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                acc[j][0] *= alpha[0]; acc[j][1] *= alpha[0];
                acc[j][2] *= alpha[1]; acc[j][3] *= alpha[1];
            }
#pragma unroll
            for (int kb = 0; kb < SB_PAGE / 16; ++kb) {   // 16 keys at a time
                unsigned int pf[4];
                pf[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
                pf[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
                pf[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
                pf[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    unsigned int b[4];
                    ldmatrix_x4_trans(b, vs + tile_off<D>(kb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, j + (lane >> 4)));
                    mma_bf16(acc[j], pf, b[0], b[1]);
                    mma_bf16(acc[j + 1], pf, b[2], b[3]);
                }
            }
        }
        __syncthreads();  // everyone is done with this stage before the copy after next lands in it
    }
    cp_async_wait<0>();

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const int cc = (lane & 3) * 2;
    if (tr0 < total) {
        const float inv = 1.0f / l[0];
        __nv_bfloat16* o = out + ((long long)(row0 + tr0 / G) * n_heads + kvh * G + tr0 % G) * D;
#pragma unroll
        for (int j = 0; j < NT; ++j)
            *reinterpret_cast<__nv_bfloat162*>(o + j * 8 + cc) = __floats2bfloat162_rn(acc[j][0] * inv, acc[j][1] * inv);
    }
    if (tr1 < total) {
        const float inv = 1.0f / l[1];
        __nv_bfloat16* o = out + ((long long)(row0 + tr1 / G) * n_heads + kvh * G + tr1 % G) * D;
#pragma unroll
        for (int j = 0; j < NT; ++j)
            *reinterpret_cast<__nv_bfloat162*>(o + j * 8 + cc) = __floats2bfloat162_rn(acc[j][2] * inv, acc[j][3] * inv);
    }
}

template <int D> static int launch_prefill(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale,
                                           int window, int max_q_len, cudaStream_t stream) {
    const int smem = AP_ROWS * D * 2 + 2 * 2 * SB_PAGE * D * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int G = n_heads / kv.n_kv_heads;
    const long long tiles = ((long long)max_q_len * G + AP_ROWS - 1) / AP_ROWS;
    if (tiles > 65535 || batch.n_seqs > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(kv.n_kv_heads, (unsigned int)tiles, batch.n_seqs);
    sb_launch(attn_prefill_kernel<D>, grid, AP_WARPS * 32, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, batch, kv,
                                                                  n_heads, scale * 1.4426950408889634f, window);
    return (int)cudaGetLastError();
}

// q, out [rows, n_heads * head_dim] bfloat16; max_q_len bounds the rows any sequence brings (it sizes the
// grid; blocks beyond a sequence's rows return at once).  Takes head_dim 64 or 128; anything else is refused.
extern "C" int sb_attn_prefill(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                               int max_q_len, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (n_heads % kv.n_kv_heads || max_q_len < 1) return (int)cudaErrorInvalidValue;
    if (kv.head_dim == 128) return launch_prefill<128>(q, out, batch, kv, n_heads, scale, window, max_q_len, stream);
    if (kv.head_dim == 64) return launch_prefill<64>(q, out, batch, kv, n_heads, scale, window, max_q_len, stream);
    return (int)cudaErrorInvalidValue;
}
