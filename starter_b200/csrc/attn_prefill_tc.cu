// Prefill attention on the Blackwell tensor cores: S = Q K^T and O = P V by tcgen05.mma, S and the
// page's O in tensor memory, keys and values brought in by TMA.  Head size 128, bfloat16.
//
// Same meaning and numerics as attn_prefill.cu (reference: engine/model.py:268-274 for the call,
// engine/kernels/attention.py:9-11,75 for the numerics and the mask): scores, maximum, exp and sum in
// 32-bit, probabilities rounded to bfloat16 before they meet V, 32-bit accumulation, one division.
//
// Layout of the work.  As in attn_prefill.cu the query rows of one sequence and one key/value head are
// the pairs (new position, query head of the group), position-major; a block takes 128 of them, one per
// thread and per lane of tensor memory.  Per key page (64 keys, one cache page):
//   a thread issues  S[128 x 64] = Q[128 x 128] K^T          (8 tcgen05.mma of K = 16, both operands K-major)
//   every row thread reads its row of S from tensor memory, masks, updates its running maximum and sum,
//   and writes its row of P (bfloat16) back into tensor memory, over the first half of the S it read
//   the thread issues  O[128 x 128] += P[128 x 64] V         (4 tcgen05.mma with P read from tensor memory; V as
//                                                             it lies in the cache, [key][d], is the MN-major form)
//   O stays in tensor memory across the pages; the rows rescale it only when their reference maximum moves.
// Who does what.  Warps 0-3 own the rows (softmax).  One thread of a fifth warp issues every tcgen05.mma, one thread
// of a sixth warp every TMA copy, and neither does anything else; two more warps only make the second group of four
// whole, so that it can hand registers to the first (setmaxnreg: the block starts with 128 a thread, the rows go on
// with 216, the others with 40; measured on one box against 192 threads of 168 registers: 55.8 -> 52.9 us at 2,048
// tokens, 155.8 -> 155.1 at 4,096, 505 -> 512 at 8,192: the short prompt, whose time is that of its longest blocks,
// gains; the split of the registers itself does not matter, 168 / 192 / 216 for the rows give the same times).  (A thread that also owned a row made its whole
// block wait; one thread issuing both products and copies needed ~2,500 clocks a page for its ~500 instructions and
// dozen barrier look-ups, and the rows waited for it: 612 -> 503 us at 8,192 tokens when the two were parted and the
// operand descriptors computed once.)  The products run ahead of the softmax: S of page i + 1 goes into the second of
// two S buffers in tensor memory while the rows work on page i, and O += P V of page i runs while they start on
// page i + 1.  Keys arrive two pages ahead and values one page ahead, in two stages each.  Rows, products and copies
// meet only through mbarriers (keys landed, values landed, S ready, O done, P written); there is no block-wide
// barrier inside the loop.  Two blocks share an SM (97 KB of shared memory and 256 columns of tensor memory each).
// Measured on a B200, and what it means for this kernel: the tensor core takes 48 clocks for a product of N = 64
// and 64 for N = 128 (K = 16), whether operand A comes from shared or tensor memory and however the products
// depend on one another, but a group of products that ends in a commit costs 250-450 clocks more when the block
// has nothing else queued (two blocks fill one another's gaps: together 620 clocks a page); the exp2 unit takes
// 8 clocks per warp instruction, so a page's 64 exponentials per row cost 512 clocks per warp, 587 when two warps
// share a scheduler, 800 for a warp alone.  With two blocks per SM a page per block takes ~1,900 clocks: ~1,150
// for the exponentials of both blocks' rows (they share the exp2 unit) and ~700 for the trips to tensor memory and
// the barriers around them.  Exponentials on the FMA units (a cubic) were measured and are slower at two warps per
// scheduler; so were two threads per row, and the read of the next S overlapped with the write of P.
// Every wait on an mbarrier is bounded; on a time-out the block raises SB_STATUS_TIMEOUT and a flag in shared
// memory that ends every other wait of the block, which then frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "tc_utils.cuh"

#define PT_ROWS 128
#define PT_D 128
#define PT_IDS 128
#define PT_THREADS 256   // two groups of four warps: the rows; and the warp of the thread that issues the products, that of the thread that
                         // issues the copies and two spare ones, which together hand most of their registers to the rows

#ifdef SB_TIMELINE
// Tuning builds only: clock stamps of one block's issuer and of its first row, per page: [page][8].
static __device__ long long* pt_timeline = nullptr;
extern "C" int sb_attn_prefill_tc_timeline(long long* p) { return (int)cudaMemcpyToSymbol(pt_timeline, &p, sizeof(p)); }
#define PT_STAMP(page, what) do { if (pt_timeline && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (page) < 64) pt_timeline[(page) * 8 + (what)] = clock64(); } while (0)
#else
#define PT_STAMP(page, what) ((void)0)
#endif


__global__ void __launch_bounds__(PT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, SbBatch batch, SbKV kv,
                       int n_heads, float scale_log2, int window, int* status) {
    constexpr int Q_ATOM = PT_ROWS * 128;          // bytes of a [128 rows][64 d] block of Q
    constexpr int KV_ATOM = SB_PAGE * 128;         // bytes of a [64 keys][64 d] block of K or V
    constexpr int STAGE = 2 * KV_ATOM;             // one page of keys (or values) of one kv head
    extern __shared__ __align__(1024) unsigned char smem[];   // no static shared memory: the window starts 1024-aligned
    unsigned char* q_s = smem;                     // 2 blocks of [128][64]
    unsigned char* k_s = q_s + 2 * Q_ATOM;         // [2 stages][2 blocks of [64][64]]
    unsigned char* v_s = k_s + 2 * STAGE;          // [2 stages][2 blocks of [64][64]]
    uint64_t* bars = (uint64_t*)(v_s + 2 * STAGE);
    uint64_t* k_full = bars;                       // [2] keys of a page have landed in stage i & 1
    uint64_t* v_full = bars + 2;                   // [2] values likewise
    uint64_t* s_done = bars + 4;                   // [2] S of page i is in S buffer i & 1 (and every product issued before it is done)
    uint64_t* o_done = bars + 6;                   // [2] O += P V of page i is done
    uint64_t* p_ready = bars + 8;                  // every row has read S of page i and written its P (128 arrivals)
    uint32_t* tmem_slot = (uint32_t*)(bars + 9);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* s_pages = (int*)(tmem_slot + 4);          // [PT_IDS] ids of the block's next pages
    if ((smem_u32(smem) & 1023u) != 0) {           // the swizzled tiles need it; never seen, but never assumed
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_TIMEOUT);
        return;
    }

    const int seq = blockIdx.z, kvh = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int G = n_heads / kv.n_kv_heads;
    const int slot = batch.seq_slot[seq];
    const int row0 = batch.cu_q[seq];
    const int q_len = batch.cu_q[seq + 1] - row0;
    const int start = batch.lengths[slot];
    const int total = q_len * G;
    // Blocks start in the order of their index, x fastest: with the kv head in x and the row tile in y, the blocks of a
    // sequence start longest first across all heads (latest rows = most keys), and the short ones fill the gaps at the
    // end.  With the tile in x the long blocks of the last heads started late: 78 against 58 us at 2,048 tokens.
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int t0 = tile * PT_ROWS;
    if (t0 >= total) return;
    const int t_last = min(t0 + PT_ROWS, total) - 1;
    const int pos_min = start + t0 / G, pos_max = start + t_last / G;
    const int lo_min = window > 0 ? max(0, pos_min - window + 1) : 0;
    const int first_page = lo_min / SB_PAGE, last_page = pos_max / SB_PAGE;
    const int n_pages = last_page - first_page + 1;

    const int* table = kv.table + (long long)slot * kv.table_width;
    // Up to here only the batch's description and the lengths were read, which the kernel before this one (the
    // rotary encoding and cache store) does not write; from here on its queries, keys and values are.
    pdl_wait();
    if (tid == PT_ROWS) {
        // The issuing thread sets the barriers up and asks for the first keys and values at once, so that they
        // travel while the rows stage their queries and tensor memory is handed out.
#pragma unroll
        for (int b = 0; b < 8; ++b) mbar_init(&bars[b], 1);
        mbar_init(p_ready, PT_ROWS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < 2 && i < n_pages; ++i) {
            int lp = first_page + i;
            if (kv.ring_pages) lp %= kv.ring_pages;
            const int y = (max(table[lp], 0) * kv.n_kv_heads + kvh) * SB_PAGE;
            mbar_expect_tx(&k_full[i], STAGE);
            tma_load_2d(k_s + i * STAGE, &map_k, 0, y, &k_full[i]);
            tma_load_2d(k_s + i * STAGE + KV_ATOM, &map_k, 64, y, &k_full[i]);
            if (i == 0) {
                mbar_expect_tx(&v_full[0], STAGE);
                tma_load_2d(v_s, &map_v, 0, y, &v_full[0]);
                tma_load_2d(v_s + KV_ATOM, &map_v, 64, y, &v_full[0]);
            }
        }
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // This thread's query row into shared memory, in the swizzled K-major layout the tensor core reads.
    const bool owns_row = tid < PT_ROWS;
    const int t = t0 + tid;
    const int pos = t < total ? start + t / G : -1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (owns_row) {
        const __nv_bfloat16* src = q + ((long long)(row0 + (t < total ? t / G : 0)) * n_heads + kvh * G + (t < total ? t % G : 0)) * PT_D;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (t < total) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(q_s + (c >> 3) * Q_ATOM + tid * 128 + (((c & 7) ^ (tid & 7)) << 4)) = v;
        }
    }
    // Ids of the block's pages: a ring of PT_IDS entries in two halves.  Both halves are filled at the start;
    // every 64 pages the rows refill the half whose pages are behind them with the pages 64 to 127 ahead.
    auto load_ids = [&](int first, int count) {
        for (int j = tid; j < count && first + j < n_pages; j += PT_ROWS) {
            int lp = first_page + first + j;
            if (kv.ring_pages) lp %= kv.ring_pages;
            s_pages[(first + j) & (PT_IDS - 1)] = max(table[lp], 0);
        }
    };
    if (owns_row) load_ids(0, PT_IDS);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q was written by ordinary stores
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // The rows hold a page's 64 scores and their packed probabilities in registers; the other warps need a few dozen.
    // The block starts with 128 registers a thread and deals them out anew, each group at the head of its own branch;
    // the branches do not meet again (code after a meeting would have to live with the smaller number).
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_row = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 lanes
    const uint32_t idesc_s = umma_idesc(SB_PAGE, 0), idesc_o = umma_idesc(PT_D, 1);
    constexpr uint32_t O_COL = 2 * SB_PAGE;        // tensor memory: S buffers at columns 0 and 64, O from 128

    if (!owns_row) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
        // ---- two threads of two further warps.  One issues the products, the other the copies; each has only its own
        // waits in its loop (one thread doing both needed ~2,500 clocks a page for its ~500 instructions and a dozen
        // barrier look-ups, and the rows waited for it).  Page i lives in stage i & 1; a barrier of index i & 1 is in
        // phase (i >> 1) & 1 when page i's event completes.
        if (tid == PT_ROWS) {
            // The descriptors of the operands: one each for Q and for K and V of both stages; a step of 16 columns (32
            // bytes) or a further block of 64 columns adds a constant to the address field.
            const uint64_t q_desc0 = desc_k_major(q_s);
            const uint64_t k_desc0[2] = {desc_k_major(k_s), desc_k_major(k_s + STAGE)};
            const uint64_t v_desc0[2] = {desc_mn_major(v_s, KV_ATOM), desc_mn_major(v_s + STAGE, KV_ATOM)};
            auto issue_s = [&](int i) {   // S of page i into S buffer i & 1
                mbar_wait(&k_full[i & 1], (i >> 1) & 1, abort_flag, status);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < PT_D / 16; ++ks)
                    tc_mma(tmem + (i & 1) * SB_PAGE, q_desc0 + (ks >> 2) * (Q_ATOM >> 4) + 2 * (ks & 3),
                           k_desc0[i & 1] + (ks >> 2) * (KV_ATOM >> 4) + 2 * (ks & 3), idesc_s, ks > 0 ? 1u : 0u);
                tc_commit(&s_done[i & 1]);
            };
            issue_s(0);
            for (int i = 0; i < n_pages && !*abort_flag; ++i) {
                const int b = i & 1;
                // S of the next page: its buffer was read by the rows in iteration i - 1 (p_ready of i - 1, waited for
                // below), and the product that read P from it was issued before this one.
                if (i + 1 < n_pages) issue_s(i + 1);
                PT_STAMP(i, 0);
                mbar_wait(p_ready, i & 1, abort_flag, status);        // P of page i is written (and O rescaled if need be)
                PT_STAMP(i, 1);
                mbar_wait(&v_full[b], (i >> 1) & 1, abort_flag, status);
                if (*abort_flag) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < SB_PAGE / 16; ++ks)   // 16 keys per step: 32 bytes = 8 columns along P's rows
                    tc_mma_ts(tmem + O_COL, tmem + b * SB_PAGE + 8 * ks, v_desc0[b] + ks * (2048 >> 4), idesc_o,
                              (i > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&o_done[b]);
                PT_STAMP(i, 2);
            }
        } else if (tid == PT_ROWS + 32) {
            // The copies.  Keys of pages 0 and 1 and values of page 0 were asked for at the block's start.
            auto issue_kv = [&](int i, unsigned char* base, const CUtensorMap* map, uint64_t* bar) {
                const int y = (s_pages[i & (PT_IDS - 1)] * kv.n_kv_heads + kvh) * SB_PAGE;
                mbar_expect_tx(bar, STAGE);
                tma_load_2d(base + (i & 1) * STAGE, map, 0, y, bar);
                tma_load_2d(base + (i & 1) * STAGE + KV_ATOM, map, 64, y, bar);
            };
            for (int i = 0; i < n_pages && !*abort_flag; ++i) {
                if (i + 1 < n_pages) {   // values of the next page go into the stage of page i - 1, once its product is done
                    if (i > 0) mbar_wait(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, status);
                    if (*abort_flag) break;
                    issue_kv(i + 1, v_s, &map_v, &v_full[(i + 1) & 1]);
                }
                if (i + 2 < n_pages) {   // keys two pages ahead go into the stage of page i, once S of page i has read it
                    mbar_wait(&s_done[i & 1], (i >> 1) & 1, abort_flag, status);
                    if (*abort_flag) break;
                    issue_kv(i + 2, k_s, &map_k, &k_full[i & 1]);
                }
            }
            if (*abort_flag) {   // leaving early: give the copies in flight a bounded time to land
                const long long t_abort = clock64();
                while (clock64() - t_abort < (1ll << 22)) {}
            }
        }
        tc_fence_before();
        __syncthreads();   // the block's last meeting: the rows free tensor memory after it
        return;
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;" ::: "memory");
        // ---- the rows.  The output accumulates in tensor memory across pages.  The probabilities of a page are
        // taken relative to a reference maximum m_ref that is raised only when the row's maximum exceeds it by
        // more than 8 (in the log2 domain): then the row's sum and its accumulator are rescaled once.  Until then
        // a probability may be as large as 2^8, which bfloat16 and the 32-bit sums hold without loss, and
        // the final division by the sum removes the common factor.
        float m_ref = -INFINITY, l_run = 0.f;
        const int lo_max = window > 0 ? max(0, pos_max - window + 1) : 0;
        for (int i = 0; i < n_pages; ++i) {
            const int b = i & 1;
            if (i > 0 && (i & 63) == 0) load_ids(i + 64, 64);   // read by the issuer 62 pages (and as many barriers) from now
            if (tid == 0) PT_STAMP(i, 7);
            mbar_wait(&s_done[b], (i >> 1) & 1, abort_flag, status);
            if (*abort_flag) break;
            tc_fence_after();
            if (tid == 0) PT_STAMP(i, 3);

            // This thread's row of scores: mask (only where the page is not wholly visible), maximum, probabilities.
            const int key0 = (first_page + i) * SB_PAGE;
            float s[SB_PAGE];
            {
                uint32_t* raw = reinterpret_cast<uint32_t*>(s);   // both halves asked for, then one wait
                tc_ld32_async(tmem_row + b * SB_PAGE, raw);
                tc_ld32_async(tmem_row + b * SB_PAGE + 32, raw + 32);
                tc_wait_ld();
            }
            tc_fence_before();   // ordered before the arrival below, after which the issuer may overwrite this buffer
            if (tid == 0) PT_STAMP(i, 4);
            const bool whole_page_visible = key0 + SB_PAGE - 1 <= pos_min && key0 >= lo_max && t_last == t0 + PT_ROWS - 1;
            if (!whole_page_visible) {
#pragma unroll
                for (int c = 0; c < SB_PAGE; ++c) {
                    const int n = key0 + c;
                    if (!(n <= pos && n >= lo)) s[c] = -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains of three-input maxima
#pragma unroll
            for (int c = 0; c < SB_PAGE; c += 8) {
                mx4[0] = max_of_three(mx4[0], s[c], s[c + 1]); mx4[1] = max_of_three(mx4[1], s[c + 2], s[c + 3]);
                mx4[2] = max_of_three(mx4[2], s[c + 4], s[c + 5]); mx4[3] = max_of_three(mx4[3], s[c + 6], s[c + 7]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale_log2 > 0: the maximum commutes with it
            float alpha = 1.0f;
            if (mx > m_ref + 8.0f || m_ref == -INFINITY) {
                const float m_new = fmaxf(m_ref, mx);
                alpha = m_new == -INFINITY ? 1.0f : exp2f(m_ref - m_new);   // 0 when the reference was -inf
                m_ref = m_new;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            uint4 packed[SB_PAGE / 8];
            // The rows' time is their instruction count: scale-and-shift and the running sums work on pairs.
            const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-m_use, -m_use);
            float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < SB_PAGE; c += 8) {
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed[c >> 3]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 x = fma_pair(make_float2(s[c + 2 * e], s[c + 2 * e + 1]), scale2, shift2);
                    const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    sum2[e] = add_pair(sum2[e], pr);
                    h2[e] = __floats2bfloat162_rn(pr.x, pr.y);
                }
            }
            l_run = l_run * alpha + (((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y)) + ((sum2[2].x + sum2[2].y) + (sum2[3].x + sum2[3].y)));

            // The accumulator of earlier pages moves to the new reference (rare after the first pages): O += P V of
            // the page before must be done before it is rescaled.
            if (i > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                mbar_wait(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, status);
                if (*abort_flag) break;
                tc_fence_after();
#pragma unroll
                for (int d0 = 0; d0 < PT_D; d0 += 32) {
                    float o[32];
                    tc_ld32(tmem_row + O_COL + d0, o);
#pragma unroll
                    for (int d = 0; d < 32; ++d) o[d] *= alpha;
                    tc_st32(tmem_row + O_COL + d0, o);
                }
            }
            // Values of keys that no row of this block may see (beyond its last position, before its first window)
            // are stale: they meet probabilities of exactly zero, but zero times an infinity or a NaN left by the
            // page's former owner would not be zero.  Only a block's last (and, with a window, first) page has such
            // rows; thread k clears the row of key k once the values have landed.
            if (key0 + SB_PAGE - 1 > pos_max || key0 < lo_min) {
                mbar_wait(&v_full[b], (i >> 1) & 1, abort_flag, status);
                if (*abort_flag) break;
                if (tid < SB_PAGE && (key0 + tid > pos_max || key0 + tid < lo_min)) {
                    unsigned char* vt = v_s + b * STAGE;
#pragma unroll
                    for (int c = 0; c < 16; ++c)   // [2 blocks of 64 columns][64 keys][128 bytes]: the whole row, whatever the swizzle
                        *reinterpret_cast<uint4*>(vt + (c >> 3) * KV_ATOM + tid * 128 + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // ordinary stores, read by the tensor core
                }
            }
            // P goes where this row's S was: 64 bfloat16 = 32 columns of the S buffer, which the product reads as its
            // operand A straight from tensor memory.  (The tensor core runs a block's products in the order they were
            // issued: S of page i + 2, which overwrites this buffer, is issued after O += P V of page i.)
            if (tid == 0) PT_STAMP(i, 5);
            tc_st32_u32(tmem_row + b * SB_PAGE, reinterpret_cast<const uint32_t*>(packed));
            tc_fence_before();
            mbar_arrive(p_ready);
            if (tid == 0) PT_STAMP(i, 6);
        }
        if (!*abort_flag) {   // the last product, then this row's output
            mbar_wait(&o_done[(n_pages - 1) & 1], ((n_pages - 1) >> 1) & 1, abort_flag, status);
            tc_fence_after();
        }
        if (!*abort_flag) {
            const float inv = 1.0f / l_run;
            __nv_bfloat16* o_row = out + ((long long)(row0 + (t < total ? t / G : 0)) * n_heads + kvh * G + (t < total ? t % G : 0)) * PT_D;
#pragma unroll
            for (int d0 = 0; d0 < PT_D; d0 += 32) {
                float o[32];
                tc_ld32(tmem_row + O_COL + d0, o);
                if (t < total) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 packed;
                        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                        *reinterpret_cast<uint4*>(o_row + d0 + d) = packed;
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();
        if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
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
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// The pages of one layer's keys (or values) as a matrix [pages * kv_heads * 64 rows][128 columns] of
// bfloat16, read in boxes of 64 rows x 64 columns with the 128-byte swizzle.
static int make_page_map(CUtensorMap* map, const void* ptr, long long rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {PT_D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {PT_D * 2};
    cuuint32_t box[2] = {64, SB_PAGE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// q, out [rows, n_heads * 128] bfloat16; n_pages: pages in the layer's pool (the null page included);
// max_q_len bounds the rows any sequence brings.  Head size 128 only.
extern "C" int sb_attn_prefill_tc(const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale, int window,
                                  int max_q_len, int n_pages, int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (kv.head_dim != PT_D || n_heads % kv.n_kv_heads || max_q_len < 1 || n_pages < 1) return (int)cudaErrorInvalidValue;
    const int smem = 2 * PT_ROWS * 128 + 4 * 2 * SB_PAGE * 128 + 96 + PT_IDS * 4;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap mk, mv;
    const long long rows = (long long)n_pages * kv.n_kv_heads * SB_PAGE;
    int e = make_page_map(&mk, kv.k, rows);
    if (e) return e;
    e = make_page_map(&mv, kv.v, rows);
    if (e) return e;
    const int G = n_heads / kv.n_kv_heads;
    const long long tiles = ((long long)max_q_len * G + PT_ROWS - 1) / PT_ROWS;
    if (tiles > 65535 || batch.n_seqs > 65535) return (int)cudaErrorInvalidValue;
    dim3 grid(kv.n_kv_heads, (unsigned int)tiles, batch.n_seqs);
    sb_launch(attn_prefill_tc_kernel, grid, PT_THREADS, smem, stream, mk, mv, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, batch, kv, n_heads,
              scale * 1.4426950408889634f, window, status);
    return (int)cudaGetLastError();
}
