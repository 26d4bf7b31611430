// Shared definitions of the sm_100a kernels: element types, the step's batch
// description, the paged key/value view of one layer, and small helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SB_PAGE 64  // tokens per cache page; must match starter_b200.cache.cache.PAGE

enum { SB_F32 = 0, SB_BF16 = 1 };
enum { SB_STATUS_BAD_TOKEN = 1, SB_STATUS_NO_PAGE = 2 };

// A step's ragged batch.  Row r belongs to sequence row_seq[r]; that sequence sits in
// cache slot seq_slot[s], brought rows cu_q[s]..cu_q[s+1]-1, and held lengths[slot]
// tokens before the step, so row r stands at position lengths[slot] + r - cu_q[s].
struct SbBatch {
    const int* seq_slot;
    const int* cu_q;
    const int* row_seq;
    const int* lengths;
    int n_seqs;
    int n_rows;
    int null_slot;
    int reserved;
};

// One layer's keys and values: pages [page][kv_head][SB_PAGE][head_dim]; the page of
// position p of a slot is table[slot][p / SB_PAGE], or table[slot][(p / SB_PAGE) % ring_pages]
// for a window group that keeps a ring of pages.
struct SbKV {
    void* k;
    void* v;
    const int* table;
    int table_width;
    int ring_pages;
    int n_kv_heads;
    int head_dim;
};

template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// The value as it reads back after being stored in T.
template <class T> __device__ __forceinline__ float rnd(float v) { return to_f<T>(from_f<T>(v)); }

// 2^x in one instruction (relative error 2^-22, tiny results flushed to zero; 2^-inf = 0).  The probabilities of
// the attention kernels are rounded to bfloat16 right after, so the full-precision routine buys nothing there.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two 32-bit operations in one instruction (sm_100): a * b + c and a + b on pairs, each element rounded as the single
// operation rounds it; and the largest of three.  For loops whose time is their instruction count.
__device__ __forceinline__ float2 fma_pair(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 add_pair(float2 a, float2 b) {
    float2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ void row_place(const SbBatch& b, int row, int& slot, int& pos) {
    const int s = b.row_seq[row];
    slot = b.seq_slot[s];
    pos = b.lengths[slot] + row - b.cu_q[s];
}

// Element offset of [page][kv_head][pos % SB_PAGE][0] for a slot's position, or -1 when the
// slot has no page there.
__device__ __forceinline__ long long kv_offset(const SbKV& kv, int slot, int pos, int kv_head) {
    int lp = pos / SB_PAGE;
    if (kv.ring_pages) lp %= kv.ring_pages;
    if (lp >= kv.table_width) return -1;
    const int page = kv.table[(long long)slot * kv.table_width + lp];
    if (page < 0) return -1;
    return (((long long)page * kv.n_kv_heads + kv_head) * SB_PAGE + (pos % SB_PAGE)) * kv.head_dim;
}

// Programmatic dependent launch.  A kernel launched with the attribute may start while the kernel before
// it in the stream is still running; it must call pdl_wait() before it reads anything that kernel
// wrote (or writes anything that kernel reads).  What comes before the wait (fetching weights, setting
// up barriers) overlaps the predecessor's tail.  pdl_launch_dependents() lets the next kernel in the
// stream start its own preamble before this one has ended; a kernel that never calls it releases its
// successor when it ends.  Without the attribute both are no-ops.
// Measured on a decode step of 36 layers at batch 8 (B200): attribute and waits alone 3.32 ms against
// 3.45 ms without; the early release in the matrix products as well 3.30 ms (and 369 against 358 tokens
// a second at batch 1); an early release in the attention kernels as well 3.55 ms, so they have none.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Ask for `bytes` at p to be brought into L2 without waiting for them (p 16-byte aligned, bytes a multiple of 16).
__device__ __forceinline__ void l2_prefetch(const void* p, unsigned int bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Share `part` of `parts` of the range [p, p + total): one thread asks for it in pieces of 16 KB.
__device__ __forceinline__ void l2_prefetch_share(const void* p, long long total, long long part, long long parts) {
    if (p == nullptr || total <= 0) return;
    const long long share = (((total + parts - 1) / parts) + 255) & ~255ll;
    long long lo = part * share;
    const long long hi = lo + share < total ? lo + share : (total & ~15ll);
    constexpr long long PIECE = 16384;
    for (; lo < hi; lo += PIECE)
        l2_prefetch(reinterpret_cast<const unsigned char*>(p) + lo, (unsigned int)(hi - lo < PIECE ? hi - lo : PIECE));
}

// Tuning aid, compiled in with -DSB_TIMELINE only: thread 0 of a block appends (time, kernel, milestone, block)
// to a log on the device, from which a script draws the step's timeline.  Each source file has its own
// pointer to the log, set through the function that SB_TIMELINE_SETTER defines for it.
#ifdef SB_TIMELINE
static __device__ unsigned long long* sb_tl_log = nullptr;   // [0] entries used, [1] capacity, then pairs (time, tag)
__device__ __forceinline__ void sb_stamp(int kernel, int milestone) {
    if (threadIdx.x != 0 || sb_tl_log == nullptr) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned long long i = atomicAdd(sb_tl_log, 1ull);
    if (i >= sb_tl_log[1]) return;
    const unsigned long long block = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    sb_tl_log[2 + 2 * i] = t;
    sb_tl_log[3 + 2 * i] = ((unsigned long long)kernel << 48) | ((unsigned long long)milestone << 40) | block;
}
#define SB_TIMELINE_SETTER(name) \
    extern "C" int sb_timeline_##name(void* log) { return (int)cudaMemcpyToSymbol(sb_tl_log, &log, sizeof(log)); }
#else
#define sb_stamp(kernel, milestone) ((void)0)
#define SB_TIMELINE_SETTER(name)
#endif

extern int sb_pdl_flag;  // set through sb_set_pdl(); defined in rows.cu

template <typename... Exp, typename... Act>
static inline void sb_launch(void (*kernel)(Exp...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Act&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = sb_pdl_flag ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, static_cast<Act&&>(args)...);
}

// The same with the blocks grouped into clusters of `cluster` blocks (a dimension of 0 or 1 = no grouping).
template <typename... Exp, typename... Act>
static inline void sb_launch_cluster(void (*kernel)(Exp...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t stream,
                                     Act&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (sb_pdl_flag) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    config.attrs = attr;
    config.numAttrs = n;
    cudaLaunchKernelEx(&config, kernel, static_cast<Act&&>(args)...);
}

#define SB_LAUNCH_CHECK() return (int)cudaGetLastError()
