// Causal grouped-query attention of a step's rows over the paged cache: any head size up
// to 256, any number of heads and groups, any mix of row counts per sequence, with or
// without a window.  One warp per (row, query head); keys in order, 32 at a time.
//
// Reference: engine/kernels/attention.py:24-92.  Scores (q.k)*scale, running maximum,
// exp and the sum l in 32-bit; the probabilities are rounded to T before they meet V
// (attention.py:83); the 32-bit accumulator is divided by l once at the end
// (attention.py:86-87).  Key n is visible to the row at position p when n <= p
// (attention.py:75) and, with a window, p - n < window.  Query head h reads key/value head
// h / (n_heads / n_kv_heads).  Tiles start at multiples of 32 in key index, so a row's
// result depends on its position and its keys only, not on the batch around it.
#include "common.cuh"

#define AG_MAX_D 256

// q . k over D elements, in index order; 16-byte loads when the row allows them.
__device__ __forceinline__ float dot_row(const float* qs, const float* kr, int D) {
    float dot = 0.f;
    if ((D & 3) == 0) {
        for (int d = 0; d < D; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(kr + d);
            dot = fmaf(qs[d], v.x, dot);
            dot = fmaf(qs[d + 1], v.y, dot);
            dot = fmaf(qs[d + 2], v.z, dot);
            dot = fmaf(qs[d + 3], v.w, dot);
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], kr[d], dot);
    }
    return dot;
}

__device__ __forceinline__ float dot_row(const float* qs, const __nv_bfloat16* kr, int D) {
    float dot = 0.f;
    if ((D & 7) == 0) {
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                dot = fmaf(qs[d + 2 * e], f.x, dot);
                dot = fmaf(qs[d + 2 * e + 1], f.y, dot);
            }
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], __bfloat162float(kr[d]), dot);
    }
    return dot;
}

template <class T>
__global__ void attention_general_kernel(const T* __restrict__ q, T* __restrict__ out, SbBatch batch, SbKV kv,
                                         int n_heads, float scale, int window) {
    __shared__ float qs[AG_MAX_D];
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int D = kv.head_dim;
    const int kvh = head / (n_heads / kv.n_kv_heads);
    int slot, pos;
    row_place(batch, row, slot, pos);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    const T* qr = q + ((long long)row * n_heads + head) * D;
    for (int d = lane; d < D; d += 32) qs[d] = to_f<T>(qr[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_D / 32];
#pragma unroll
    for (int j = 0; j < AG_MAX_D / 32; ++j) acc[j] = 0.f;
    const T* kbase = (const T*)kv.k;
    const T* vbase = (const T*)kv.v;

    for (int n0 = (lo / 32) * 32; n0 <= pos; n0 += 32) {
        const int n = n0 + lane;
        const bool valid = n >= lo && n <= pos;
        long long off = valid ? kv_offset(kv, slot, n, kvh) : -1;
        float s = -INFINITY;
        if (off >= 0) {
            s = dot_row(qs, kbase + off, D) * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;  // no key of this tile has a page: nothing to add
        const float p = off >= 0 ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + warp_sum(p);
        m = m_new;
        const float pr = rnd<T>(p);
#pragma unroll
        for (int j = 0; j < AG_MAX_D / 32; ++j) acc[j] *= alpha;
        for (int t = 0; t < 32; ++t) {
            const long long voff = __shfl_sync(0xffffffffu, off, t);
            const float pt = __shfl_sync(0xffffffffu, pr, t);
            if (voff < 0) continue;
            const T* vr = vbase + voff;
#pragma unroll
            for (int j = 0; j < AG_MAX_D / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < D) acc[j] = fmaf(pt, to_f<T>(vr[d]), acc[j]);
            }
        }
    }
    T* orow = out + ((long long)row * n_heads + head) * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < AG_MAX_D / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < D) orow[d] = from_f<T>(acc[j] * inv);
    }
}

// q, out [rows, n_heads * head_dim]; window <= 0 means every earlier key.
extern "C" int sb_attention_general(int dtype, const void* q, void* out, SbBatch batch, SbKV kv, int n_heads, float scale,
                                    int window, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (kv.head_dim > AG_MAX_D || n_heads % kv.n_kv_heads) return (int)cudaErrorInvalidValue;
    dim3 grid(batch.n_rows, n_heads);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(attention_general_kernel<float>, grid, 32, 0, stream, (const float*)q, (float*)out, batch, kv, n_heads, scale, window);
    else
        sb_launch(attention_general_kernel<__nv_bfloat16>, grid, 32, 0, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, batch,
                                                                         kv, n_heads, scale, window);
    SB_LAUNCH_CHECK();
}
