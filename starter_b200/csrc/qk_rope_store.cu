// Per-head RMSNorm of q and k, rotary positions, q to its buffer, k and v into the paged cache.
//
// Reference: engine/kernels/rope.py:19-30 (row arithmetic) and :95-144 (one launch for all
// heads): n = T(x * rsqrt(mean(x^2) + eps)); y = T(w * n); with rotate-half pairing (d, d + R/2)
//   out[d]       = T( T(y[d] * cos) + T(-y[d + R/2] * sin) )
//   out[d + R/2] = T( T(y[d + R/2] * cos) + T(y[d] * sin) )
// and v copied as it is.  T is float (nothing is rounded) or bfloat16.  The cos/sin tables
// hold R/2 columns per position, because columns d and d + R/2 share an angle
// (engine/model.py:91).  A row's position is its sequence's length before the step plus
// its place among the sequence's new rows.
#include "common.cuh"

#define QK_MAX_D 512

// grid (rows, n_heads + n_kv_heads), one warp per head vector.
template <class T, class W>
__global__ void qk_rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, SbBatch batch, SbKV kv,
                                     int n_heads, int n_kv_heads, const W* __restrict__ q_norm_w,
                                     const W* __restrict__ k_norm_w, float eps, const T* __restrict__ cos_t,
                                     const T* __restrict__ sin_t, int rotary_dim, int* status) {
    __shared__ float y[QK_MAX_D];
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int D = kv.head_dim;
    const int width = (n_heads + 2 * n_kv_heads) * D;
    const bool is_q = head < n_heads;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const T* src = qkv + (long long)row * width + (long long)head * D;
    const W* w = is_q ? q_norm_w : k_norm_w;

    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float v = to_f<T>(src[d]);
        y[d] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    __syncwarp();
    if (w != nullptr) {
        const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) {
            const float n = rnd<T>(__fmul_rn(y[d], rstd));
            y[d] = rnd<T>(__fmul_rn(to_f<W>(w[d]), n));
        }
        __syncwarp();
    }

    T* dst;
    if (is_q) {
        dst = q_out + (long long)row * n_heads * D + (long long)head * D;
    } else {
        const long long off = kv_offset(kv, slot, pos, head - n_heads);
        if (off < 0) {
            if (lane == 0) atomicOr(status, SB_STATUS_NO_PAGE);
            return;
        }
        dst = (T*)kv.k + off;
        const T* vsrc = src + (long long)n_kv_heads * D;
        T* vdst = (T*)kv.v + off;
        for (int d = lane; d < D; d += 32) vdst[d] = vsrc[d];
    }
    const int half = rotary_dim / 2;
    for (int d = lane; d < D; d += 32) {
        float o = y[d];
        if (cos_t != nullptr && d < rotary_dim) {
            const int j = d < half ? d : d - half;
            const float c = to_f<T>(cos_t[(long long)pos * half + j]);
            const float s = to_f<T>(sin_t[(long long)pos * half + j]);
            const float a = rnd<T>(__fmul_rn(y[d], c));
            const float b = d < half ? rnd<T>(__fmul_rn(-y[d + half], s)) : rnd<T>(__fmul_rn(y[d - half], s));
            o = __fadd_rn(a, b);
        }
        dst[d] = from_f<T>(o);
    }
}

// qkv [rows, (n_heads + 2 n_kv_heads) * D]; q_out [rows, n_heads * D]; norm weights may be null
// (no per-head norm); cos/sin [positions, rotary_dim / 2] may be null (no rotary encoding).
// With n_kv_heads == 0 only q is processed and nothing is stored (a layer that reads another's cache).
extern "C" int sb_qk_rope_store(int dtype, int wdtype, const void* qkv, void* q_out, SbBatch batch, SbKV kv, int n_heads,
                                int n_kv_heads, const void* q_norm_w, const void* k_norm_w, float eps, const void* cos_t,
                                const void* sin_t, int rotary_dim, int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (kv.head_dim > QK_MAX_D || rotary_dim > kv.head_dim || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    dim3 grid(batch.n_rows, n_heads + n_kv_heads);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define SB_QK(T, W)                                                                                                    \
    sb_launch(qk_rope_store_kernel<T, W>, grid, 32, 0, stream, (const T*)qkv, (T*)q_out, batch, kv, n_heads, n_kv_heads,        \
                                                        (const W*)q_norm_w, (const W*)k_norm_w, eps, (const T*)cos_t,   \
                                                        (const T*)sin_t, rotary_dim, status)
    if (dtype == SB_F32) {
        if (wdtype != SB_F32) return (int)cudaErrorInvalidValue;
        SB_QK(float, float);
    } else if (wdtype == SB_F32) {
        SB_QK(__nv_bfloat16, float);
    } else {
        SB_QK(__nv_bfloat16, __nv_bfloat16);
    }
#undef SB_QK
    SB_LAUNCH_CHECK();
}
