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
    sb_stamp(3, 0);
    pdl_wait();
    pdl_launch_dependents();   // the attention that follows looks up its pages and fetches old keys meanwhile
    sb_stamp(3, 1);
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
    sb_stamp(3, 2);
}


// The common case on the tensor-core path: bfloat16, head size 128, rotary over the whole head.  One block
// per row, a warp per head in turns, four consecutive values per lane (8-byte accesses); the rotate-half
// partner of a lane's values sits in lane ^ 16.
template <class W>
__global__ void __launch_bounds__(256)
qk_rope_store_d128_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out, SbBatch batch, SbKV kv,
                          int n_heads, int n_kv_heads, const W* __restrict__ q_norm_w, const W* __restrict__ k_norm_w,
                          float eps, const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                          int* status) {
    pdl_wait();
    pdl_launch_dependents();   // the attention that follows looks up its pages and fetches old keys meanwhile
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int width = (n_heads + 2 * n_kv_heads) * 128;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const int d0 = lane * 4, j0 = d0 & 63;
    __nv_bfloat162 c2[2], s2[2];
    {
        const uint2 craw = *reinterpret_cast<const uint2*>(cos_t + (long long)pos * 64 + j0);
        const uint2 sraw = *reinterpret_cast<const uint2*>(sin_t + (long long)pos * 64 + j0);
        c2[0] = reinterpret_cast<const __nv_bfloat162*>(&craw)[0];
        c2[1] = reinterpret_cast<const __nv_bfloat162*>(&craw)[1];
        s2[0] = reinterpret_cast<const __nv_bfloat162*>(&sraw)[0];
        s2[1] = reinterpret_cast<const __nv_bfloat162*>(&sraw)[1];
    }
    // A warp takes the heads warp, warp + 8, ...; it asks for the rows of up to QK_AHEAD of them (and the value rows that
    // go with key heads) before it works on the first: one 256-byte row in flight per warp left the memory idle (26 us
    // for 2,048 rows of the 4B shape, whose bytes need 8).
    constexpr int QK_AHEAD = 5;
    const int all_heads = n_heads + n_kv_heads;
    for (int first = warp; first < all_heads; first += 8 * QK_AHEAD) {
    uint2 raws[QK_AHEAD], vraws[QK_AHEAD];
#pragma unroll
    for (int u = 0; u < QK_AHEAD; ++u) {
        const int head = first + 8 * u;
        raws[u] = vraws[u] = make_uint2(0u, 0u);
        if (head < all_heads) {
            const __nv_bfloat16* src = qkv + (long long)row * width + (long long)head * 128;
            raws[u] = *reinterpret_cast<const uint2*>(src + d0);
            if (head >= n_heads) vraws[u] = *reinterpret_cast<const uint2*>(src + (long long)n_kv_heads * 128 + d0);
        }
    }
#pragma unroll
    for (int u = 0; u < QK_AHEAD; ++u) {
        const int head = first + 8 * u;
        if (head >= all_heads) break;
        const bool is_q = head < n_heads;
        const W* w = is_q ? q_norm_w : k_norm_w;
        const uint2 raw = raws[u];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        // The product of two bfloat16 numbers is exact in 32-bit, so a packed bfloat16 multiply (one rounding) gives
        // the bits of "multiply in 32-bit, then round"; likewise the packed add of two rounded products.  Only the
        // normalisation multiplies by a 32-bit factor and stays in 32-bit.
        __nv_bfloat162 y2[2] = {h2[0], h2[1]};
        if (w != nullptr) {
            const float2 v01 = __bfloat1622float2(h2[0]), v23 = __bfloat1622float2(h2[1]);
            float ss = v01.x * v01.x;
            ss = fmaf(v01.y, v01.y, ss); ss = fmaf(v23.x, v23.x, ss); ss = fmaf(v23.y, v23.y, ss);
            ss = warp_sum(ss);
            const float rstd = 1.0f / sqrtf(ss / 128.0f + eps);
            const __nv_bfloat162 n01 = __floats2bfloat162_rn(__fmul_rn(v01.x, rstd), __fmul_rn(v01.y, rstd));
            const __nv_bfloat162 n23 = __floats2bfloat162_rn(__fmul_rn(v23.x, rstd), __fmul_rn(v23.y, rstd));
            if (sizeof(W) == 2) {
                const uint2 wraw = *reinterpret_cast<const uint2*>(w + d0);
                const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
                y2[0] = __hmul2(w2[0], n01);
                y2[1] = __hmul2(w2[1], n23);
            } else {
                const float2 f01 = __bfloat1622float2(n01), f23 = __bfloat1622float2(n23);
                y2[0] = __floats2bfloat162_rn(__fmul_rn(to_f<W>(w[d0]), f01.x), __fmul_rn(to_f<W>(w[d0 + 1]), f01.y));
                y2[1] = __floats2bfloat162_rn(__fmul_rn(to_f<W>(w[d0 + 2]), f23.x), __fmul_rn(to_f<W>(w[d0 + 3]), f23.y));
            }
        }
        uint2 res;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            unsigned int partner = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const unsigned int*>(&y2[e]), 16);
            if (lane < 16) partner ^= 0x80008000u;          // the first half of a head meets minus its partner
            const __nv_bfloat162 a = __hmul2(y2[e], c2[e]);
            const __nv_bfloat162 b = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&partner), s2[e]);
            r2[e] = __hadd2(a, b);
        }
        __nv_bfloat16* dst;
        if (is_q) {
            dst = q_out + (long long)row * n_heads * 128 + (long long)head * 128;
        } else {
            const long long off = kv_offset(kv, slot, pos, head - n_heads);
            if (off < 0) {
                if (lane == 0) atomicOr(status, SB_STATUS_NO_PAGE);
                continue;
            }
            dst = (__nv_bfloat16*)kv.k + off;
            *reinterpret_cast<uint2*>((__nv_bfloat16*)kv.v + off + d0) = vraws[u];
        }
        *reinterpret_cast<uint2*>(dst + d0) = res;
    }
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
    // (few rows, as in decode: a warp per head over many small blocks spreads over more SMs and is faster)
    if (dtype == SB_BF16 && kv.head_dim == 128 && rotary_dim == 128 && cos_t != nullptr && batch.n_rows >= 256) {
        if (wdtype == SB_F32)
            sb_launch(qk_rope_store_d128_kernel<float>, batch.n_rows, 256, 0, stream, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out,
                      batch, kv, n_heads, n_kv_heads, (const float*)q_norm_w, (const float*)k_norm_w, eps,
                      (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, status);
        else
            sb_launch(qk_rope_store_d128_kernel<__nv_bfloat16>, batch.n_rows, 256, 0, stream, (const __nv_bfloat16*)qkv,
                      (__nv_bfloat16*)q_out, batch, kv, n_heads, n_kv_heads, (const __nv_bfloat16*)q_norm_w,
                      (const __nv_bfloat16*)k_norm_w, eps, (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, status);
        SB_LAUNCH_CHECK();
    }
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

SB_TIMELINE_SETTER(rope)
