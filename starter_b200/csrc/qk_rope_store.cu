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


// The common case on the tensor-core path: bfloat16, head size 128, rotary over the whole head.  A block takes rows in
// turn (four blocks per SM at most); half a warp per head (eight consecutive values = 16 bytes per lane, the rotate-half partner of a lane's values in
// lane ^ 8), so a warp works on two heads at once and on the heads 16 further in turns.  A warp asks for the rows
// of all the heads of a turn (and the value rows that go with key heads) before it works on the first: one row in
// flight per warp left the memory idle (26 us for 2,048 rows of the 4B shape, whose bytes need 8).
// The product of two bfloat16 numbers is exact in 32-bit, so a packed bfloat16 multiply (one rounding) gives the
// bits of "multiply in 32-bit, then round", and likewise the packed add of two rounded products; only the
// normalisation multiplies by a 32-bit factor and stays in 32-bit.  The _rn forms matter: the plain ones may be
// contracted into one fused multiply-add, which drops the rounding of the first product (a fifth of the values then
// differ from the formula by one step).
template <class W>
__global__ void __launch_bounds__(256)
qk_rope_store_d128_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out, SbBatch batch, SbKV kv,
                          int n_heads, int n_kv_heads, const W* __restrict__ q_norm_w, const W* __restrict__ k_norm_w,
                          float eps, const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                          int* status) {
    pdl_wait();
    pdl_launch_dependents();   // the attention that follows looks up its pages and fetches old keys meanwhile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, hl = lane & 15;
    const int width = (n_heads + 2 * n_kv_heads) * 128;
    for (int row = blockIdx.x; row < batch.n_rows; row += gridDim.x) {   // a block takes several rows in turn
    int slot = 0, pos = 0;
    const int d0 = hl * 8, j0 = d0 & 63;
    uint4 craw, sraw;
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&craw);
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&sraw);
    constexpr int QK_AHEAD = 3;
    const int all_heads = n_heads + n_kv_heads;
    for (int base = 2 * warp; base < all_heads; base += 16 * QK_AHEAD) {
        uint4 raws[QK_AHEAD], vraws[QK_AHEAD];
#pragma unroll
        for (int u = 0; u < QK_AHEAD; ++u) {
            const int head = base + half + 16 * u;
            raws[u] = vraws[u] = make_uint4(0u, 0u, 0u, 0u);
            if (head < all_heads) {
                const __nv_bfloat16* src = qkv + (long long)row * width + (long long)head * 128;
                raws[u] = *reinterpret_cast<const uint4*>(src + d0);
                if (head >= n_heads) vraws[u] = *reinterpret_cast<const uint4*>(src + (long long)n_kv_heads * 128 + d0);
            }
        }
        if (base == 2 * warp) {
            // Where the row stands (three look-ups, each waiting for the one before) and its table entries are asked
            // for after the row itself, which depends on none of them.
            row_place(batch, row, slot, pos);
            craw = *reinterpret_cast<const uint4*>(cos_t + (long long)pos * 64 + j0);
            sraw = *reinterpret_cast<const uint4*>(sin_t + (long long)pos * 64 + j0);
        }
#pragma unroll
        for (int u = 0; u < QK_AHEAD; ++u) {
            const int head = base + half + 16 * u;
            if (base + 16 * u >= all_heads) break;          // the same for both halves of the warp
            const bool active = head < all_heads, is_q = head < n_heads;
            const W* w = is_q ? q_norm_w : k_norm_w;
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raws[u]);
            __nv_bfloat162 y2[4] = {h2[0], h2[1], h2[2], h2[3]};
            float f[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 v = __bfloat1622float2(h2[e]);
                f[2 * e] = v.x;
                f[2 * e + 1] = v.y;
            }
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // over the 16 lanes of the head
            if (w != nullptr) {
                const float rstd = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 n = __floats2bfloat162_rn(__fmul_rn(f[2 * e], rstd), __fmul_rn(f[2 * e + 1], rstd));
                    if (sizeof(W) == 2) {
                        y2[e] = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(w + d0 + 2 * e), n);
                    } else {
                        const float2 nf = __bfloat1622float2(n);
                        y2[e] = __floats2bfloat162_rn(__fmul_rn(to_f<W>(w[d0 + 2 * e]), nf.x), __fmul_rn(to_f<W>(w[d0 + 2 * e + 1]), nf.y));
                    }
                }
            }
            uint4 res;
            __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                unsigned int partner = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const unsigned int*>(&y2[e]), 8);
                if (hl < 8) partner ^= 0x80008000u;          // the first half of a head meets minus its partner
                const __nv_bfloat162 a = __hmul2_rn(y2[e], c2[e]);
                const __nv_bfloat162 b = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&partner), s2[e]);
                r2[e] = __hadd2_rn(a, b);
            }
            if (!active) continue;
            __nv_bfloat16* dst;
            if (is_q) {
                dst = q_out + (long long)row * n_heads * 128 + (long long)head * 128;
            } else {
                const long long off = kv_offset(kv, slot, pos, head - n_heads);
                if (off < 0) {
                    if (hl == 0) atomicOr(status, SB_STATUS_NO_PAGE);
                    continue;
                }
                dst = (__nv_bfloat16*)kv.k + off;
                *reinterpret_cast<uint4*>((__nv_bfloat16*)kv.v + off + d0) = vraws[u];
            }
            *reinterpret_cast<uint4*>(dst + d0) = res;
        }
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
        const int d128_blocks = batch.n_rows < 148 * 4 ? batch.n_rows : 148 * 4;
        if (wdtype == SB_F32)
            sb_launch(qk_rope_store_d128_kernel<float>, d128_blocks, 256, 0, stream, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out,
                      batch, kv, n_heads, n_kv_heads, (const float*)q_norm_w, (const float*)k_norm_w, eps,
                      (const __nv_bfloat16*)cos_t, (const __nv_bfloat16*)sin_t, status);
        else
            sb_launch(qk_rope_store_d128_kernel<__nv_bfloat16>, d128_blocks, 256, 0, stream, (const __nv_bfloat16*)qkv,
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
