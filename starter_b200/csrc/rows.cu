// Row-wise kernels: embedding gather, row gather, RMSNorm with and without the residual
// add, SwiGLU, and the end-of-step length update.  T is the activation type (float or
// bfloat16), W the norm weight's type (a weight stored in 32-bit stays 32-bit).
//
// Formulas of the reference: engine/kernels/rmsnorm.py:31-45 (norm: 32-bit mean of squares,
// the normalised value rounded to T before the weight multiply),
// engine/kernels/add_rmsnorm.py:21-29 (sum rounded to T, stored, then normed),
// engine/kernels/swiglu.py:21-24 (silu in 32-bit, rounded, times up, rounded).
#include "common.cuh"

template <class T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                             int hidden, int vocab, int* status) {
    pdl_wait();
    pdl_launch_dependents();   // a small kernel: its successor may fetch its weights meanwhile
    const int row = blockIdx.x;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const T* src = table + (long long)tok * hidden;
    T* dst = out + (long long)row * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = src[c];
}

template <class T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ rows, T* __restrict__ out, int width) {
    pdl_wait();
    pdl_launch_dependents();
    const T* src = x + (long long)rows[blockIdx.x] * width;
    T* dst = out + (long long)blockIdx.x * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

// One block per row.  ADD: x <- T(x + delta) first.
template <class T, class W, bool ADD>
__global__ void rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const W* __restrict__ weight,
                               T* __restrict__ out, int width, float eps) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();   // the product that follows fetches its first weights while the rows are normed
    T* xr = x + (long long)blockIdx.x * width;
    const T* dr = ADD ? delta + (long long)blockIdx.x * width : nullptr;
    T* yr = out + (long long)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = to_f<T>(xr[c]);
        if (ADD) {
            v = rnd<T>(__fadd_rn(v, to_f<T>(dr[c])));
            xr[c] = from_f<T>(v);
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float n = rnd<T>(__fmul_rn(to_f<T>(xr[c]), rstd));
        yr[c] = from_f<T>(__fmul_rn(n, to_f<W>(weight[c])));
    }
}

// bfloat16 rows whose width is a multiple of 8 and at most 8192: every thread holds eight
// consecutive values, so the row is read once and the whole norm is one pass.
template <class W, bool ADD>
__global__ void rmsnorm_vec_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                   const W* __restrict__ weight, __nv_bfloat16* __restrict__ out, int width, float eps) {
    __shared__ float red[33];
    sb_stamp(1, 0);
    const long long base = (long long)blockIdx.x * width;
    const int c = threadIdx.x * 8;
    const bool active = c < width;
    float wv[8];   // the norm's weights do not depend on the kernel before this one: asked for before the wait
#pragma unroll
    for (int e = 0; e < 8; ++e) wv[e] = active ? to_f<W>(weight[c + e]) : 0.f;
    pdl_wait();
    pdl_launch_dependents();
    sb_stamp(1, 1);
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + base + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            v[2 * e] = f.x;
            v[2 * e + 1] = f.y;
        }
        if (ADD) {
            const uint4 draw = *reinterpret_cast<const uint4*>(delta + base + c);
            const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&draw);
            uint4 sum;
            __nv_bfloat162* sh = reinterpret_cast<__nv_bfloat162*>(&sum);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(dh[e]);
                sh[e] = __floats2bfloat162_rn(__fadd_rn(v[2 * e], f.x), __fadd_rn(v[2 * e + 1], f.y));
                const float2 back = __bfloat1622float2(sh[e]);
                v[2 * e] = back.x;
                v[2 * e + 1] = back.y;
            }
            *reinterpret_cast<uint4*>(x + base + c) = sum;
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
    ss = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
    if (active) {
        uint4 res;
        __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float n0 = rnd<__nv_bfloat16>(__fmul_rn(v[2 * e], rstd)), n1 = rnd<__nv_bfloat16>(__fmul_rn(v[2 * e + 1], rstd));
            rh[e] = __floats2bfloat162_rn(__fmul_rn(n0, wv[2 * e]), __fmul_rn(n1, wv[2 * e + 1]));
        }
        *reinterpret_cast<uint4*>(out + base + c) = res;
    }
    sb_stamp(1, 2);
}

// Many rows (prefill): a warp per row, the whole row in the lanes' registers as packed bfloat16 (NV vectors of
// eight values per lane), no block-wide barrier.  A block per row with one 16-byte load per thread and two barriers
// kept too few bytes in flight: 12 us for 2,048 rows of 2,560 where the bytes need 6.5.
template <class W, bool ADD, int NV>
__global__ void __launch_bounds__(128)
rmsnorm_warp_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta, const W* __restrict__ weight,
                    __nv_bfloat16* __restrict__ out, int rows, int width, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const long long base = (long long)row * width;
    const int nvec = width >> 3;
    uint4 vals[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        vals[i] = idx < nvec ? *reinterpret_cast<const uint4*>(x + base + idx * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (ADD) {
        uint4 ds[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            ds[i] = idx < nvec ? *reinterpret_cast<const uint4*>(delta + base + idx * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            __nv_bfloat162* vh = reinterpret_cast<__nv_bfloat162*>(&vals[i]);
            const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&ds[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(vh[e]), b = __bfloat1622float2(dh[e]);
                vh[e] = __floats2bfloat162_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));   // the sum is rounded, then normed
            }
            const int idx = lane + 32 * i;
            if (idx < nvec) *reinterpret_cast<uint4*>(x + base + idx * 8) = vals[i];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vals[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = __bfloat1622float2(vh[e]);
            ss = fmaf(a.x, a.x, ss);
            ss = fmaf(a.y, a.y, ss);
        }
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + 32 * i;
        if (idx >= nvec) continue;
        float wv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) wv[e] = to_f<W>(weight[idx * 8 + e]);
        const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vals[i]);
        uint4 res;
        __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = __bfloat1622float2(vh[e]);
            const float n0 = rnd<__nv_bfloat16>(__fmul_rn(a.x, rstd)), n1 = rnd<__nv_bfloat16>(__fmul_rn(a.y, rstd));
            rh[e] = __floats2bfloat162_rn(__fmul_rn(n0, wv[2 * e]), __fmul_rn(n1, wv[2 * e + 1]));
        }
        *reinterpret_cast<uint4*>(out + base + idx * 8) = res;
    }
}

template <class T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
    pdl_wait();
    const long long row = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const float g = to_f<T>(gu[row * 2 * inter + c]);
    const float u = to_f<T>(gu[row * 2 * inter + inter + c]);
    const float s = rnd<T>(g / (1.0f + expf(-g)));
    out[row * inter + c] = from_f<T>(__fmul_rn(s, u));
}

// bfloat16 rows whose half-width is a multiple of 8: eight values per thread, 16-byte accesses.
__global__ void swiglu_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter, long long total8) {
    pdl_wait();
    const int per_row = inter / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / per_row;
        const int c = (int)(i % per_row) * 8;
        const uint4 graw = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + c);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + c);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 res;
        __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(gh[e]), u = __bfloat1622float2(uh[e]);
            // 2^x and the division by the fast units: their error (2^-21) is far below the bfloat16 rounding that follows
            const float s0 = rnd<__nv_bfloat16>(__fdividef(g.x, 1.0f + __expf(-g.x))), s1 = rnd<__nv_bfloat16>(__fdividef(g.y, 1.0f + __expf(-g.y)));
            rh[e] = __floats2bfloat162_rn(__fmul_rn(s0, u.x), __fmul_rn(s1, u.y));
        }
        *reinterpret_cast<uint4*>(out + row * inter + c) = res;
    }
}

__global__ void advance_lengths_kernel(SbBatch b, int* lengths) {
    pdl_wait();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= b.n_seqs) return;
    const int slot = b.seq_slot[s];
    if (slot != b.null_slot) lengths[slot] += b.cu_q[s + 1] - b.cu_q[s];
}

static inline int row_threads(int width) {
    int t = 32;
    while (t < 256 && t * 4 < width) t <<= 1;
    return t;
}

int sb_pdl_flag = 0;

extern "C" {

// 1: launch every kernel of this library with programmatic dependent launch; 0: plain stream order.
void sb_set_pdl(int on) { sb_pdl_flag = on ? 1 : 0; }

int sb_embed(int dtype, const int* tokens, const void* table, void* out, int rows, int hidden, int vocab, int* status,
             cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == SB_F32)
        sb_launch(embed_kernel<float>, rows, row_threads(hidden), 0, stream, tokens, (const float*)table, (float*)out, hidden, vocab, status);
    else
        sb_launch(embed_kernel<__nv_bfloat16>, rows, row_threads(hidden), 0, stream, tokens, (const __nv_bfloat16*)table,
                                                                                (__nv_bfloat16*)out, hidden, vocab, status);
    SB_LAUNCH_CHECK();
}

int sb_gather_rows(int dtype, const void* x, const int* rows, void* out, int n_rows, int width, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == SB_F32)
        sb_launch(gather_rows_kernel<float>, n_rows, row_threads(width), 0, stream, (const float*)x, rows, (float*)out, width);
    else
        sb_launch(gather_rows_kernel<__nv_bfloat16>, n_rows, row_threads(width), 0, stream, (const __nv_bfloat16*)x, rows,
                                                                                      (__nv_bfloat16*)out, width);
    SB_LAUNCH_CHECK();
}

// x [rows, width] (updated in place when delta is given), weight [width] of dtype wdtype, out [rows, width].
int sb_rmsnorm(int dtype, int wdtype, void* x, const void* delta, const void* weight, void* out, int rows, int width,
               float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int th = row_threads(width);
#define SB_NORM(T, W)                                                                                             \
    do {                                                                                                          \
        if (delta)                                                                                                \
            sb_launch(rmsnorm_kernel<T, W, true>, rows, th, 0, stream, (T*)x, (const T*)delta, (const W*)weight, (T*)out, width, eps); \
        else                                                                                                      \
            sb_launch(rmsnorm_kernel<T, W, false>, rows, th, 0, stream, (T*)x, nullptr, (const W*)weight, (T*)out, width, eps);        \
    } while (0)
    if (dtype == SB_F32) {
        if (wdtype != SB_F32) return (int)cudaErrorInvalidValue;
        SB_NORM(float, float);
    } else if ((width & 7) == 0 && width <= 8192) {
        if (rows >= 128 && width <= 8 * 32 * 16) {   // many rows: a warp per row
            const int nv = (width / 8 + 31) / 32;
            const int blocks = (rows + 3) / 4;
#define SB_WNORM2(W, ADD, NV)                                                                                         \
    sb_launch(rmsnorm_warp_kernel<W, ADD, NV>, blocks, 128, 0, stream, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta,           \
              (const W*)weight, (__nv_bfloat16*)out, rows, width, eps)
#define SB_WNORM1(W, ADD)                                                                                             \
    do {                                                                                                             \
        if (nv <= 4) SB_WNORM2(W, ADD, 4); else if (nv <= 8) SB_WNORM2(W, ADD, 8);                                   \
        else if (nv <= 12) SB_WNORM2(W, ADD, 12); else SB_WNORM2(W, ADD, 16);                                        \
    } while (0)
            if (wdtype == SB_F32) { if (delta) SB_WNORM1(float, true); else SB_WNORM1(float, false); }
            else { if (delta) SB_WNORM1(__nv_bfloat16, true); else SB_WNORM1(__nv_bfloat16, false); }
#undef SB_WNORM1
#undef SB_WNORM2
            SB_LAUNCH_CHECK();
        }
        const int vt = ((width / 8 + 31) / 32) * 32;
#define SB_VNORM(W)                                                                                                  \
    do {                                                                                                             \
        if (delta)                                                                                                   \
            sb_launch(rmsnorm_vec_kernel<W, true>, rows, vt, 0, stream, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta,      \
                                                                  (const W*)weight, (__nv_bfloat16*)out, width, eps); \
        else                                                                                                         \
            sb_launch(rmsnorm_vec_kernel<W, false>, rows, vt, 0, stream, (__nv_bfloat16*)x, nullptr, (const W*)weight,       \
                                                                   (__nv_bfloat16*)out, width, eps);                 \
    } while (0)
        if (wdtype == SB_F32) SB_VNORM(float); else SB_VNORM(__nv_bfloat16);
#undef SB_VNORM
    } else if (wdtype == SB_F32) {
        SB_NORM(__nv_bfloat16, float);
    } else {
        SB_NORM(__nv_bfloat16, __nv_bfloat16);
    }
#undef SB_NORM
    SB_LAUNCH_CHECK();
}

int sb_swiglu(int dtype, const void* gu, void* out, int rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == SB_BF16 && (inter & 7) == 0) {
        const long long total8 = (long long)rows * (inter / 8);
        const int blocks = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        sb_launch(swiglu_vec_kernel, blocks, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, total8);
        SB_LAUNCH_CHECK();
    }
    dim3 grid(rows, (inter + 255) / 256);
    if (dtype == SB_F32)
        sb_launch(swiglu_kernel<float>, grid, 256, 0, stream, (const float*)gu, (float*)out, inter);
    else
        sb_launch(swiglu_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter);
    SB_LAUNCH_CHECK();
}

int sb_advance_lengths(SbBatch b, int* lengths, cudaStream_t stream) {
    if (b.n_seqs <= 0) return 0;
    sb_launch(advance_lengths_kernel, (b.n_seqs + 127) / 128, 128, 0, stream, b, lengths);
    SB_LAUNCH_CHECK();
}

const char* sb_error_string(int code) { return cudaGetErrorString((cudaError_t)code); }

}  // extern "C"

SB_TIMELINE_SETTER(rows)
