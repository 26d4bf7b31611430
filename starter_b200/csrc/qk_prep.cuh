// The preparation of a decode step's queries and new key inside an attention kernel: per-head RMSNorm of q and k
// (engine/kernels/rope.py:19-25), the rotary encoding with its three roundings (:26-30), the queries of one kv head's
// group laid out as the 16-row tile the tensor core reads, and the new key and value written into the paged cache
// (:86-91).  The reference runs this as a kernel of its own between the projection and the attention
// (engine/model.py:202-205); inside the attention kernel it costs no launch and no trip of q through memory.
#pragma once

#include "common.cuh"
#include "mma_utils.cuh"

// What the fused preparation needs besides the cache.  qkv [rows, (n_heads + 2 * n_kv_heads) * D], or
// [rows, n_heads * D] when store_kv is 0 (a layer that reads another layer's cache); norm weights
// bfloat16 or float (norm_f32), null = no per-head norm; cos/sin [positions, D / 2] bfloat16, null = no
// rotary encoding (otherwise over the whole head).
struct SbFusedQK {
    const __nv_bfloat16* qkv;
    const void* q_norm;
    const void* k_norm;
    const __nv_bfloat16* cos_t;
    const __nv_bfloat16* sin_t;
    int* status;
    float eps;
    int norm_f32;
    int store_kv;
    int reserved;
    const void* next_w;        // a matrix (16-byte aligned) that the kernel after this one streams: asked into L2 when
    long long next_bytes;      // this kernel's keys are read, so that memory stays busy through its merge; or null
};

__device__ __forceinline__ void unpack4(const uint2 raw, float (&v)[4]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

__device__ __forceinline__ void load_norm4(const void* w, int norm_f32, int d0, float (&v)[4]) {
    if (norm_f32) {
        const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + d0);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
        unpack4(*reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(w) + d0), v);
    }
}

// The G query heads of (row, kv head) into rows 0..G-1 of the tile q_s ([16][D] bfloat16, tile_off layout; rows beyond
// G are zeroed), each by one warp in turn; with owns_new one more job norms and rotates the new key head and stores
// it and its value at element offset new_off of the cache (new_off < 0: no page there, flagged in the status word).
// Called by all WARPS * 32 threads of the block; the caller puts a block-wide barrier after it.
template <int D, int WARPS>
__device__ __forceinline__ void prepare_group(const SbFusedQK& fused, const SbKV& kv, unsigned char* q_s, int row, int kvh,
                                              int n_heads, int G, int pos, bool owns_new, long long new_off) {
    constexpr int CH = D / 8;
    constexpr int LANES = D / 4;                           // lanes that hold a head, four values each
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int d0 = lane * 4;
    const bool holds = lane < LANES;
    float rc[4] = {1.f, 1.f, 1.f, 1.f}, rs[4] = {0.f, 0.f, 0.f, 0.f}, wq[4] = {1.f, 1.f, 1.f, 1.f};
    if (holds) {
        if (fused.cos_t != nullptr) {
            const int j0 = d0 % (D / 2);
            unpack4(*reinterpret_cast<const uint2*>(fused.cos_t + (long long)pos * (D / 2) + j0), rc);
            unpack4(*reinterpret_cast<const uint2*>(fused.sin_t + (long long)pos * (D / 2) + j0), rs);
        }
        if (fused.q_norm != nullptr) load_norm4(fused.q_norm, fused.norm_f32, d0, wq);
    }
    for (int i = tid; i < 16 * CH; i += WARPS * 32) {
        const int r = i / CH, c = i % CH;
        if (r >= G) *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = make_uint4(0u, 0u, 0u, 0u);
    }
    const int width = (n_heads + (fused.store_kv ? 2 * kv.n_kv_heads : 0)) * D;
    const __nv_bfloat16* qkv_row = fused.qkv + (long long)row * width;
    const int n_jobs = G + (owns_new ? 1 : 0);          // job G: the key head (and the value's copy)
    for (int job = warp; job < n_jobs; job += WARPS) {
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
}
