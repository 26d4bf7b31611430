// General matrix product C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, any M, N, K.
//
// This is the true 32-bit product of the float32 path (no tensor-core, no reduced-precision
// mode) and the fallback of the bfloat16 path for shapes the tensor-core kernels refuse.
// Each output element is one running sum over k = 0..K-1 in order, so a row's result does
// not depend on how many other rows the call has.  The reference's products are
// `x @ W.T` with W as [out, in] (engine/model.py:291,295,297,299).
#include "common.cuh"

#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <class TA, class TO>
__global__ void __launch_bounds__(256) gemm_general_kernel(const TA* __restrict__ A, const TA* __restrict__ W,
                                                           TO* __restrict__ C, int M, int N, int K) {
    __shared__ float As[GG_BK][GG_BM + 4];
    __shared__ float Ws[GG_BK][GG_BN + 4];
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
    const int tx = tid % 16, ty = tid / 16;  // thread computes rows ty*4.., cols tx*4..
    const int lr = tid / 4, lk = (tid % 4) * 4;  // loader: row lr, k offset lk..lk+3
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GG_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + e][lr] = (am < M && k < K) ? to_f<TA>(A[(long long)am * K + k]) : 0.f;
            Ws[lk + e][lr] = (wn < N && k < K) ? to_f<TA>(W[(long long)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GG_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(long long)m * N + n] = from_f<TO>(acc[i][j]);
        }
    }
}

extern "C" int sb_gemm_general(int dtype, int out_f32, const void* A, const void* W, void* C, int M, int N, int K,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GG_BN - 1) / GG_BN, (M + GG_BM - 1) / GG_BM);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (dtype == SB_F32)
        sb_launch(gemm_general_kernel<float, float>, grid, 256, 0, stream, (const float*)A, (const float*)W, (float*)C, M, N, K);
    else if (out_f32)
        sb_launch(gemm_general_kernel<__nv_bfloat16, float>, grid, 256, 0, stream, (const __nv_bfloat16*)A, (const __nv_bfloat16*)W,
                                                                           (float*)C, M, N, K);
    else
        sb_launch(gemm_general_kernel<__nv_bfloat16, __nv_bfloat16>, grid, 256, 0, stream, 
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, (__nv_bfloat16*)C, M, N, K);
    SB_LAUNCH_CHECK();
}
