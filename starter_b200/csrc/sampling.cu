// Token selection from 32-bit logits: greedy argmax and temperature / top-k sampling.
//
// Greedy follows the reference (engine/engine.py:204,207) with its tie rule: the lowest
// index among equal maxima (engine/kernels/topk.py:4-5,27,32-33).  The reference samples
// greedily only; the temperature / top-k draw is this library's own and is defined so that
// it is a pure function of the logits and one uniform number u:
//   kept set = the top_k largest logits (all if top_k <= 0), ties at the edge toward lower
//   indices; weight_i = exp((l_i - max) / T) over the kept set; the token is the first
//   index, in index order, whose running sum of weights exceeds u * total.
//   u = top 24 bits of a splitmix64 finaliser over (seed, request, step), times 2^-24.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned int ordered_key(float v) {
    const unsigned int b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // larger float <=> larger key
}

// Best (value, index) of a block; lowest index among equal values.  Result valid in thread 0.
__device__ __forceinline__ void block_best(float& bv, int& bi, float* best_v, int* best_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        bv = lane < n_warps ? best_v[lane] : -INFINITY;
        bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
    }
}

// Stage 1: grid (rows, chunks); each block finds the best of its slice of the row.
// Stage 2 (chunks == 1 or the second launch): one block per row over the stage-1 candidates.
__global__ void argmax_kernel(const float* __restrict__ values, const int* __restrict__ indices, int n, int row_stride,
                              float* __restrict__ out_v, int* __restrict__ out_i) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int chunks = gridDim.y;
    pdl_wait();
    const int per = (((n + chunks - 1) / chunks) + 3) & ~3;   // slices start at multiples of four values
    const int begin = min(n, (int)blockIdx.y * per), end = min(n, begin + per);
    const float* row = values + (long long)blockIdx.x * row_stride;
    const int* idx = indices ? indices + (long long)blockIdx.x * row_stride : nullptr;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (idx == nullptr && (row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(values) & 15) == 0) {
        // four values per load; a thread sees its indices in rising order, so ">" keeps the lowest index of equals
        const int end4 = begin + ((end - begin) & ~3);
        for (int i = begin + threadIdx.x * 4; i < end4; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            if (bi == 0x7fffffff || v.x > bv) { bv = v.x; bi = i; }
            if (v.y > bv) { bv = v.y; bi = i + 1; }
            if (v.z > bv) { bv = v.z; bi = i + 2; }
            if (v.w > bv) { bv = v.w; bi = i + 3; }
        }
        for (int i = end4 + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            if (bi == 0x7fffffff || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            const int id = idx ? idx[i] : i;
            if (bi == 0x7fffffff || v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
        }
    }
    block_best(bv, bi, best_v, best_i);
    if (threadIdx.x == 0) {
        if (out_v) out_v[blockIdx.x * chunks + blockIdx.y] = bv;
        out_i[blockIdx.x * chunks + blockIdx.y] = bi;
    }
}

__device__ __forceinline__ float uniform_from_counter(unsigned long long seed, unsigned long long request,
                                                      unsigned long long step) {
    unsigned long long z = seed * 0x9E3779B97F4A7C15ull + request * 0xBF58476D1CE4E5B9ull +
                           step * 0x94D049BB133111EBull + 0x2545F4914F6CDD1Dull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Exclusive prefix over the block's threads, in thread order; returns the thread's prefix and
// leaves the block total in *total.  T is float or int.
template <class V>
__device__ __forceinline__ V block_exclusive_scan(V v, V* warp_totals, V* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    V inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const V t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        V w = warp_totals[lane];
        V winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const V t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        warp_totals[lane] = winc - w;
        if (lane == 31) *total = winc;
    }
    __syncthreads();
    return warp_totals[warp] + inc - v;
}

// One block of SAMPLE_THREADS per row; thread t owns the indices [t*chunk, (t+1)*chunk).
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, float temperature, int top_k,
              unsigned long long seed, const int* __restrict__ request_ids, int* __restrict__ steps, int advance,
              const unsigned int* __restrict__ device_params) {
    __shared__ unsigned int hist[256];
    __shared__ float red[33];
    __shared__ float fw[32];
    __shared__ int iw[32];
    __shared__ float f_total;
    __shared__ int i_total;
    __shared__ unsigned int s_prefix;
    __shared__ int s_need;
    __shared__ int s_token;
    pdl_wait();
    if (device_params) {  // a captured step reads what the host wrote for this batch, not what was captured
        temperature = __uint_as_float(device_params[0]);
        top_k = (int)device_params[1];
        seed = (unsigned long long)device_params[2] | ((unsigned long long)device_params[3] << 32);
    }
    const float* row = logits + (long long)blockIdx.x * vocab;
    const int tid = threadIdx.x;
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);

    // The k-th largest logit by radix select over order-preserving keys, 8 bits a pass.
    unsigned int threshold = 0;  // keys >= threshold are candidates; 0 keeps everything
    int ties_kept = 0x7fffffff;  // how many keys equal to the threshold are kept (lowest indices)
    if (top_k > 0 && top_k < vocab) {
        if (tid == 0) { s_prefix = 0; s_need = top_k; }
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            const unsigned int prefix = s_prefix;
            const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = begin; i < end; ++i) {
                const unsigned int key = ordered_key(row[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                int need = s_need, b = 255;
                for (; b > 0; --b) {
                    if ((int)hist[b] >= need) break;
                    need -= (int)hist[b];
                }
                s_prefix = prefix | ((unsigned int)b << shift);
                s_need = need;
            }
            __syncthreads();
        }
        threshold = s_prefix;
        ties_kept = s_need;
    }
    // Rank of each key equal to the threshold, in index order, to keep the lowest indices.
    int my_ties = 0;
    if (threshold != 0)
        for (int i = begin; i < end; ++i) my_ties += ordered_key(row[i]) == threshold;
    int ties_before = 0;
    if (threshold != 0) ties_before = block_exclusive_scan<int>(my_ties, iw, &i_total);

    // Maximum of the kept logits (the maximum of all logits is always kept).
    float mx = -INFINITY;
    for (int i = begin; i < end; ++i) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float t = red[tid];
        t = warp_max(t);
        if (tid == 0) red[32] = t;
    }
    __syncthreads();
    mx = red[32];

    const float inv_t = 1.0f / temperature;
    float mine = 0.f;
    int seen = ties_before;
    for (int i = begin; i < end; ++i) {
        const float v = row[i];
        const unsigned int key = ordered_key(v);
        bool keep = key > threshold || threshold == 0;
        if (threshold != 0 && key == threshold) keep = seen++ < ties_kept;
        if (keep) mine += expf((v - mx) * inv_t);
    }
    const float before = block_exclusive_scan<float>(mine, fw, &f_total);
    const float total = f_total;
    const int request = request_ids ? request_ids[blockIdx.x] : blockIdx.x;
    const int step = steps ? steps[blockIdx.x] : 0;
    const float target = uniform_from_counter(seed, (unsigned long long)request, (unsigned long long)step) * total;
    // The owner of the crossing is the last thread (in index order) with kept weight whose
    // prefix does not exceed the target; it walks its own indices to the first one whose
    // running sum exceeds the target, or to its last kept index if rounding hides the crossing.
    if (tid == 0) s_token = -1;
    __syncthreads();
    if (mine > 0.f && before <= target) atomicMax(&s_token, tid);
    __syncthreads();
    const int owner = s_token < 0 ? 0 : s_token;
    __syncthreads();
    if (tid == owner) {
        float running = before;
        int tok = -1;
        seen = ties_before;
        for (int i = begin; i < end; ++i) {
            const float v = row[i];
            const unsigned int key = ordered_key(v);
            bool keep = key > threshold || threshold == 0;
            if (threshold != 0 && key == threshold) keep = seen++ < ties_kept;
            if (!keep) continue;
            running += expf((v - mx) * inv_t);
            tok = i;
            if (running > target) break;
        }
        s_token = tok;
    }
    __syncthreads();
    if (tid == 0) {
        out[blockIdx.x] = s_token;
        if (steps && advance) steps[blockIdx.x] = step + 1;
    }
}

extern "C" {

// scratch_v, scratch_i: rows * SB_ARGMAX_CHUNKS entries each, for the candidates of stage 1.
int sb_argmax(const float* logits, int* out, int rows, int vocab, float* scratch_v, int* scratch_i, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int chunks = vocab >= 16384 ? 32 : 1;
    if (chunks == 1) {
        sb_launch(argmax_kernel, dim3(rows, 1), 1024, 0, stream, logits, nullptr, vocab, vocab, nullptr, out);
    } else {
        sb_launch(argmax_kernel, dim3(rows, chunks), 512, 0, stream, logits, nullptr, vocab, vocab, scratch_v, scratch_i);
        sb_launch(argmax_kernel, dim3(rows, 1), 32, 0, stream, scratch_v, scratch_i, chunks, chunks, nullptr, out);
    }
    SB_LAUNCH_CHECK();
}

// request_ids [rows] and steps [rows] key the uniform number of each row; with advance != 0 the
// kernel adds one to each row's step after use, so a replayed step draws a fresh number.
// device_params (or null): four 32-bit words on the device {temperature's float bits, top_k, seed low,
// seed high} that replace the three arguments of the same names when the kernel runs.
int sb_sample(const float* logits, int* out, int rows, int vocab, float temperature, int top_k, unsigned long long seed,
              const int* request_ids, int* steps, int advance, const unsigned int* device_params, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (!device_params && !(temperature > 0.f)) return (int)cudaErrorInvalidValue;
    sb_launch(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, out, vocab, temperature, top_k, seed, request_ids, steps,
              advance, device_params);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
