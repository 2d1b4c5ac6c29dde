// Token choice from float32 logits [rows, vocab]: greedy, or temperature sampling with
// optional top-k / top-p, one thread block per row.
//
// Greedy: the largest logit; of equal logits the lowest index wins
// (src/backend/ops/argmax/cpu/argmax_cpu.cpp:15-19).
//
// Sampling, following src/frontend/sampler/sampler.cpp:195-265 and :410-490 in meaning:
//   z_i = logit_i / temperature;  w_i = exp(z_i - max z);  S = sum w
//   top-k keeps the k largest w (entries equal to the k-th largest are all kept);
//   top-p then keeps the smallest set of largest entries whose mass reaches top_p * S,
//     mass counted on the un-renormalised w, among the entries top-k kept;
//   the kept entries are renormalised and the token is the first index i, in index order,
//     whose running sum exceeds u * (kept mass), u in [0, 1) given by the caller.
// The reference's CPU sampler walks the kept set in order of probability instead of index;
// the distribution is the same.  All sums run in a fixed order (per-thread contiguous chunks,
// then a fixed tree), so a row's result does not depend on the other rows.
#define ZI_PDL_BIT 8
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(sampling)

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned int order_key(float v) {
    // monotone map float -> uint32 (larger float -> larger key); NaN is treated as the smallest
    if (v != v) return 0u;
    unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgPair { float v; int i; };

__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgPair block_argmax(const float* __restrict__ row, int vocab, ArgPair* scratch) {
    ArgPair best; best.v = -INFINITY; best.i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = ld_dep(row + i);
        if (v != v) v = -INFINITY;
        ArgPair c; c.v = v; c.i = i;
        best = better(best, c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair c;
        c.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        c.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, c);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    ArgPair r; r.v = -INFINITY; r.i = 0x7fffffff;
    if (lane < nwarps) r = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair c;
        c.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        c.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, c);
    }
    if (r.i == 0x7fffffff) r.i = 0;       // a row of NaN / -inf only
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, long long row_stride) {
    __shared__ ArgPair scratch[32];
    pdl_trigger_early();
    pdl_wait();
    pdl_trigger_late();
    const ArgPair r = block_argmax(logits + (size_t)blockIdx.x * row_stride, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

ZI_EXPORT int zi_argmax(const float* logits, int* out, int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return zi_fail("argmax: vocab=%d must be positive", vocab);
    zi_launch(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, out, vocab, row_stride);
    return zi_check_launch("argmax");
}

// CTRL-style repetition penalty on the listed tokens of one row, in place:
// l > 0 ? l / penalty : l * penalty (src/frontend/sampler/sampler.cpp:439-451).  A token that
// is listed several times is penalised once per listing, as in the reference's loop.
__global__ void repetition_penalty_kernel(float* __restrict__ row, const int* __restrict__ tokens, int n, int vocab,
                                          float penalty) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        for (int t = 0; t < n; ++t) {
            const int id = tokens[t];
            if (id < 0 || id >= vocab) continue;
            const float l = row[id];
            row[id] = l > 0.0f ? l / penalty : l * penalty;
        }
    }
}

ZI_EXPORT int zi_repetition_penalty(float* row, const int* tokens, int n, int vocab, float penalty, cudaStream_t stream) {
    if (n <= 0 || penalty == 1.0f) return 0;
    if (!(penalty > 0.0f)) return zi_fail("repetition_penalty=%f must be positive", penalty);
    repetition_penalty_kernel<<<1, 32, 0, stream>>>(row, tokens, n, vocab, penalty);
    return zi_check_launch("repetition_penalty");
}

// Sum over the block of a per-thread double-free float pair (count, mass) in a fixed order.
__device__ __forceinline__ float2 block_sum2(float2 v, float2* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
        v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float2 r = (lane < nwarps) ? scratch[lane] : make_float2(0.0f, 0.0f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        r.x += __shfl_xor_sync(0xffffffffu, r.x, o);
        r.y += __shfl_xor_sync(0xffffffffu, r.y, o);
    }
    return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int vocab, long long row_stride) {
    __shared__ ArgPair ascratch[32];
    __shared__ float fscratch[32];
    __shared__ float2 pscratch[32];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature[r];
    const ArgPair top = block_argmax(row, vocab, ascratch);
    if (!(temp > 0.0f)) {                      // greedy row
        if (threadIdx.x == 0) out[r] = top.i;
        return;
    }
    const float zmax = top.v / temp;
    // contiguous chunk of this thread
    const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = threadIdx.x * per < vocab ? threadIdx.x * per : vocab;
    const int end = begin + per < vocab ? begin + per : vocab;

    // total mass S
    float s = 0.0f;
    for (int i = begin; i < end; ++i) {
        float v = row[i];
        if (v == v) s += expf(v / temp - zmax);
    }
    const float S = block_sum(s, fscratch);

    // threshold key: entries with order_key(z) >= thr are kept
    unsigned int thr = 0u;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        unsigned int t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = t | (1u << bit);
            float cnt = 0.0f;
            for (int i = begin; i < end; ++i) cnt += (order_key(row[i] / temp) >= cand) ? 1.0f : 0.0f;
            const float2 tot = block_sum2(make_float2(cnt, 0.0f), pscratch);
            if (tot.x >= (float)k) t = cand;
        }
        thr = t;
    }
    const float p = top_p[r];
    if (p < 1.0f) {
        // largest key t with mass{key >= max(t, thr)} >= p * S; if even the whole top-k set has less, keep it all
        const float need = p * S;
        unsigned int t = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned int cand = t | (1u << bit);
            const unsigned int eff = cand > thr ? cand : thr;
            float mass = 0.0f;
            for (int i = begin; i < end; ++i) {
                const float z = row[i] / temp;
                if (z == z && order_key(z) >= eff) mass += expf(z - zmax);
            }
            const float2 tot = block_sum2(make_float2(0.0f, mass), pscratch);
            if (tot.y >= need) t = cand;
        }
        if (t > thr) thr = t;
    }

    // kept mass per chunk, then the chunk that holds the target, then the entry
    float mine = 0.0f;
    for (int i = begin; i < end; ++i) {
        const float z = row[i] / temp;
        if (z == z && order_key(z) >= thr) mine += expf(z - zmax);
    }
    chunk_sum[threadIdx.x] = mine;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        // sequential scan over 1024 chunk sums: fixed order, a few microseconds
        float total = 0.0f;
        for (int t = 0; t < SAMPLE_THREADS; ++t) total += chunk_sum[t];
        const float target = uniform[r] * total;
        float run = 0.0f;
        int owner = -1;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            if (chunk_sum[t] > 0.0f) {
                if (target < run + chunk_sum[t]) { owner = t; break; }
                run += chunk_sum[t];
            }
        }
        int pick = -1;
        if (owner >= 0) {
            const int b = owner * per, e = (b + per < vocab) ? b + per : vocab;
            for (int i = b; i < e; ++i) {
                const float z = row[i] / temp;
                if (z == z && order_key(z) >= thr) {
                    const float w = expf(z - zmax);
                    pick = i;                        // last kept entry of the chunk if rounding overshoots
                    if (target < run + w) break;
                    run += w;
                }
            }
        }
        if (pick < 0) pick = top.i;                  // floating-point slack: the most probable token
        chosen = pick;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[r] = chosen;
}

ZI_EXPORT int zi_sample(const float* logits, int* out, const float* temperature, const int* top_k, const float* top_p,
                        const float* uniform, int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return zi_fail("sample: vocab=%d must be positive", vocab);
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, out, temperature, top_k, top_p, uniform, vocab, row_stride);
    return zi_check_launch("sample");
}

// Hand-over between decode steps that run back to back on the device: the chosen token becomes
// the next input and every position moves on by one.  A token may carry several position numbers (`axes`
// runs, `axis_stride` elements apart); all of them move.
__global__ void advance_decode_kernel(int* __restrict__ ids, int* __restrict__ pos, const int* __restrict__ sampled, int n,
                                      int axes, long long axis_stride) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger_early();
    pdl_wait();
    pdl_trigger_late();
    if (i < n) {
        ids[i] = ld_dep(sampled + i);
        for (int a = 0; a < axes; ++a) pos[a * axis_stride + i] += 1;
    }
}

ZI_EXPORT int zi_advance_decode(int* ids, int* pos, const int* sampled, int n, int axes, long long axis_stride,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (axes < 1 || (axes > 1 && axis_stride < n)) return zi_fail("advance_decode: %d position axes %lld apart for %d rows", axes, axis_stride, n);
    zi_launch(advance_decode_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, pos, (const int*)sampled, n, axes, axis_stride);
    return zi_check_launch("advance_decode");
}
