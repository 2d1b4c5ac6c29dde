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
#include <cooperative_groups.h>

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

// The best of row[begin, end) (consecutive threads on consecutive entries).
__device__ ArgPair block_best(ArgPair best, ArgPair* scratch);
__device__ ArgPair block_argmax(const float* __restrict__ row, int begin, int end, ArgPair* scratch) {
    ArgPair best; best.v = -INFINITY; best.i = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float v = ld_dep(row + i);
        if (v != v) v = -INFINITY;
        ArgPair c; c.v = v; c.i = i;
        best = better(best, c);
    }
    return block_best(best, scratch);
}
// The best of the threads' candidates; every thread gets it.
__device__ ArgPair block_best(ArgPair best, ArgPair* scratch) {
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
    return r;                              // index 0x7fffffff: nothing but NaN / -inf in the range
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, long long row_stride) {
    __shared__ ArgPair scratch[32];
    pdl_trigger_early();
    pdl_wait();
    pdl_trigger_late();
    const ArgPair r = block_argmax(logits + (size_t)blockIdx.x * row_stride, 0, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i == 0x7fffffff ? 0 : r.i;
}

// A large vocabulary in two stages: one block per row would walk 600 KB alone (35 us for 151,936 entries,
// whatever the number of rows); `slices` blocks per row leave the best of their slice in `part` [rows][slices]
// (value, index), and one warp per row takes the best of those, the lowest index among equals as before.
#define ARGMAX_SLICE 4096
#define ARGMAX_MAX_SLICES 32
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_slices_kernel(const float* __restrict__ logits, ArgPair* __restrict__ part, int vocab, long long row_stride, int slices) {
    __shared__ ArgPair scratch[32];
    const int per = (vocab + slices - 1) / slices;
    const int begin = blockIdx.y * per, end = min(vocab, begin + per);
    const ArgPair r = block_argmax(logits + (size_t)blockIdx.x * row_stride, begin, end, scratch);
    if (threadIdx.x == 0) part[(size_t)blockIdx.x * slices + blockIdx.y] = r;
}
__global__ void argmax_merge_kernel(const ArgPair* __restrict__ part, int* __restrict__ out, int slices) {
    ArgPair r; r.v = -INFINITY; r.i = 0x7fffffff;
    if ((int)threadIdx.x < slices) r = part[(size_t)blockIdx.x * slices + threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair c;
        c.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        c.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, c);
    }
    if (threadIdx.x == 0) out[blockIdx.x] = r.i == 0x7fffffff ? 0 : r.i;
}

ZI_EXPORT int zi_argmax_slices(int vocab) {
    const int s = (vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
    return s > ARGMAX_MAX_SLICES ? ARGMAX_MAX_SLICES : (s < 1 ? 1 : s);
}

// part: scratch of rows * zi_argmax_slices(vocab) * 2 words when that number is above one (else unused, may be null).
ZI_EXPORT int zi_argmax(const float* logits, int* out, int rows, int vocab, long long row_stride, void* part, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return zi_fail("argmax: vocab=%d must be positive", vocab);
    const int slices = zi_argmax_slices(vocab);
    if (slices == 1 || !part) {
        zi_launch(argmax_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, out, vocab, row_stride);
        return zi_check_launch("argmax");
    }
    if (rows > 65535) return zi_fail("argmax: %d rows are more than one launch takes", rows);
    argmax_slices_kernel<<<dim3(rows, slices), SAMPLE_THREADS, 0, stream>>>(logits, (ArgPair*)part, vocab, row_stride, slices);
    argmax_merge_kernel<<<rows, 32, 0, stream>>>((const ArgPair*)part, out, slices);
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

// ---- sampling ---------------------------------------------------------------------------------------------
// A cluster of eight blocks of 1,024 threads per row: block c walks the c-th eighth of the row, every thread with
// eight independent loads in flight, and what the blocks find (best entry, sums, bin totals, masses) is exchanged
// through distributed shared memory and added in the order of the blocks, so every block holds the same numbers
// and takes the same decisions.  (One block per row walked 600 KB alone, one load in flight per thread: 55 us a
// sweep at 151,936 entries.)
//
// Thresholds.  top-k wants the k-th largest entry, top-p the largest entry t such that the entries >= t (among
// those top-k kept) hold top_p of the mass.  Both are found digit by digit on the order-preserving key of the
// *logit* (z = logit / temperature is monotone in the logit, so no division is needed to compare): a sweep
// deals the entries whose higher digits equal the digits found so far into 32 bins by their next five bits, each
// thread adding into a column of its own in shared memory (no atomics: a bin's total is its 1,024 columns added in
// a fixed order by one warp, then the eight blocks' totals in the order of the blocks), and the bins are walked
// from the top.  Seven sweeps resolve 32 bits.  The threshold found is the key of an entry of the row; the kept
// set is then {z >= z of that entry}, which takes entries whose z equals it after the division along, as the rule
// on ties asks.  (Before: 32 sweeps per threshold, one bit each.)
//
// Choice.  A block's part of the row is cut into 32 stretches, one per warp, lanes on consecutive entries; the
// blocks' and warps' kept masses locate the stretch that holds u * (kept mass), and that warp walks its stretch 32
// entries at a time with a prefix sum over the lanes until the running sum passes the target.
namespace cg = cooperative_groups;

#define SAMPLE_CLUSTER 8
#define SAMPLE_UNROLL 8
#define SAMPLE_BITS 5
#define SAMPLE_BINS (1 << SAMPLE_BITS)
#define SAMPLE_WALK_UNROLL 4

// What a block shows to the others of its cluster.  Two copies used in turn: a block writes copy n + 1 only after
// the cluster barrier of exchange n + 1's predecessor, which every block passes after it has read copy n.
struct SampleShare {
    ArgPair best;
    float sum;
    float mass;                                // kept mass of this block's part of the row
    float totals[SAMPLE_BINS];
};

__device__ __forceinline__ float sample_nan() { return __int_as_float(0x7fc00000); }

// f(v, i) for every entry of row[begin, end) that is not NaN; consecutive threads on consecutive entries,
// SAMPLE_UNROLL loads in flight per thread.
template <typename F>
__device__ __forceinline__ void sample_sweep(const float* __restrict__ row, int begin, int end, F f) {
    for (int base = begin; base < end; base += SAMPLE_THREADS * SAMPLE_UNROLL) {
        float v[SAMPLE_UNROLL];
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            const int i = base + j * SAMPLE_THREADS + (int)threadIdx.x;
            v[j] = i < end ? row[i] : sample_nan();
        }
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j)
            if (v[j] == v[j]) f(v[j], base + j * SAMPLE_THREADS + (int)threadIdx.x);
    }
}

// The largest key t with weight{key >= max(t, floor_key)} >= need, where an entry's weight is 1 (MASS = false:
// need is a count) or exp(z - zmax) (MASS = true); the smallest such key of the row if all of them together do
// not reach it, 0 if there is none.  The answer is the key of an entry of the row.  Every thread of every block of
// the cluster calls it and gets the same answer.
template <bool MASS>
__device__ unsigned int find_threshold(cg::cluster_group& cluster, const float* __restrict__ row, int begin, int end,
                                       float temp, float zmax, float need, unsigned int floor_key, float* acc,
                                       SampleShare* share, int& turn, volatile unsigned int* s_prefix) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int prefix = 0u;
    float above = 0.0f;                        // weight of the entries above the digits found so far (warp 0 keeps it)
    for (int top = 32; top > 0; ) {
        // the digit of this sweep: bits [shift, top), top being the lowest bit resolved so far (the last digit is short)
        const int shift = top >= SAMPLE_BITS ? top - SAMPLE_BITS : 0;
        const unsigned int digit_mask = (1u << (top - shift)) - 1u;
#pragma unroll
        for (int b = 0; b < SAMPLE_BINS; ++b) acc[b * SAMPLE_THREADS + threadIdx.x] = 0.0f;
        sample_sweep(row, begin, end, [&](float v, int) {
            const unsigned int key = order_key(v);
            if (key < floor_key) return;
            if (top < 32 && (key >> top) != (prefix >> top)) return;
            const unsigned int d = (key >> shift) & digit_mask;
            acc[d * SAMPLE_THREADS + threadIdx.x] += MASS ? expf(v / temp - zmax) : 1.0f;
        });
        __syncthreads();
        {   // this block's total of bin `warp`: its columns in lane-strided order, then a fixed tree over the lanes
            float v = 0.0f;
            for (int t = lane; t < SAMPLE_THREADS; t += 32) v += acc[warp * SAMPLE_THREADS + t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) share[turn].totals[warp] = v;
        }
        cluster.sync();
        if (warp == 0) {
            // lane b: bin b over the blocks, in their order; then the bins from the top
            float t = 0.0f;
#pragma unroll
            for (int c = 0; c < SAMPLE_CLUSTER; ++c) t += cluster.map_shared_rank(&share[turn], c)->totals[lane];
            float from_top = t;                                 // bins lane .. 31, added from the top down
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_down_sync(0xffffffffu, from_top, o);
                if (lane + o < 32) from_top += up;
            }
            // the highest bin that holds something and reaches the need with all above it; if none does (the
            // whole is short of the need, or rounding), the lowest bin that holds something
            const unsigned int held = __ballot_sync(0xffffffffu, t > 0.0f);
            const unsigned int reach = __ballot_sync(0xffffffffu, t > 0.0f && above + from_top >= need);
            const int digit = reach ? 31 - __clz(reach) : (held ? __ffs(held) - 1 : 0);
            // entries above the chosen bin stay above for good
            const float beyond = __shfl_sync(0xffffffffu, from_top - t, digit);
            above += digit < 31 ? beyond : 0.0f;
            if (lane == 0) *s_prefix = prefix | ((unsigned int)digit << shift);
        }
        turn ^= 1;
        __syncthreads();
        prefix = *s_prefix;
        top = shift;
    }
    __syncthreads();                           // everyone has read the last digit before s_prefix is written again
    return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int vocab, long long row_stride) {
    extern __shared__ float acc[];             // [SAMPLE_BINS][SAMPLE_THREADS]
    __shared__ SampleShare share[2];
    __shared__ ArgPair ascratch[32];
    __shared__ float fscratch[32];
    __shared__ float warp_mass[32];
    __shared__ unsigned int s_prefix;
    __shared__ float s_run, s_target;          // s_run: kept mass before the owner's stretch
    __shared__ int s_owner;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.x;               // gridDim.x == SAMPLE_CLUSTER: rank in the cluster
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature[r];
    // this block's part of the row, in 32 stretches of a multiple of 32 entries
    const int per = (((vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER + 31) / 32 + 31) / 32 * 32;
    const int cbegin = min(vocab, rank * per * 32), cend = min(vocab, cbegin + per * 32);
    int turn = 0;

    // the largest entry of the row
    ArgPair top; top.v = -INFINITY; top.i = 0x7fffffff;
    sample_sweep(row, cbegin, cend, [&](float v, int i) { ArgPair c; c.v = v; c.i = i; top = better(top, c); });
    top = block_best(top, ascratch);
    if (threadIdx.x == 0) share[turn].best = top;
    cluster.sync();
    top.v = -INFINITY; top.i = 0x7fffffff;
#pragma unroll
    for (int c = 0; c < SAMPLE_CLUSTER; ++c) top = better(top, cluster.map_shared_rank(&share[turn], c)->best);
    turn ^= 1;
    if (top.i == 0x7fffffff) top.i = 0;
    if (!(temp > 0.0f) || top.v == -INFINITY) {             // greedy row, or nothing to weigh: the first index
        if (rank == 0 && threadIdx.x == 0) out[r] = top.i;
        cluster.sync();                        // nobody leaves while its memory is still read
        return;
    }
    const float zmax = top.v / temp;

    // thresholds as keys of logits
    unsigned int thr_v = 0u;
    const int k = top_k[r];
    if (k > 0 && k < vocab)
        thr_v = find_threshold<false>(cluster, row, cbegin, cend, temp, zmax, (float)k, 0u, acc, share, turn, &s_prefix);
    const float p = top_p[r];
    if (p < 1.0f) {
        // total mass S, the blocks' sums in their order
        float s = 0.0f;
        sample_sweep(row, cbegin, cend, [&](float v, int) { s += expf(v / temp - zmax); });
        s = block_sum(s, fscratch);
        if (threadIdx.x == 0) share[turn].sum = s;
        cluster.sync();
        float S = 0.0f;
#pragma unroll
        for (int c = 0; c < SAMPLE_CLUSTER; ++c) S += cluster.map_shared_rank(&share[turn], c)->sum;
        turn ^= 1;
        const unsigned int t = find_threshold<true>(cluster, row, cbegin, cend, temp, zmax, p * S, thr_v, acc, share, turn, &s_prefix);
        if (t > thr_v) thr_v = t;
    }
    // the kept set in terms of z: everything whose z is at least the z of the threshold's entry
    unsigned int thr = 0u;
    if (thr_v != 0u) {
        const unsigned int u = (thr_v & 0x80000000u) ? (thr_v & 0x7fffffffu) : ~thr_v;      // the key's float
        thr = order_key(__uint_as_float(u) / temp);
    }

    // kept mass of each warp's stretch, SAMPLE_UNROLL loads in flight per lane
    const int begin = min(cend, cbegin + warp * per), end = min(cend, begin + per);
    float mine = 0.0f;
    for (int base = begin; base < end; base += 32 * SAMPLE_UNROLL) {
        float v[SAMPLE_UNROLL];
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            const int i = base + j * 32 + lane;
            v[j] = i < end ? row[i] : sample_nan();
        }
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            const float z = v[j] / temp;
            if (z == z && order_key(z) >= thr) mine += expf(z - zmax);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) warp_mass[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.0f;
        for (int w = 0; w < 32; ++w) m += warp_mass[w];
        share[turn].mass = m;
    }
    cluster.sync();
    if (threadIdx.x == 0) {
        // the block, then the warp, whose stretch holds the target; rounding may leave the target at or past the
        // end of the kept mass: then the last stretch that keeps anything
        float mass[SAMPLE_CLUSTER], total = 0.0f;
#pragma unroll
        for (int c = 0; c < SAMPLE_CLUSTER; ++c) { mass[c] = cluster.map_shared_rank(&share[turn], c)->mass; total += mass[c]; }
        const float target = uniform[r] * total;
        float run = 0.0f;
        int owner_block = -1, last_block = -1;
#pragma unroll
        for (int c = 0; c < SAMPLE_CLUSTER; ++c) {
            if (owner_block >= 0 || !(mass[c] > 0.0f)) continue;
            last_block = c;
            if (target < run + mass[c]) owner_block = c; else run += mass[c];
        }
        if (owner_block < 0 && last_block >= 0) { owner_block = last_block; run -= mass[last_block]; }
        int owner = -1;
        if (owner_block == rank) {
            int last = -1;
            for (int w = 0; w < 32; ++w) {
                if (!(warp_mass[w] > 0.0f)) continue;
                last = w;
                if (target < run + warp_mass[w]) { owner = w; break; }
                run += warp_mass[w];
            }
            if (owner < 0) { owner = last; run -= warp_mass[last]; }
        }
        if (owner_block < 0 && rank == 0) out[r] = top.i;      // nothing kept anywhere (all -inf): the most probable token
        s_owner = owner; s_run = run; s_target = target;
    }
    __syncthreads();
    if (warp == s_owner) {
        // this warp's stretch in index order, 32 entries at a time
        float run = s_run;
        const float target = s_target;
        int pick = -1, last_kept = -1;
        for (int base = begin; base < end && pick < 0; base += 32 * SAMPLE_WALK_UNROLL) {
            float v[SAMPLE_WALK_UNROLL];
#pragma unroll
            for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) {
                const int i = base + j * 32 + lane;
                v[j] = i < end ? row[i] : sample_nan();
            }
#pragma unroll
            for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) {
                const float z = v[j] / temp;
                float w = 0.0f;
                if (z == z && order_key(z) >= thr) w = expf(z - zmax);
                float incl = w;                                 // inclusive prefix sum over the lanes
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                const unsigned int hit = __ballot_sync(0xffffffffu, w > 0.0f && target < run + incl);
                const unsigned int kept = __ballot_sync(0xffffffffu, w > 0.0f);
                if (pick < 0) {
                    if (hit) pick = base + j * 32 + (__ffs(hit) - 1);
                    else if (kept) last_kept = base + j * 32 + (31 - __clz(kept));
                }
                run += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        if (pick < 0) pick = last_kept;                         // rounding overshoot: the stretch's last kept entry
        if (lane == 0) out[r] = pick >= 0 ? pick : top.i;
    }
    cluster.sync();                            // nobody leaves while its memory is still read
}

ZI_EXPORT int zi_sample(const float* logits, int* out, const float* temperature, const int* top_k, const float* top_p,
                        const float* uniform, int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return zi_fail("sample: vocab=%d must be positive", vocab);
    if (rows > 65535) return zi_fail("sample: %d rows are more than one launch takes", rows);
    const size_t smem = (size_t)SAMPLE_BINS * SAMPLE_THREADS * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return zi_fail("sample: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SAMPLE_CLUSTER, rows);
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SAMPLE_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, logits, out, temperature, top_k, top_p, uniform, vocab, row_stride);
    if (e != cudaSuccess) return zi_fail("sample: launch failed: %s", cudaGetErrorString(e));
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
