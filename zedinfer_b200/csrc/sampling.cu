// Token choice from float32 logits [rows, vocab]: greedy, or temperature sampling with
// optional top-k / top-p, one thread block per row.
//
// Greedy: the largest logit; of equal logits the lowest index wins
// (src/backend/ops/argmax/cpu/argmax_cpu.cpp:15-19).
//
// Sampling, following src/frontend/sampler/sampler.cpp:195-265 and :410-490 in meaning:
//   z_i = logit_i / temperature;  w_i = exp(z_i - max z);  S = sum w
//     (w_i is computed as 2^((logit_i - max logit) * log2(e) / temperature), see Weigh; which entries equal the
//     k-th or the last of top-p is still decided on z, the quotient)
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

__device__ __forceinline__ float key_value(unsigned int key) {              // the float whose order_key is `key`
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
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
#define ARGMAX_THREADS 512
#define ARGMAX_UNROLL 8
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_slices_kernel(const float* __restrict__ logits, ArgPair* __restrict__ part, int vocab, long long row_stride, int slices) {
    __shared__ ArgPair scratch[32];
    const int per = (vocab + slices - 1) / slices;
    const int begin = blockIdx.y * per, end = min(vocab, begin + per);
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    // a slice of 4,096 entries is one round of eight loads per thread, all of them in flight together
    ArgPair best; best.v = -INFINITY; best.i = 0x7fffffff;
    for (int base = begin; base < end; base += ARGMAX_THREADS * ARGMAX_UNROLL) {
        float v[ARGMAX_UNROLL];
#pragma unroll
        for (int j = 0; j < ARGMAX_UNROLL; ++j) {
            const int i = base + j * ARGMAX_THREADS + (int)threadIdx.x;
            v[j] = i < end ? row[i] : -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < ARGMAX_UNROLL; ++j) {
            const int i = base + j * ARGMAX_THREADS + (int)threadIdx.x;
            if (i >= end) continue;
            ArgPair c; c.v = v[j] != v[j] ? -INFINITY : v[j]; c.i = i;
            best = better(best, c);
        }
    }
    const ArgPair r = block_best(best, scratch);
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
    argmax_slices_kernel<<<dim3(rows, slices), ARGMAX_THREADS, 0, stream>>>(logits, (ArgPair*)part, vocab, row_stride, slices);
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

// The same penalty from a table kept on the device: counts[slot][token] = how often the request in that slot has
// generated the token.  A row's logits are penalised as many times as the token was generated (the reference's loop
// over the generated tokens, src/frontend/sampler/sampler.cpp:439-451, in any order: a logit keeps its sign under
// the penalty, so the order of the listings does not matter).  The host then never sends the generated tokens, and
// a step that was launched before the host has read the step before it finds the table up to date.
//   rows whose slot is negative or whose penalty is 1 are left alone.
__global__ void penalty_rows_kernel(float* __restrict__ logits, const int* __restrict__ counts, const int* __restrict__ slots,
                                    const float* __restrict__ penalty, int vocab, long long row_stride, long long count_stride) {
    const int r = blockIdx.y;
    const int slot = slots[r];
    const float p = penalty[r];
    if (slot < 0 || p == 1.0f || !(p > 0.0f)) return;
    float* row = logits + (size_t)r * row_stride;
    const int* cnt = counts + (size_t)slot * count_stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
        int c = cnt[i];
        if (c <= 0) continue;
        float l = row[i];
        for (; c > 0; --c) l = l > 0.0f ? l / p : l * p;
        row[i] = l;
    }
}

// counts[slots[r]][tokens[r]] += 1 for the rows whose slot is not negative: the tokens a step has just chosen.
__global__ void count_tokens_kernel(int* __restrict__ counts, const int* __restrict__ slots, const int* __restrict__ tokens,
                                    int rows, int vocab, long long count_stride) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int slot = slots[r], t = tokens[r];
    if (slot < 0 || t < 0 || t >= vocab) return;
    counts[(size_t)slot * count_stride + t] += 1;              // one row per slot: nobody else adds to this entry
}

// counts_row[tokens[j]] += 1 for a list of tokens (a request that comes back after its slot was given away).
__global__ void count_token_list_kernel(int* __restrict__ counts_row, const int* __restrict__ tokens, int n, int vocab) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const int t = tokens[j];
    if (t >= 0 && t < vocab) atomicAdd(counts_row + t, 1);
}

ZI_EXPORT int zi_penalty_rows(float* logits, const int* counts, const int* slots, const float* penalty, int rows, int vocab,
                              long long row_stride, long long count_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return zi_fail("penalty_rows: rows=%d vocab=%d", rows, vocab);
    int blocks = (vocab + 4 * 256 - 1) / (4 * 256);
    if (blocks > 64) blocks = 64;
    penalty_rows_kernel<<<dim3(blocks, rows), 256, 0, stream>>>(logits, counts, slots, penalty, vocab, row_stride, count_stride);
    return zi_check_launch("penalty_rows");
}

ZI_EXPORT int zi_count_tokens(int* counts, const int* slots, const int* tokens, int rows, int vocab, long long count_stride,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    count_tokens_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(counts, slots, tokens, rows, vocab, count_stride);
    return zi_check_launch("count_tokens");
}

ZI_EXPORT int zi_count_token_list(int* counts_row, const int* tokens, int n, int vocab, cudaStream_t stream) {
    if (n <= 0) return 0;
    count_token_list_kernel<<<(n + 255) / 256, 256, 0, stream>>>(counts_row, tokens, n, vocab);
    return zi_check_launch("count_token_list");
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
// The short way.  A search seldom has to run to its last digit: as soon as the entries at or above the bin where
// the threshold lies are few enough (SAMPLE_LIST), they are gathered into the first block's shared memory and the
// rest (the exact k-th largest, top-p's running sums by size, the choice by index) is done there on a sorted list.
// Three sweeps usually get top-k there, two or three get top-p there when a few tokens hold most of the mass.
// 8 rows of 151,936 entries, a few likely tokens, top-k 20 + top-p 0.8: 36 us (18 sweeps the long way: 98 us).
//
// Choice (the long way).  A block's part of the row is cut into 32 stretches, one per warp, lanes on consecutive
// entries; the blocks' and warps' kept masses locate the stretch that holds u * (kept mass), and that warp walks
// its stretch 32 entries at a time with a prefix sum over the lanes until the running sum passes the target.
namespace cg = cooperative_groups;

#define SAMPLE_CLUSTER 8
#define SAMPLE_UNROLL 8
#define SAMPLE_BITS 5
#define SAMPLE_BINS (1 << SAMPLE_BITS)
#define SAMPLE_WALK_UNROLL 8

// What a block shows to the others of its cluster.  Two copies used in turn: a block writes copy n + 1 only after
// the cluster barrier of exchange n + 1's predecessor, which every block passes after it has read copy n.
struct SampleShare {
    ArgPair best;
    float sum;
    float mass;                                // kept mass of this block's part of the row
    int count;                                 // entries this block gathered
    float totals[SAMPLE_BINS];
};

__device__ __forceinline__ float sample_nan() { return __int_as_float(0x7fc00000); }

// An entry's weight exp(z - max z), z = logit / temperature, computed as 2^((logit - max logit) * log2(e) / temperature):
// the same number up to rounding (the difference of the logits is formed first, so near the maximum it is the more
// accurate of the two), and a sweep over the row pays no division per entry.
struct Weigh {
    float vmax, c;                             // c = log2(e) / temperature
    __device__ __forceinline__ float operator()(float v) const { return exp2f((v - vmax) * c); }
};

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
// need is a count) or wt(logit) (MASS = true); the smallest such key of the row if all of them together do
// not reach it, 0 if there is none.  The answer is the key of an entry of the row.  Every thread of every block of
// the cluster calls it and gets the same answer.
// stop_at > 0: the search ends as soon as the digits found so far leave at most stop_at (weight of) entries at or
// above them, those of the bin where the answer lies included; the key returned is then that bin's lowest (its
// unresolved low bits zero), `exact` is false, and whoever gathers the entries >= key finds the answer among them.
struct Threshold { unsigned int key; bool exact; };
template <bool MASS>
__device__ Threshold find_threshold(cg::cluster_group& cluster, const float* __restrict__ row, int begin, int end,
                                    const Weigh wt, float need, unsigned int floor_key, float stop_at,
                                    unsigned int kmax, float* acc, SampleShare* share, int& turn,
                                    volatile unsigned int* s_prefix, volatile float* s_reach) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int prefix = 0u;
    float above = 0.0f;                        // weight of the entries above the digits found so far (warp 0 keeps it)
    int top = 32;                              // the lowest bit resolved so far
    // kmax: the largest key of the row.  The first digit is almost always kmax's own (sign and the upper bits of the
    // exponent): the search begins below it, and starts over from the top only if kmax's bin alone falls short.
    bool guessing = kmax != 0u;
    if (guessing) { top = 32 - SAMPLE_BITS; prefix = kmax >> top << top; }
    while (top > 0) {
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
            acc[d * SAMPLE_THREADS + threadIdx.x] += MASS ? wt(v) : 1.0f;
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
            const float whole = __shfl_sync(0xffffffffu, from_top, 0);
            if (guessing && !(whole >= need)) {
                if (lane == 0) *s_reach = -1.0f;                // the guessed bin does not hold the answer
            } else {
                // the highest bin that holds something and reaches the need with all above it; if none does (the
                // whole is short of the need, or rounding), the lowest bin that holds something
                const unsigned int held = __ballot_sync(0xffffffffu, t > 0.0f);
                const unsigned int reach = __ballot_sync(0xffffffffu, t > 0.0f && above + from_top >= need);
                const int digit = reach ? 31 - __clz(reach) : (held ? __ffs(held) - 1 : 0);
                // entries above the chosen bin stay above for good
                const float beyond = __shfl_sync(0xffffffffu, from_top - t, digit);
                const float in_bin = __shfl_sync(0xffffffffu, t, digit);
                above += digit < 31 ? beyond : 0.0f;
                if (lane == 0) { *s_prefix = prefix | ((unsigned int)digit << shift); *s_reach = above + in_bin; }
            }
        }
        turn ^= 1;
        __syncthreads();
        const float reach = *s_reach;
        if (guessing) {
            guessing = false;
            if (reach < 0.0f) { prefix = 0u; top = 32; continue; }       // from the top (above is still 0)
        }
        prefix = *s_prefix;
        top = shift;
        if (stop_at > 0.0f) {
            // entries at or above the bin: counted, or (by mass) at most their mass over the least weight an entry
            // there can have, with a margin for rounding
            const float entries = MASS ? 1.02f * reach / wt(key_value(prefix)) : reach;
            if (entries <= stop_at) break;
        }
    }
    __syncthreads();                           // everyone has read the last digit before s_prefix is written again
    Threshold found; found.key = prefix; found.exact = top == 0;
    return found;
}

// ---- the short way: the entries that top-k keeps, gathered into one block's shared memory ----------------------
// With top-k at work the kept set is small (k entries and what ties with the k-th).  The blocks gather it, the
// first block takes all of it through distributed shared memory, and top-p and the choice are done there on a few
// hundred entries instead of in nine more sweeps over the row: sorted by size for top-p (running sums in that
// order), sorted by index for the choice.  Sorting makes the result independent of the order of gathering.  A kept
// set beyond SAMPLE_LIST entries (a k that large, or a k-th entry that ties with thousands) goes the long way.
#define SAMPLE_LIST 2048                       // entries that are gathered (by each block from its part, by the first from all)

// Bitonic sort of a[0, n2) (n2 a power of two, at most 2 * SAMPLE_THREADS) in shared memory, ascending.
__device__ void sort_ascending(unsigned long long* a, int n2) {
    for (int k = 2; k <= n2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int pair = threadIdx.x; pair < (n2 >> 1); pair += SAMPLE_THREADS) {
                const int t = ((pair & ~(j - 1)) << 1) | (pair & (j - 1)), o = t | j;      // the pair's lower and upper place
                const unsigned long long x = a[t], y = a[o];
                const bool up = (t & k) == 0;
                if ((x > y) == up) { a[t] = y; a[o] = x; }
            }
            __syncthreads();
        }
    }
}

// Running sums over 2 * SAMPLE_THREADS values in order, two per thread (w0 before w1): what lies before w0.  The
// order of the additions is fixed: pairs, lanes, warps.
__device__ float running_sum_before(float w0, float w1, float* scratch, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float incl = w0 + w1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    float before = 0.0f, all = 0.0f;
    for (int w = 0; w < 32; ++w) {                      // 32 additions in order, the same in every thread
        if (w == warp) before = all;
        all += scratch[w];
    }
    *total = all;
    return before + (incl - (w0 + w1));
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int vocab, long long row_stride) {
    extern __shared__ float acc[];             // [SAMPLE_BINS][SAMPLE_THREADS]; later the gathered entries
    __shared__ SampleShare share[2];
    __shared__ ArgPair ascratch[32];
    __shared__ float fscratch[32];
    __shared__ float warp_mass[32];
    __shared__ unsigned int s_prefix;
    __shared__ float s_run, s_target, s_reach; // s_run: kept mass before the owner's stretch
    __shared__ int s_owner, s_count, s_first, s_last;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = blockIdx.x;               // gridDim.x == SAMPLE_CLUSTER: rank in the cluster
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature[r];
    const int k = top_k[r];
    const float p = top_p[r];
    const bool sampled = temp > 0.0f;
    const bool by_k = sampled && k > 0 && k < vocab, by_p = sampled && p < 1.0f;
    // this block's part of the row, in 32 stretches of a multiple of 32 entries
    const int per = (((vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER + 31) / 32 + 31) / 32 * 32;
    const int cbegin = min(vocab, rank * per * 32), cend = min(vocab, cbegin + per * 32);
    int turn = 0;

    // One sweep for the largest entry of the row and the mass of every warp's stretch (each warp walks its stretch,
    // lanes on consecutive entries, SAMPLE_UNROLL loads in flight per lane): a lane keeps the mass of its entries
    // relative to the largest z it has met, and rescales when it meets a larger one.  The masses give top-p its total;
    // with neither top-k nor top-p at work they are the kept masses already, and the row is not swept again.
    const int begin = min(cend, cbegin + warp * per), end = min(cend, begin + per);
    const bool whole = sampled && !by_k && !by_p;              // everything is kept
    ArgPair top; top.v = -INFINITY; top.i = 0x7fffffff;
    float m = -INFINITY, s = 0.0f;                             // the lane's largest logit, its mass relative to that
    const float wc = sampled ? 1.4426950408889634f / temp : 0.0f;
    for (int base = begin; base < end; base += 32 * SAMPLE_UNROLL) {
        float v[SAMPLE_UNROLL];
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            const int i = base + j * 32 + lane;
            v[j] = i < end ? row[i] : sample_nan();
        }
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            if (v[j] != v[j]) continue;
            ArgPair c; c.v = v[j]; c.i = base + j * 32 + lane;
            top = better(top, c);
            if (by_p || whole) {
                if (v[j] > m) { s = s * exp2f((m - v[j]) * wc) + 1.0f; m = v[j]; }
                else if (v[j] > -INFINITY) s += exp2f((v[j] - m) * wc);
            }
        }
    }
    top = block_best(top, ascratch);
    if (threadIdx.x == 0) share[turn].best = top;
    cluster.sync();
    top.v = -INFINITY; top.i = 0x7fffffff;
#pragma unroll
    for (int c = 0; c < SAMPLE_CLUSTER; ++c) top = better(top, cluster.map_shared_rank(&share[turn], c)->best);
    turn ^= 1;
    if (top.i == 0x7fffffff) top.i = 0;
    if (!sampled || top.v == -INFINITY) {      // greedy row, or nothing to weigh: the first index
        if (rank == 0 && threadIdx.x == 0) out[r] = top.i;
        cluster.sync();                        // nobody leaves while its memory is still read
        return;
    }
    Weigh wt; wt.vmax = top.v; wt.c = wc;
    const unsigned int kmax = order_key(top.v);
    float S = 0.0f;                            // total mass: the lanes' sums brought to the row's largest logit, stretches and blocks in their order
    if (by_p || whole) {
        float mine = s > 0.0f ? s * wt(m) : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        if (lane == 0) warp_mass[warp] = mine;
        __syncthreads();
    }
    if (by_p) {
        if (threadIdx.x == 0) {
            float mass = 0.0f;
            for (int w = 0; w < 32; ++w) mass += warp_mass[w];
            share[turn].sum = mass;
        }
        cluster.sync();
#pragma unroll
        for (int c = 0; c < SAMPLE_CLUSTER; ++c) S += cluster.map_shared_rank(&share[turn], c)->sum;
        turn ^= 1;
    }

    // thresholds as keys of logits
    unsigned int thr_v = 0u;
    bool listed = false;                       // the search stopped early (or was for top-k): what is kept may fit the list
    bool exact = true;                         // thr_v is the threshold itself, not the lowest key of the bin where it lies
    if (by_k || by_p) {
        // the search (for the k-th largest; without top-k, for the entry where top-p's mass is reached) stops as soon
        // as the entries at or above the bin where it lies are sure to fit the list
        const Threshold found = by_k
            ? find_threshold<false>(cluster, row, cbegin, cend, wt, (float)k, 0u, (float)SAMPLE_LIST, kmax, acc,
                                    share, turn, &s_prefix, &s_reach)
            : find_threshold<true>(cluster, row, cbegin, cend, wt, p * S, 0u, (float)SAMPLE_LIST, kmax, acc,
                                   share, turn, &s_prefix, &s_reach);
        thr_v = found.key;
        exact = found.exact;
        listed = by_k || !found.exact;
    }
    if (listed) {
        // gather them (what is kept is among them)
        unsigned long long* local = reinterpret_cast<unsigned long long*>(acc);                 // [SAMPLE_LIST]
        unsigned long long* list = local + SAMPLE_LIST;                                         // [SAMPLE_LIST], used in block 0
        if (threadIdx.x == 0) s_count = 0;
        __syncthreads();
        sample_sweep(row, cbegin, cend, [&](float v, int i) {
            if (order_key(v) >= thr_v) {
                const int slot = atomicAdd(&s_count, 1);
                if (slot < SAMPLE_LIST) local[slot] = ((unsigned long long)(unsigned int)i << 32) | order_key(v);
            }
        });
        __syncthreads();
        if (threadIdx.x == 0) share[turn].count = s_count;
        cluster.sync();
        int n = 0, before = 0;
    #pragma unroll
    for (int c = 0; c < SAMPLE_CLUSTER; ++c) {
            const int cnt = cluster.map_shared_rank(&share[turn], c)->count;
            if (c < rank) before += cnt;
            n += cnt;
        }
        turn ^= 1;
        if (n <= SAMPLE_LIST) {                // the same n in every block (and then no block's share is cut short)
            unsigned long long* list0 = cluster.map_shared_rank(list, 0);
            for (int e = threadIdx.x; e < s_count; e += SAMPLE_THREADS) list0[before + e] = local[e];
            cluster.sync();
            // From here on nobody reads another block's memory: the others leave (and make room for the next rows'
            // blocks) while the first finishes the row.
            if (rank != 0) return;
            {
                int n2 = 2;
                while (n2 < n) n2 <<= 1;
                const int e0 = 2 * threadIdx.x, e1 = e0 + 1;           // this thread's two places in the sorted orders
                // by size, the lower index first among equals: descending = ascending in the complement
                for (int t = threadIdx.x; t < n2; t += SAMPLE_THREADS) {
                    const unsigned long long e = list[t];
                    list[t] = t < n ? ~(((e & 0xffffffffull) << 32) | (0xffffffffull - (e >> 32))) : ~0ull;
                }
                __syncthreads();
                sort_ascending(list, n2);
                // the k-th largest; what equals it is kept with it
                if (by_k && n > 0) thr_v = (unsigned int)(~list[min(k, n) - 1] >> 32);
                if (by_p) {
                    float w0 = 0.0f, w1 = 0.0f;
                    if (e0 < n) { const unsigned int key = (unsigned int)(~list[e0] >> 32); if (key >= thr_v) w0 = wt(key_value(key)); }
                    if (e1 < n) { const unsigned int key = (unsigned int)(~list[e1] >> 32); if (key >= thr_v) w1 = wt(key_value(key)); }
                    float all;
                    const float before0 = running_sum_before(w0, w1, fscratch, &all);
                    if (threadIdx.x == 0) s_first = 0x7fffffff;
                    __syncthreads();
                    const float need = p * S;
                    if (w0 > 0.0f && before0 + w0 >= need) atomicMin(&s_first, e0);
                    else if (w1 > 0.0f && before0 + w0 + w1 >= need) atomicMin(&s_first, e1);
                    __syncthreads();
                    if (s_first < n) thr_v = (unsigned int)(~list[s_first] >> 32);      // never below the k-th largest
                }
                // the kept set in terms of z, as on the long way; in this order it is the list's first `kept` entries
                const unsigned int thr = order_key(key_value(thr_v) / temp);
                if (threadIdx.x == 0) s_last = -1;
                __syncthreads();
                if (e1 < n && order_key(key_value((unsigned int)(~list[e1] >> 32)) / temp) >= thr) atomicMax(&s_last, e1);
                else if (e0 < n && order_key(key_value((unsigned int)(~list[e0] >> 32)) / temp) >= thr) atomicMax(&s_last, e0);
                __syncthreads();
                const int kept = s_last + 1;
                int k2 = 2;
                while (k2 < kept) k2 <<= 1;
                // those back to (index, key), in the order of the indices
                for (int t = threadIdx.x; t < k2; t += SAMPLE_THREADS) {
                    const unsigned long long e = ~list[t];
                    list[t] = t < kept ? (((0xffffffffull - (e & 0xffffffffull)) << 32) | (e >> 32)) : ~0ull;
                }
                __syncthreads();
                sort_ascending(list, k2);
                float w0 = 0.0f, w1 = 0.0f;
                if (e0 < kept) w0 = wt(key_value((unsigned int)list[e0]));
                if (e1 < kept) w1 = wt(key_value((unsigned int)list[e1]));
                float total;
                const float before0 = running_sum_before(w0, w1, fscratch, &total);
                if (threadIdx.x == 0) { s_first = 0x7fffffff; s_last = -1; }
                __syncthreads();
                const float target = uniform[r] * total;
                if (w0 > 0.0f && target < before0 + w0) atomicMin(&s_first, e0);
                else if (w1 > 0.0f && target < before0 + w0 + w1) atomicMin(&s_first, e1);
                if (w1 > 0.0f) atomicMax(&s_last, e1);
                else if (w0 > 0.0f) atomicMax(&s_last, e0);
                __syncthreads();
                if (threadIdx.x == 0) {
                    const int at = s_first < kept ? s_first : s_last;               // rounding overshoot: the last kept entry
                    out[r] = at >= 0 ? (int)(list[at] >> 32) : top.i;
                }
            }
            return;
        }
        // too many for the list: the search ran to its end without the kept set getting small (thousands tie with the
        // k-th largest, or top-p alone keeps thousands), and thr_v is exact.  The long way.
        if (!exact) {
            // (A search that stopped early promised that the list would do.  Should that promise ever be broken, the
            // bin's lowest key must not pass for the threshold: search again, to the end.)
            thr_v = by_k ? find_threshold<false>(cluster, row, cbegin, cend, wt, (float)k, 0u, 0.0f, kmax, acc, share, turn,
                                                 &s_prefix, &s_reach).key
                         : find_threshold<true>(cluster, row, cbegin, cend, wt, p * S, 0u, 0.0f, kmax, acc, share, turn,
                                                &s_prefix, &s_reach).key;
        }
    }
    if (by_p && by_k) {
        const unsigned int t = find_threshold<true>(cluster, row, cbegin, cend, wt, p * S, thr_v, 0.0f, kmax, acc,
                                                    share, turn, &s_prefix, &s_reach).key;
        if (t > thr_v) thr_v = t;
    }
    // the kept set in terms of z: everything whose z is at least the z of the threshold's entry.  z grows with the
    // logit, so that is everything from some logit on: `cut`, found by stepping down from the threshold's logit while
    // the quotient stays the same (a step or two; with a temperature so large that 64 steps do not reach the end,
    // every entry is divided and compared instead).
    unsigned int thr = 0u, cut = 0u;
    bool by_cut = true;
    if (thr_v != 0u) {
        thr = order_key(key_value(thr_v) / temp);
        cut = thr_v;
        for (int step = 0; cut > 1u && order_key(key_value(cut - 1u) / temp) >= thr; ++step) {
            if (step == 64) { by_cut = false; break; }
            --cut;
        }
    }
    auto is_kept = [&](float v) { return v == v && (by_cut ? order_key(v) >= cut : order_key(v / temp) >= thr); };

    // kept mass of each warp's stretch (known already where everything is kept)
    float mine = 0.0f;
    for (int base = begin; base < end && !whole; base += 32 * SAMPLE_UNROLL) {
        float v[SAMPLE_UNROLL];
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j) {
            const int i = base + j * 32 + lane;
            v[j] = i < end ? row[i] : sample_nan();
        }
#pragma unroll
        for (int j = 0; j < SAMPLE_UNROLL; ++j)
            if (is_kept(v[j])) mine += wt(v[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0 && !whole) warp_mass[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mass = 0.0f;
        for (int w = 0; w < 32; ++w) mass += warp_mass[w];
        share[turn].mass = mass;
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
        if (owner_block < 0 && rank == 0) out[r] = top.i;      // nothing kept anywhere: the most probable token
        s_owner = owner; s_run = run; s_target = target;
    }
    cluster.sync();                            // every block has read the others' masses: nobody's memory is read from here on
    if (warp == s_owner) {
        // This warp's stretch in index order, SAMPLE_WALK_UNROLL runs of 32 entries at a time: their weights and the
        // runs' masses first (independent of one another), then the runs in order until the running sum passes the
        // target, and a prefix sum over the lanes of that run alone.
        float run = s_run;
        const float target = s_target;
        int pick = -1, last_kept = -1;
        for (int base = begin; base < end && pick < 0; base += 32 * SAMPLE_WALK_UNROLL) {
            float w[SAMPLE_WALK_UNROLL], mass[SAMPLE_WALK_UNROLL];
#pragma unroll
            for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) {
                const int i = base + j * 32 + lane;
                w[j] = i < end ? row[i] : sample_nan();
            }
#pragma unroll
            for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) {
                w[j] = is_kept(w[j]) ? wt(w[j]) : 0.0f;
                mass[j] = w[j];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) mass[j] += __shfl_xor_sync(0xffffffffu, mass[j], o);
            }
#pragma unroll
            for (int j = 0; j < SAMPLE_WALK_UNROLL; ++j) {
                if (pick >= 0 || !(mass[j] > 0.0f)) continue;                      // the same in every lane
                const unsigned int kept = __ballot_sync(0xffffffffu, w[j] > 0.0f);
                if (target < run + mass[j]) {
                    float incl = w[j];                          // inclusive prefix sum over the lanes
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const float up = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += up;
                    }
                    const unsigned int hit = __ballot_sync(0xffffffffu, w[j] > 0.0f && target < run + incl);
                    // rounding (the run's mass was added in another order): the run's last kept entry
                    pick = base + j * 32 + (hit ? __ffs(hit) - 1 : 31 - __clz(kept));
                } else {
                    last_kept = base + j * 32 + (31 - __clz(kept));
                    run += mass[j];
                }
            }
        }
        if (pick < 0) pick = last_kept;                         // rounding overshoot: the stretch's last kept entry
        if (lane == 0) out[r] = pick >= 0 ? pick : top.i;
    }
}

ZI_EXPORT int zi_sample(const float* logits, int* out, const float* temperature, const int* top_k, const float* top_p,
                        const float* uniform, int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return zi_fail("sample: vocab=%d must be positive", vocab);
    if (rows > 65535) return zi_fail("sample: %d rows are more than one launch takes", rows);
    if (vocab > (1 << 24)) return zi_fail("sample: vocab=%d is beyond 16,777,216 (entries are counted in float32)", vocab);
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
