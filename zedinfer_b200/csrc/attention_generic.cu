// Paged causal attention, one warp per (query token, query head); float32 or bfloat16 storage,
// float32 arithmetic.  Takes any head_dim that is a multiple of 8 up to 256, any number of
// heads and groups, any page size, and an optional window.
//
// This kernel is the whole 32-bit path and the general fallback of the bfloat16 path.  A query
// at absolute position P sees the keys lo..P of its own request, lo = max(0, P - window + 1)
// (window 0 = all keys).  Keys are visited in tiles of 32 starting at lo with one online-softmax
// rule, so the result for a query depends on P and the cache contents alone: not on how the
// prompt was cut into steps, nor on what else is in the batch.
//
// Cache addressing (one call's slice of the pool): element (page, kv, kvh, off, d) lives at
//   cache + page*page_stride + kv*kv_stride + (kvh*page_size + off)*head_dim + d.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(attention_generic)

#define WARPS 4
#define MAX_DREG 8            // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                       const int* __restrict__ tables, const int* __restrict__ tok_seg,
                       const int* __restrict__ pos, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                       int page_size, int max_blocks, long long page_stride, long long kv_stride, int window,
                       float scale) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem + warp * head_dim;                                     // this warp's query
    long long* rows = reinterpret_cast<long long*>(smem + WARPS * head_dim) + warp * 32;   // key row offsets
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int n = (int)(item / n_heads), h = (int)(item - (long long)n * n_heads);
    const int kvh = h / (n_heads / n_kv_heads);
    const int P = pos[n];
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    const int* table = tables + (size_t)tok_seg[n] * max_blocks;
    const T* qrow = q + ((size_t)n * n_heads + h) * head_dim;
    for (int d = lane; d < head_dim; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_DREG];
#pragma unroll
    for (int i = 0; i < MAX_DREG; ++i) acc[i] = 0.0f;

    for (int j0 = lo; j0 <= P; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= P;
        float s = -INFINITY;
        long long roff = 0;
        if (valid) {
            const int page = table[j / page_size];
            roff = (long long)page * page_stride + ((long long)kvh * page_size + (j % page_size)) * head_dim;
            const T* krow = cache + roff;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d += 8) {
                float kv[8];
                load8(krow + d, kv);
#pragma unroll
                for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
            }
            s = dot * scale;
        }
        rows[lane] = roff;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);          // first tile: exp(-inf) = 0
        l = l * corr + warp_sum(p);
        m = m_new;
        __syncwarp();
        const int cnt = (P - j0 + 1) < 32 ? (P - j0 + 1) : 32;
#pragma unroll
        for (int i = 0; i < MAX_DREG; ++i) acc[i] *= corr;
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vrow = cache + rows[jj] + kv_stride;
#pragma unroll
            for (int i = 0; i < MAX_DREG; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32<T>(vrow[d]), acc[i]);
            }
        }
        __syncwarp();
    }
    const float inv = 1.0f / l;
    T* orow = out + ((size_t)n * n_heads + h) * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_DREG; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

ZI_EXPORT int zi_paged_attention(const void* q, const void* cache, void* out, int dtype, const int* tables,
                                 const int* tok_seg, const int* pos, int n_tokens, int n_heads, int n_kv_heads,
                                 int head_dim, int page_size, int max_blocks, long long page_stride,
                                 long long kv_stride, int window, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim % 8 != 0 || head_dim > 32 * MAX_DREG)
        return zi_fail("attention: head_dim=%d must be a multiple of 8 and at most %d", head_dim, 32 * MAX_DREG);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return zi_fail("attention: %d query heads cannot share %d key/value heads", n_heads, n_kv_heads);
    if (page_size <= 0 || max_blocks <= 0) return zi_fail("attention: page_size=%d max_blocks=%d", page_size, max_blocks);
    const long long items = (long long)n_tokens * n_heads;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 0x7fffffffLL) return zi_fail("attention: too many (token, head) pairs: %lld", items);
    const size_t smem = (size_t)WARPS * head_dim * sizeof(float) + (size_t)WARPS * 32 * sizeof(long long);
    ZI_DISPATCH(dtype, T, {
        paged_attention_kernel<T><<<(unsigned)blocks, WARPS * 32, smem, stream>>>(
            (const T*)q, (const T*)cache, (T*)out, tables, tok_seg, pos, n_tokens, n_heads, n_kv_heads, head_dim,
            page_size, max_blocks, page_stride, kv_stride, window, scale);
    });
    return zi_check_launch("paged_attention");
}
