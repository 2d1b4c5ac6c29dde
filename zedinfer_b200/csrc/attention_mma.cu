// Paged causal attention for bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulate),
// head_dim 64 or 128, any number of heads and groups, any page size, optional window.
//
//   decode  : one query token per request.  The query heads that share a key/value head form the
//             rows of one 16-row tile, so the keys and values of a request cross the memory bus once
//             per key/value head.  A cluster of eight thread blocks shares a query group: the 64-key
//             tiles of the context are dealt out to the blocks in turn (a function of the query's own
//             position, never of the batch), each block keeps three tiles in flight, and the eight
//             partial results are merged in rank order through distributed shared memory.  No scratch
//             in global memory, no atomics.
//   prefill : a portion of a prompt.  One thread block per (64 query rows, query head); it walks the
//             keys from the window's start to the diagonal in tiles of 64 with an online softmax.
//
// Keys and values are gathered row by row through the block table with 16-byte cp.async copies
// into shared memory (double buffered, XOR-swizzled so that ldmatrix is conflict free).  Rows
// outside the range a query may see are zero-filled, never read: pages hold stale data beyond a
// request's length, and pages that a window has passed may be gone.
//
// Cache addressing (one call's slice of the pool): element (page, kv, kvh, off, d) lives at
//   cache + page*page_stride + kv*kv_stride + (kvh*page_size + off)*head_dim + d.
#define ZI_PDL_BIT 4
#include "tcgen05.cuh"

#include <cooperative_groups.h>

ZI_DEFINE_LAST_ERROR(attention_mma)

#define ATT_THREADS 128
#define TILE_KEYS 64
#define DEC_CLUSTER 8
#define DEC_STAGES 3
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` of row `row` in a swizzled [rows][HD] bfloat16 tile.
template <int HD> __device__ __forceinline__ uint32_t swz(int row, int c) {
    return (uint32_t)(row * HD * 2 + ((c ^ (row & 7)) << 4));
}

struct CacheRef {
    const bf16* base;
    const int* table;
    long long page_stride, kv_stride;
    int page_size, page_shift, kvh;
};

__device__ __forceinline__ const bf16* key_row(const CacheRef& cr, int key, int hd) {
    int blk, off;
    if (cr.page_shift >= 0) { blk = key >> cr.page_shift; off = key & (cr.page_size - 1); }
    else { blk = key / cr.page_size; off = key - blk * cr.page_size; }
    const int page = cr.table[blk];
    return cr.base + (long long)page * cr.page_stride + ((long long)cr.kvh * cr.page_size + off) * hd;
}

// Copy keys key0 .. key0+63 (K and V rows) into the swizzled tiles; rows outside [lo, hi] become zeros.
// Two threads share a row and take alternate 16-byte chunks, so the page lookup and the address
// arithmetic happen once per row and thread, and a pair of threads reads whole 32-byte sectors.
template <int HD>
__device__ __forceinline__ void load_kv_tile(const CacheRef& cr, uint32_t sK, uint32_t sV, int key0, int lo, int hi) {
    constexpr int CH = HD / 8;
    const int h = threadIdx.x & 1;
    for (int row = threadIdx.x >> 1; row < TILE_KEYS; row += ATT_THREADS / 2) {
        const int key = key0 + row;
        const bool valid = key >= lo && key <= hi;
        const bf16* src = valid ? key_row(cr, key, HD) : cr.base;
        const bf16* srcv = valid ? src + cr.kv_stride : cr.base;
        const uint32_t rowoff = (uint32_t)(row * HD * 2);
        const int r7 = row & 7;
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) {
            const int c = 2 * j + h;
            const uint32_t off = rowoff + (uint32_t)((c ^ r7) << 4);
            cp_async16(sK + off, valid ? src + c * 8 : src, valid);
            cp_async16(sV + off, valid ? srcv + c * 8 : srcv, valid);
        }
    }
}

// S[nt] (16 rows x 8 keys each) = Q (16 x HD, fragments in registers) . K^T for NKT*8 keys from row `row0`.
template <int HD, int NKT>
__device__ __forceinline__ void qk_scores(float (&S)[NKT][4], const uint32_t (&qf)[HD / 16][4], uint32_t sK, int row0, int lane) {
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt) {
        S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.0f;
        const int row = row0 + nt * 8 + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < HD / 32; ++kk) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, sK + swz<HD>(row, kk * 4 + (lane >> 3)));
            mma_bf16(S[nt], qf[2 * kk], b0, b1);
            mma_bf16(S[nt], qf[2 * kk + 1], b2, b3);
        }
    }
}

// O (16 x HD) += P (16 x NKT*8, probabilities in S) . V for the keys from row `row0`.
template <int HD, int NKT>
__device__ __forceinline__ void pv_accumulate(float (&O)[HD / 8][4], const float (&S)[NKT][4], uint32_t sV, int row0, int lane) {
#pragma unroll
    for (int kt = 0; kt < NKT / 2; ++kt) {
        uint32_t a[4];
        a[0] = pack_bf16(S[2 * kt][0], S[2 * kt][1]);
        a[1] = pack_bf16(S[2 * kt][2], S[2 * kt][3]);
        a[2] = pack_bf16(S[2 * kt + 1][0], S[2 * kt + 1][1]);
        a[3] = pack_bf16(S[2 * kt + 1][2], S[2 * kt + 1][3]);
        const int row = row0 + kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int dn = 0; dn < HD / 16; ++dn) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, sV + swz<HD>(row, dn * 2 + (lane >> 4)));
            mma_bf16(O[2 * dn], a, b0, b1);
            mma_bf16(O[2 * dn + 1], a, b2, b3);
        }
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));       // exp2(-inf) = +0
    return y;
}

// Online softmax step on a warp's score tile.  Thread holds rows g = lane/4 (values [0],[1]) and g+8
// ([2],[3]) at keys key0 + nt*8 + (lane%4)*2 + {0,1}.  lo / hi: first / last key each row may see.
// S comes in as raw dot products and leaves as probabilities relative to the running maximum; m is kept
// in units of raw scores (scale2 > 0, so the maximum is the same), and exp2(s*scale2 - m*scale2) is one
// fused multiply-add and one ex2.  MASKED = false is for tiles every row of the warp sees in full.
template <int HD, int NKT, bool MASKED = true>
__device__ __forceinline__ void softmax_step(float (&S)[NKT][4], float (&O)[HD / 8][4], float (&m)[2], float (&l)[2],
                                             int key0, int lane, int lo0, int hi0, int lo1, int hi1, float scale2) {
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (MASKED) {
                const int key = key0 + nt * 8 + (lane & 3) * 2 + e;
                if (!(key >= lo0 && key <= hi0)) S[nt][e] = -INFINITY;
                if (!(key >= lo1 && key <= hi1)) S[nt][2 + e] = -INFINITY;
            }
            mx0 = fmaxf(mx0, S[nt][e]);
            mx1 = fmaxf(mx1, S[nt][2 + e]);
        }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float use0 = mn0 == -INFINITY ? 0.0f : mn0, use1 = mn1 == -INFINITY ? 0.0f : mn1;
    const float c0 = fast_exp2((m[0] - use0) * scale2), c1 = fast_exp2((m[1] - use1) * scale2);   // first tile: 0
    const float b0 = -use0 * scale2, b1 = -use1 * scale2;
    m[0] = mn0;
    m[1] = mn1;
    float r0 = 0.0f, r1 = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float p0 = fast_exp2(fmaf(S[nt][e], scale2, b0)), p1 = fast_exp2(fmaf(S[nt][2 + e], scale2, b1));
            S[nt][e] = p0;
            S[nt][2 + e] = p1;
            r0 += p0;
            r1 += p1;
        }
    }
    l[0] = l[0] * c0 + r0;           // per-thread part of the row sum; the four threads of a row add up at the end
    l[1] = l[1] * c1 + r1;
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) {
        O[dn][0] *= c0; O[dn][1] *= c0;
        O[dn][2] *= c1; O[dn][3] *= c1;
    }
}

// =======================================================================================
// decode
// =======================================================================================
// grid (DEC_CLUSTER, n_kv_heads * q_blocks, n_tokens), thread-block clusters of DEC_CLUSTER along x;
// q_blocks = ceil(group / 16).  The blocks of a cluster share one query group: block r takes the 64-key
// tiles r, r + DEC_CLUSTER, ... of the visible range (a function of the query's own position only), streams
// them through a three-stage cp.async ring, and leaves (m, l, O) of its keys in its shared memory.  After a
// cluster barrier every block reads the eight partial results through distributed shared memory and writes
// one eighth of the output columns, adding the blocks in rank order.
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS)
decode_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, bf16* __restrict__ out,
                        const int* __restrict__ tables, const int* __restrict__ tok_seg,
                        const int* __restrict__ pos, int n_heads, int n_kv_heads, int q_blocks, int page_size,
                        int page_shift, int max_blocks, long long page_stride, long long kv_stride, int window,
                        float scale2) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = TILE_KEYS * HD * 2;
    constexpr int OS = HD + 8;                                    // padded row of float32 partial results
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = blockIdx.x;                                  // gridDim.x == DEC_CLUSTER: rank in the cluster
    const int kvh = blockIdx.y / q_blocks, qb = blockIdx.y - kvh * q_blocks;
    const int n = blockIdx.z;
    const int group = n_heads / n_kv_heads;
    pdl_trigger_early();
    pdl_wait();
    const int P = ld_dep(pos + n);
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    const int t_lo = lo / TILE_KEYS, t_hi = P / TILE_KEYS;
    const int n_mine = (t_hi - t_lo - rank >= 0) ? (t_hi - t_lo - rank) / DEC_CLUSTER + 1 : 0;

    CacheRef cr;
    cr.base = cache; cr.table = tables + (size_t)tok_seg[n] * max_blocks;
    cr.page_stride = page_stride; cr.kv_stride = kv_stride; cr.page_size = page_size; cr.page_shift = page_shift; cr.kvh = kvh;

    // shared memory: Q [16][HD] | DEC_STAGES x (K tile, V tile) | result of this block: m[16], l[16], O[16][OS]
    // | in-block merge of the four warps: m[4][16], l[4][16], O[4][16][OS] (overlays the tile ring)
    const uint32_t sQ = smem_u32(smem_raw);
    unsigned char* ring = smem_raw + 16 * HD * 2;
    const uint32_t sKV = smem_u32(ring);
    float* res_m = reinterpret_cast<float*>(ring + (size_t)DEC_STAGES * 2 * TILE_BYTES);
    float* res_l = res_m + 16;
    float* res_o = res_l + 16;

    const int rows_valid = (group - qb * 16) < 16 ? (group - qb * 16) : 16;
    for (int i = threadIdx.x; i < 16 * (HD / 8); i += ATT_THREADS) {
        const int row = i / (HD / 8), c = i - row * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows_valid) {
            const int h = kvh * group + qb * 16 + row;
            v = ld_dep16(q + ((size_t)n * n_heads + h) * HD + c * 8);
        }
        *reinterpret_cast<uint4*>(smem_raw + swz<HD>(row, c)) = v;
    }
    // prologue: the first DEC_STAGES tiles of this block; one commit group per stage whether it holds a tile or not
#pragma unroll
    for (int s = 0; s < DEC_STAGES; ++s) {
        if (s < n_mine) {
            const int t = t_lo + rank + s * DEC_CLUSTER;
            load_kv_tile<HD>(cr, sKV + s * 2 * TILE_BYTES, sKV + s * 2 * TILE_BYTES + TILE_BYTES, t * TILE_KEYS, lo, P);
        }
        cp_async_commit();
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                    sQ + swz<HD>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    float O[HD / 8][4];
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) O[dn][0] = O[dn][1] = O[dn][2] = O[dn][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    for (int i = 0; i < n_mine; ++i) {
        const int stage = i % DEC_STAGES;
        cp_async_wait<DEC_STAGES - 1>();                      // all but the newest DEC_STAGES-1 groups: tile i is here
        __syncthreads();
        const uint32_t sK = sKV + stage * 2 * TILE_BYTES, sV = sK + TILE_BYTES;
        const int key0 = (t_lo + rank + i * DEC_CLUSTER) * TILE_KEYS + warp * 16;
        if (key0 <= P && key0 + 15 >= lo) {                   // this warp's 16 keys hold something visible
            float S[2][4];
            qk_scores<HD, 2>(S, qf, sK, warp * 16, lane);
            softmax_step<HD, 2>(S, O, m, l, key0, lane, lo, P, lo, P, scale2);
            pv_accumulate<HD, 2>(O, S, sV, warp * 16, lane);
        }
        __syncthreads();                                      // the stage is free again
        if (i + DEC_STAGES < n_mine) {
            const int t = t_lo + rank + (i + DEC_STAGES) * DEC_CLUSTER;
            load_kv_tile<HD>(cr, sK, sV, t * TILE_KEYS, lo, P);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    pdl_trigger_late();
    m[0] *= scale2;                                               // from raw-score units to log2 units (-inf stays)
    m[1] *= scale2;
    // row sums over the four threads of a row
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

    // merge the four warps (each saw other keys) in warp order, through the memory of the tile ring
    float* red_m = reinterpret_cast<float*>(ring);               // [4][16]
    float* red_l = red_m + 64;                                    // [4][16]
    float* red_o = red_l + 64;                                    // [4][16][OS]
    const int g = lane >> 2, tq = lane & 3;
    if (tq == 0) {
        red_m[warp * 16 + g] = m[0]; red_m[warp * 16 + g + 8] = m[1];
        red_l[warp * 16 + g] = l[0]; red_l[warp * 16 + g + 8] = l[1];
    }
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) {
        *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + g) * OS + dn * 8 + tq * 2) = make_float2(O[dn][0], O[dn][1]);
        *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + g + 8) * OS + dn * 8 + tq * 2) = make_float2(O[dn][2], O[dn][3]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * HD; i += ATT_THREADS) {
        const int row = i / HD, d = i - row * HD;
        float Mr = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) Mr = fmaxf(Mr, red_m[w * 16 + row]);
        const float ur = Mr == -INFINITY ? 0.0f : Mr;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += red_o[((size_t)w * 16 + row) * OS + d] * exp2f(red_m[w * 16 + row] - ur);
        res_o[(size_t)row * OS + d] = acc;
    }
    if (threadIdx.x < 16) {
        const int row = threadIdx.x;
        float Mr = -INFINITY;
        for (int w = 0; w < 4; ++w) Mr = fmaxf(Mr, red_m[w * 16 + row]);
        const float ur = Mr == -INFINITY ? 0.0f : Mr;
        float Lr = 0.0f;
        for (int w = 0; w < 4; ++w) Lr += red_l[w * 16 + row] * exp2f(red_m[w * 16 + row] - ur);
        res_m[row] = Mr;
        res_l[row] = Lr;
    }
    cluster.sync();                                               // every block's (m, l, O) is in place
    // block `rank` writes the columns d with d / (HD / DEC_CLUSTER) == rank, adding the blocks in rank order
    constexpr int DW = HD / DEC_CLUSTER;
    for (int i = threadIdx.x; i < rows_valid * DW; i += ATT_THREADS) {
        const int row = i / DW, d = rank * DW + (i - row * DW);
        float pm[DEC_CLUSTER], pl[DEC_CLUSTER], po[DEC_CLUSTER];
#pragma unroll
        for (int r = 0; r < DEC_CLUSTER; ++r) {
            const float* rm = cluster.map_shared_rank(res_m, r);
            pm[r] = rm[row];
            pl[r] = rm[16 + row];
            po[r] = rm[32 + (size_t)row * OS + d];
        }
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < DEC_CLUSTER; ++r) M = fmaxf(M, pm[r]);
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int r = 0; r < DEC_CLUSTER; ++r) {
            const float f = exp2f(pm[r] - M);                     // blocks without keys: exp2(-inf) = 0
            L += pl[r] * f;
            acc += po[r] * f;
        }
        const int h = kvh * group + qb * 16 + row;
        out[((size_t)n * n_heads + h) * HD + d] = __float2bfloat16_rn(acc / L);
    }
    cluster.sync();                                               // nobody leaves while its memory is still read
}

// =======================================================================================
// decode, tiles by TMA
// =======================================================================================
// A cluster of CL blocks per (request, key/value head) and the same merge, but the keys are dealt
// out in tiles of 32 to single WARPS (tile g goes to block g % CL, warp (g / CL) % 4), and every warp runs on its
// own: its tiles come by TMA through the 5-d tensor map of the layer's cache (pages straight from the block
// table, 128-byte swizzle) into a ring of its own with an mbarrier per stage, so there is no block-wide barrier
// in the loop and a whole warp's share of a 3,000-key context is in flight at once.  A warp works on 32 keys per
// step instead of 16, which halves the number of dependent ldmatrix -> mma -> softmax -> mma chains.
// Page numbers are read 32 at a time, ahead of the tiles they belong to.  Keys outside what the query may see
// are masked by position; their cache slots hold finite stale values (the pool is allocated zeroed).
#define DT_STAGES 3

// A stage of the ring holds one tile as [hd halves][keys | values][rows][128 bytes], so that one TMA box may bring the
// keys and the values of a half together.  Byte offset of 16-byte chunk c of row `row` of the keys (the values are
// ROWS * 128 bytes further on):
template <int ROWS> __device__ __forceinline__ uint32_t swz_tma(int row, int c) {
    return (uint32_t)((c >> 3) * (2 * ROWS * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}
template <int HD, int NKT>      // NKT * 8 keys per tile
__device__ __forceinline__ void qk_scores_tma(float (&S)[NKT][4], const uint32_t (&qf)[HD / 16][4], uint32_t sK, int lane) {
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt) {
        S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.0f;
        const int row = nt * 8 + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < HD / 32; ++kk) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, sK + swz_tma<NKT * 8>(row, kk * 4 + (lane >> 3)));
            mma_bf16(S[nt], qf[2 * kk], b0, b1);
            mma_bf16(S[nt], qf[2 * kk + 1], b2, b3);
        }
    }
}
template <int HD, int NKT>
__device__ __forceinline__ void pv_accumulate_tma(float (&O)[HD / 8][4], const float (&S)[NKT][4], uint32_t sV, int lane) {
#pragma unroll
    for (int kt = 0; kt < NKT / 2; ++kt) {
        uint32_t a[4];
        a[0] = pack_bf16(S[2 * kt][0], S[2 * kt][1]);
        a[1] = pack_bf16(S[2 * kt][2], S[2 * kt][3]);
        a[2] = pack_bf16(S[2 * kt + 1][0], S[2 * kt + 1][1]);
        a[3] = pack_bf16(S[2 * kt + 1][2], S[2 * kt + 1][3]);
        const int row = kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int dn = 0; dn < HD / 16; ++dn) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, sV + swz_tma<NKT * 8>(row, dn * 2 + (lane >> 4)));
            mma_bf16(O[2 * dn], a, b0, b1);
            mma_bf16(O[2 * dn + 1], a, b2, b3);
        }
    }
}

// How many of the n_splits clusters that a launch provides for one (request, key/value head) are at work for a
// request with `tiles` visible tiles: the same answer in the attention kernel and in the merge kernel.
// Sharing pays from DT_SPLIT_FROM keys on (below that one cluster is as fast and the merge is saved); each cluster
// then takes at least DT_SPLIT_KEYS keys.
#define DT_SPLIT_KEYS 1024
#define DT_SPLIT_FROM 4096
__device__ __forceinline__ int dt_effective_splits(int tiles, int n_splits, int min_split_tiles) {
    if (n_splits <= 1) return 1;
    const int e = tiles / min_split_tiles;
    return e < DT_SPLIT_FROM / DT_SPLIT_KEYS ? 1 : (e > n_splits ? n_splits : e);
}

// Adds the parts of the clusters that shared one request's keys, in the order of the keys: grid (tokens, heads),
// HD threads.  Requests whose keys one cluster took alone have their output already.
template <int HD>
__global__ void __launch_bounds__(HD)
decode_attention_merge_kernel(const float* __restrict__ part, bf16* __restrict__ out, const int* __restrict__ pos,
                              int n_heads, int window, int dt_keys, int n_splits, int min_split_tiles) {
    const int n = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int P = pos[n];
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    const int eff = dt_effective_splits(P / dt_keys - lo / dt_keys + 1, n_splits, min_split_tiles);
    if (eff == 1) return;
    const float* src = part + ((size_t)n * n_heads + h) * n_splits * (HD + 2);
    float M = -INFINITY;
    for (int s = 0; s < eff; ++s) M = fmaxf(M, src[(size_t)s * (HD + 2)]);
    float acc = 0.0f, L = 0.0f;
    for (int s = 0; s < eff; ++s) {
        const float f = exp2f(src[(size_t)s * (HD + 2)] - M);
        L += src[(size_t)s * (HD + 2) + 1] * f;
        acc += src[(size_t)s * (HD + 2) + 2 + d] * f;
    }
    out[((size_t)n * n_heads + h) * HD + d] = __float2bfloat16_rn(acc / L);
}

template <int HD, int DT_KEYS, int CL>
__global__ void __launch_bounds__(ATT_THREADS)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, bf16* __restrict__ out,
                            const int* __restrict__ tables, const int* __restrict__ tok_seg, const int* __restrict__ pos,
                            int* __restrict__ status, int n_heads, int n_kv_heads, int q_blocks, int page_size,
                            int box_rows, int max_blocks, int window, float scale2, int n_splits, int min_split_tiles,
                            float* __restrict__ part, int kv_box) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int HH = HD / 64;
    constexpr int TILE_BYTES = DT_KEYS * HD * 2;                  // K or V of one tile
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int OS = HD + 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rank = blockIdx.x;
    const int split = blockIdx.y % n_splits, unit = blockIdx.y / n_splits;
    const int kvh = unit / q_blocks, qb = unit - kvh * q_blocks;
    const int n = blockIdx.z;
    const int group = n_heads / n_kv_heads;
    const int first = rank + CL * warp;                  // this warp's first tile, counted from the first of its cluster
    // tok_seg null: token n is segment n (every decode step of the engine).  Without a window and without sharing, a
    // warp's tiles start at key 0 whatever the position is, so its first page numbers are asked for together with
    // the position instead of after it: one trip to memory less before the first tile can be fetched.
    const int* table = tables + (size_t)(tok_seg ? tok_seg[n] : n) * max_blocks;
    const int ppt = DT_KEYS / box_rows;                           // TMA boxes (pages, or parts of one page) per tile
    const bool ids_ahead = window == 0 && n_splits == 1;
    int id_base = 0, id_reg = -1;
    if (ids_ahead) {
        const int tl = lane / ppt, pg = lane - tl * ppt;
        const int blk = ((first + tl * CL * 4) * DT_KEYS + pg * box_rows) / page_size;
        if (blk < max_blocks) id_reg = table[blk];
    }
    const int P = pos[n];
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    // The visible tiles may be shared out over several clusters (long contexts of few requests, see dt_splits): as
    // many of the n_splits as leave each at least min_split_tiles tiles.  Clusters beyond that number have nothing
    // to do; with more than one at work each leaves (m, l, O) in `part` and decode_attention_merge_kernel adds them.
    const int v_lo = lo / DT_KEYS, v_hi = P / DT_KEYS;
    const int eff = dt_effective_splits(v_hi - v_lo + 1, n_splits, min_split_tiles);
    if (split >= eff) return;
    const int per = (v_hi - v_lo + eff) / eff;
    const int t_lo = v_lo + split * per, t_hi = min(v_hi, t_lo + per - 1);
    const int n_mine = (t_hi - t_lo - first >= 0) ? (t_hi - t_lo - first) / (CL * 4) + 1 : 0;

    // shared memory: ring [4 warps][DT_STAGES][K tile | V tile] (1024-aligned) | Q [16][HD] | mbarriers | result of
    // this block m[16], l[16], O[16][OS]; the merge of the four warps overlays the ring afterwards
    unsigned char* ring = smem_raw;
    unsigned char* q_raw = ring + 4 * DT_STAGES * STAGE_BYTES;
    const uint32_t sQ = smem_u32(q_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_raw + 16 * HD * 2);
    float* res_m = reinterpret_cast<float*>(bars + 4 * DT_STAGES);
    float* res_l = res_m + 16;
    float* res_o = res_l + 16;
    const uint32_t my_ring = smem_u32(ring) + warp * DT_STAGES * STAGE_BYTES;
    const uint32_t my_bars = smem_u32(bars) + warp * DT_STAGES * 8;

    if (lane == 0)
        for (int s = 0; s < DT_STAGES; ++s) mbar_init(my_bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    __syncwarp();

    // page numbers of this warp's tiles, 32 at a time: entry e = tile * ppt + page of the tile
    // loads per tile: k|v x pages x halves, or, where a tile lies in one page and the map's box takes keys and values
    // together (kv_box), one per half: issuing a load costs the lane about 60 clocks
    const int ops = kv_box ? HH : 2 * ppt * HH;
    auto load_ids = [&](int base) {
        id_base = base;
        const int e = base + lane, tl = e / ppt, pg = e - tl * ppt;
        int v = -1;
        if (tl < n_mine) {
            const int key0 = (t_lo + first + tl * CL * 4) * DT_KEYS + pg * box_rows;
            const int blk = key0 / page_size;
            if (blk < max_blocks) v = table[blk];
        }
        id_reg = v;
    };
    // This kernel may be launched while the one before it on the stream (the q/k/v product with the rotation and the
    // cache append in its epilogue) still runs: everything up to here, and the loads of tiles that hold only older
    // keys, then overlap with it.  What that kernel writes (the new token's keys and values, Q) is touched only
    // after dependent_wait().
    bool waited = false;
    auto dependent_wait = [&]() {
        if (!waited) { asm volatile("griddepcontrol.wait;\n" ::: "memory"); waited = true; }
    };
    auto issue = [&](int tl) {
        const int st = tl % DT_STAGES;
        if (t_lo + first + tl * CL * 4 >= v_hi) dependent_wait();       // the tile with the new token's key
        if ((tl + 1) * ppt > id_base + 32) load_ids(tl * ppt);
        const uint32_t bar = my_bars + 8 * st;
        if (lane == 0) mbar_expect_tx(bar, STAGE_BYTES);
        __syncwarp();
        const int kv = kv_box ? 0 : lane / (ppt * HH), rem = lane - kv * (ppt * HH);
        const int pg = kv_box ? 0 : rem / HH, hh = kv_box ? lane : rem - pg * HH;
        const int page = __shfl_sync(0xffffffffu, id_reg, (tl * ppt + pg - id_base) & 31);
        if (lane < ops) {
            const int key0 = (t_lo + first + tl * CL * 4) * DT_KEYS + pg * box_rows;
            const uint32_t dst = my_ring + st * STAGE_BYTES + hh * (2 * DT_KEYS * 128) + kv * (DT_KEYS * 128) + pg * box_rows * 128;
            tma_load_5d(dst, &map_kv, hh * 64, key0 % page_size, kvh, kv, page, bar);
        }
        __syncwarp();
    };
    if (n_mine > 0 && !ids_ahead) load_ids(0);
    for (int s = 0; s < DT_STAGES && s < n_mine; ++s) issue(s);

    const int rows_valid = (group - qb * 16) < 16 ? (group - qb * 16) : 16;
    dependent_wait();
    for (int i = threadIdx.x; i < 16 * (HD / 8); i += ATT_THREADS) {
        const int row = i / (HD / 8), c = i - row * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows_valid) {
            const int h = kvh * group + qb * 16 + row;
            // through L2: Q was written while this kernel was already running, which the read-only path must not meet
            v = __ldcg(reinterpret_cast<const uint4*>(q + ((size_t)n * n_heads + h) * HD + c * 8));
        }
        *reinterpret_cast<uint4*>(q_raw + swz<HD>(row, c)) = v;
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                    sQ + swz<HD>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    float O[HD / 8][4];
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) O[dn][0] = O[dn][1] = O[dn][2] = O[dn][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    bool ok = true;
    int failed_at = 0;
    for (int i = 0; i < n_mine; ++i) {
        const int st = i % DT_STAGES;
        if (!mbar_wait_warp(my_bars + 8 * st, (i / DT_STAGES) & 1, nullptr)) { ok = false; failed_at = i; break; }
        const uint32_t sK = my_ring + st * STAGE_BYTES, sV = sK + DT_KEYS * 128;
        const int key0 = (t_lo + first + i * CL * 4) * DT_KEYS;
        float S[DT_KEYS / 8][4];
        qk_scores_tma<HD, DT_KEYS / 8>(S, qf, sK, lane);
        if (key0 >= lo && key0 + DT_KEYS - 1 <= P) softmax_step<HD, DT_KEYS / 8, false>(S, O, m, l, key0, lane, lo, P, lo, P, scale2);
        else softmax_step<HD, DT_KEYS / 8, true>(S, O, m, l, key0, lane, lo, P, lo, P, scale2);
        pv_accumulate_tma<HD, DT_KEYS / 8>(O, S, sV, lane);
        __syncwarp();                                             // every lane has read the stage
        if (i + DT_STAGES < n_mine) issue(i + DT_STAGES);
    }
    if (!ok) {
        if (lane == 0) atomicExch(status, 31);
        // loads in flight must land before the block's memory goes away: wait (bounded) for the tiles asked for
        for (int j = failed_at; j < n_mine && j < failed_at + DT_STAGES; ++j) mbar_wait(my_bars + 8 * (j % DT_STAGES), (j / DT_STAGES) & 1, nullptr);
        m[0] = m[1] = -INFINITY; l[0] = l[1] = 0.0f;
    }
    __syncthreads();                                              // all warps are done with the ring
    m[0] *= scale2;
    m[1] *= scale2;
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

    // merge the four warps in warp order through the memory of the ring: first one factor per (warp, row) ...
    float* red_m = reinterpret_cast<float*>(ring);               // [4][16]
    float* red_l = red_m + 64;                                    // [4][16]
    float* red_f = red_l + 64;                                    // [4][16] 2^(m_w - M)
    float* red_o = red_f + 64;                                    // [4][16][OS]
    const int g = lane >> 2, tq = lane & 3;
    if (tq == 0) {
        red_m[warp * 16 + g] = m[0]; red_m[warp * 16 + g + 8] = m[1];
        red_l[warp * 16 + g] = l[0]; red_l[warp * 16 + g + 8] = l[1];
    }
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) {
        *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + g) * OS + dn * 8 + tq * 2) = make_float2(O[dn][0], O[dn][1]);
        *reinterpret_cast<float2*>(red_o + ((size_t)warp * 16 + g + 8) * OS + dn * 8 + tq * 2) = make_float2(O[dn][2], O[dn][3]);
    }
    __syncthreads();
    if (threadIdx.x < 16) {
        const int row = threadIdx.x;
        float Mr = -INFINITY;
        for (int w = 0; w < 4; ++w) Mr = fmaxf(Mr, red_m[w * 16 + row]);
        const float ur = Mr == -INFINITY ? 0.0f : Mr;
        float Lr = 0.0f;
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(red_m[w * 16 + row] - ur);
            red_f[w * 16 + row] = f;
            Lr += red_l[w * 16 + row] * f;
        }
        res_m[row] = Mr;
        res_l[row] = Lr;
    }
    __syncthreads();
    // ... then the weighted sums
    for (int i = threadIdx.x; i < 16 * (HD / 4); i += ATT_THREADS) {
        const int row = i / (HD / 4), d = (i - row * (HD / 4)) * 4;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = red_f[w * 16 + row];
            const float4 v = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + row) * OS + d);
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        *reinterpret_cast<float4*>(res_o + (size_t)row * OS + d) = acc;
    }
    cluster.sync();                                               // every block's (m, l, O) is in place
    constexpr int DW = HD / CL;
    for (int i = threadIdx.x; i < rows_valid * DW; i += ATT_THREADS) {
        const int row = i / DW, d = rank * DW + (i - row * DW);
        float pm[CL], pl[CL], po[CL];
#pragma unroll
        for (int r = 0; r < CL; ++r) {
            const float* rm = cluster.map_shared_rank(res_m, r);
            pm[r] = rm[row];
            pl[r] = rm[16 + row];
            po[r] = rm[32 + (size_t)row * OS + d];
        }
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < CL; ++r) M = fmaxf(M, pm[r]);
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int r = 0; r < CL; ++r) {
            const float f = exp2f(pm[r] - M);                     // blocks without keys: exp2(-inf) = 0
            L += pl[r] * f;
            acc += po[r] * f;
        }
        const int h = kvh * group + qb * 16 + row;
        if (eff == 1) {
            out[((size_t)n * n_heads + h) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            float* dst = part + (((size_t)n * n_heads + h) * n_splits + split) * (HD + 2);
            dst[2 + d] = acc;
            if (d == 0) { dst[0] = M; dst[1] = L; }
        }
    }
    cluster.sync();                                               // nobody leaves while its memory is still read
}

// =======================================================================================
// prefill
// =======================================================================================
// tiles [n_tiles, 3] = (index of the tile's first token, number of rows (1..64), segment).  grid (n_tiles, n_heads).
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS)
prefill_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, bf16* __restrict__ out,
                         const int* __restrict__ tables, const int* __restrict__ tiles, const int* __restrict__ pos,
                         int n_heads, int n_kv_heads, int page_size, int page_shift, int max_blocks,
                         long long page_stride, long long kv_stride, int window, float scale2) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = TILE_KEYS * HD * 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // tiles later in a portion see more keys: start them first so that the short ones fill the tail
    // a tile of the list holds up to 128 rows; this block takes one half of 64
    const int slot = gridDim.x - 1 - blockIdx.x;
    const int tile = slot >> 1, half_rows = (slot & 1) * 64;
    const int n0 = tiles[tile * 3] + half_rows, seg = tiles[tile * 3 + 2];
    const int rows = tiles[tile * 3 + 1] - half_rows < 64 ? tiles[tile * 3 + 1] - half_rows : 64;
    if (rows <= 0) return;
    const int h = blockIdx.y;
    const int kvh = h / (n_heads / n_kv_heads);
    const int p0 = pos[n0];                                       // positions of a portion are consecutive
    const int p_last = p0 + rows - 1;
    const int lo_tile = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;

    CacheRef cr;
    cr.base = cache; cr.table = tables + (size_t)seg * max_blocks;
    cr.page_stride = page_stride; cr.kv_stride = kv_stride; cr.page_size = page_size; cr.page_shift = page_shift; cr.kvh = kvh;

    const uint32_t sQ = smem_u32(smem_raw);                      // [64][HD]
    const uint32_t sKV = sQ + TILE_BYTES;
    for (int i = threadIdx.x; i < 64 * (HD / 8); i += ATT_THREADS) {
        const int row = i / (HD / 8), c = i - row * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(n0 + row) * n_heads + h) * HD + c * 8);
        *reinterpret_cast<uint4*>(smem_raw + swz<HD>(row, c)) = v;
    }
    const int t_first = lo_tile / TILE_KEYS, t_last = p_last / TILE_KEYS;
    load_kv_tile<HD>(cr, sKV, sKV + TILE_BYTES, t_first * TILE_KEYS, lo_tile, p_last);
    cp_async_commit();
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                    sQ + swz<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    float O[HD / 8][4];
#pragma unroll
    for (int dn = 0; dn < HD / 8; ++dn) O[dn][0] = O[dn][1] = O[dn][2] = O[dn][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    // the two rows of this thread and what they may see
    const int g = lane >> 2;
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int hi0 = r0 < rows ? p0 + r0 : -1, hi1 = r1 < rows ? p0 + r1 : -1;      // padding rows see nothing
    const int lo0 = (window > 0 && hi0 - window + 1 > 0) ? hi0 - window + 1 : 0;
    const int lo1 = (window > 0 && hi1 - window + 1 > 0) ? hi1 - window + 1 : 0;
    // what this warp's 16 rows may see at most
    const int w_rows = rows - warp * 16;                         // rows of this warp that exist
    const int w_hi = p0 + warp * 16 + (w_rows < 16 ? w_rows : 16) - 1;
    const int w_lo = (window > 0 && p0 + warp * 16 - window + 1 > 0) ? p0 + warp * 16 - window + 1 : 0;

    for (int t = t_first; t <= t_last; ++t) {
        const int stage = (t - t_first) & 1;
        if (t + 1 <= t_last) {
            const uint32_t nb = sKV + (stage ^ 1) * 2 * TILE_BYTES;
            load_kv_tile<HD>(cr, nb, nb + TILE_BYTES, (t + 1) * TILE_KEYS, lo_tile, p_last);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t sK = sKV + stage * 2 * TILE_BYTES, sV = sK + TILE_BYTES;
        const int key0 = t * TILE_KEYS;
        if (w_rows > 0 && key0 <= w_hi && key0 + TILE_KEYS - 1 >= w_lo) {
            float S[8][4];
            qk_scores<HD, 8>(S, qf, sK, 0, lane);
            // every existing row of the warp sees the whole tile: rows sit at p0 + warp*16 .. w_hi
            const bool full = w_rows >= 16 && key0 + TILE_KEYS - 1 <= p0 + warp * 16 &&
                              (window <= 0 || key0 >= w_hi - window + 1);
            if (full) softmax_step<HD, 8, false>(S, O, m, l, key0, lane, lo0, hi0, lo1, hi1, scale2);
            else softmax_step<HD, 8, true>(S, O, m, l, key0, lane, lo0, hi0, lo1, hi1, scale2);
            pv_accumulate<HD, 8>(O, S, sV, 0, lane);
        }
        __syncthreads();
    }
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
    const int tq = lane & 3;
    if (r0 < rows) {
        const float inv = 1.0f / l[0];
        bf16* o = out + ((size_t)(n0 + r0) * n_heads + h) * HD;
#pragma unroll
        for (int dn = 0; dn < HD / 8; ++dn)
            *reinterpret_cast<uint32_t*>(o + dn * 8 + tq * 2) = pack_bf16(O[dn][0] * inv, O[dn][1] * inv);
    }
    if (r1 < rows) {
        const float inv = 1.0f / l[1];
        bf16* o = out + ((size_t)(n0 + r1) * n_heads + h) * HD;
#pragma unroll
        for (int dn = 0; dn < HD / 8; ++dn)
            *reinterpret_cast<uint32_t*>(o + dn * 8 + tq * 2) = pack_bf16(O[dn][2] * inv, O[dn][3] * inv);
    }
}

// =======================================================================================
// entry points
// =======================================================================================
static int page_shift_of(int page_size) {
    if (page_size > 0 && (page_size & (page_size - 1)) == 0) {
        int s = 0;
        while ((1 << s) < page_size) ++s;
        return s;
    }
    return -1;
}

static int check_common(const char* what, int n_heads, int n_kv_heads, int head_dim, int page_size, int max_blocks) {
    if (head_dim != 64 && head_dim != 128)
        return zi_fail("%s: the tensor-core kernels take head_dim 64 or 128, got %d (the general kernel takes the rest)", what, head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
        return zi_fail("%s: %d query heads cannot share %d key/value heads", what, n_heads, n_kv_heads);
    if (page_size <= 0 || max_blocks <= 0) return zi_fail("%s: page_size=%d max_blocks=%d", what, page_size, max_blocks);
    return 0;
}

template <typename K> static int set_smem(K kernel, size_t bytes, const char* what) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return zi_fail("%s: cannot reserve %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
    }
    return 0;
}

template <typename K, typename... Args>
static cudaError_t launch_cluster(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = DEC_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

ZI_EXPORT int zi_decode_attention(const void* q, const void* cache, void* out, const int* tables, const int* tok_seg,
                                  const int* pos, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                  int page_size, int max_blocks, long long page_stride, long long kv_stride,
                                  int window, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (check_common("decode_attention", n_heads, n_kv_heads, head_dim, page_size, max_blocks)) return 1;
    if (n_tokens > 65535) return zi_fail("decode_attention: %d tokens are more than one launch takes (65535)", n_tokens);
    const int group = n_heads / n_kv_heads, q_blocks = (group + 15) / 16;
    if (n_kv_heads * q_blocks > 65535) return zi_fail("decode_attention: too many head blocks for one launch");
    dim3 grid(DEC_CLUSTER, n_kv_heads * q_blocks, n_tokens);
    const float scale2 = scale * LOG2E;
    const int shift = page_shift_of(page_size);
    cudaError_t e;
    if (head_dim == 128) {
        const size_t smem = 16 * 128 * 2 + DEC_STAGES * 2 * TILE_KEYS * 128 * 2 + (32 + 16 * (128 + 8)) * 4;
        if (set_smem(decode_attention_kernel<128>, smem, "decode_attention")) return 1;
        e = launch_cluster(decode_attention_kernel<128>, grid, dim3(ATT_THREADS), smem, stream,
                           (const bf16*)q, (const bf16*)cache, (bf16*)out, tables, tok_seg, pos, n_heads, n_kv_heads,
                           q_blocks, page_size, shift, max_blocks, page_stride, kv_stride, window, scale2);
    } else {
        const size_t smem = 16 * 64 * 2 + DEC_STAGES * 2 * TILE_KEYS * 64 * 2 + (32 + 16 * (64 + 8)) * 4;
        if (set_smem(decode_attention_kernel<64>, smem, "decode_attention")) return 1;
        e = launch_cluster(decode_attention_kernel<64>, grid, dim3(ATT_THREADS), smem, stream,
                           (const bf16*)q, (const bf16*)cache, (bf16*)out, tables, tok_seg, pos, n_heads, n_kv_heads,
                           q_blocks, page_size, shift, max_blocks, page_stride, kv_stride, window, scale2);
    }
    if (e != cudaSuccess) { cudaGetLastError(); return zi_fail("decode_attention: launch failed: %s", cudaGetErrorString(e)); }
    return zi_check_launch("decode_attention");
}

// The same with tiles by TMA.  n_pages: pages in the pool (the extent of the tensor map); status: one int of device
// memory, zero before; 31 afterwards means a bounded wait for a tile ran out and the output is not valid.
template <int HD, int KEYS>
static size_t dt_smem() { return 4 * DT_STAGES * 2 * KEYS * HD * 2 + 16 * HD * 2 + 4 * DT_STAGES * 8 + (32 + 16 * (HD + 8)) * 4; }

// clusters of eight blocks of the kernel that the device holds at once (a cluster needs its SMs inside one GPC);
// asked once
template <int HD, int KEYS>
static int dt_max_clusters() {
    static int cached = 0;
    if (cached) return cached;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = DEC_CLUSTER; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cfg.gridDim = dim3(DEC_CLUSTER, 64, 1); cfg.blockDim = dim3(ATT_THREADS); cfg.dynamicSmemBytes = dt_smem<HD, KEYS>();
    if (set_smem(decode_attention_tma_kernel<HD, KEYS, DEC_CLUSTER>, cfg.dynamicSmemBytes, "decode_attention_tma")) return -1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, decode_attention_tma_kernel<HD, KEYS, DEC_CLUSTER>, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
    cached = n > 0 ? n : -1;
    return cached;
}

struct DtArgs {
    const CUtensorMap* mkv; const void* q; void* out; const int* tables; const int* tok_seg; const int* pos; int* status;
    int n_tokens, n_heads, n_kv_heads, q_blocks, page_size, box_rows, max_blocks, window; float scale2; cudaStream_t stream;
    int n_splits, min_split_tiles; float* part; int kv_box;
};

template <int HD, int KEYS, int CL>
static cudaError_t dt_launch(const DtArgs& a) {
    if (set_smem(decode_attention_tma_kernel<HD, KEYS, CL>, dt_smem<HD, KEYS>(), "decode_attention_tma")) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // Few blocks: the kernel may start while its predecessor still runs (see dependent_wait() in the kernel).  Measured
    // on the 1.5B-class decode step: 1.32 -> 1.28 ms at batch 1, 1.42 -> 1.40 at 8, 1.74 -> 1.70 at 12; with 16
    // requests (256 blocks) the early blocks get in the predecessor's way, 1.80 -> 1.90 ms, so those wait their turn.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    const long long blocks = (long long)CL * a.n_kv_heads * a.q_blocks * a.n_splits * a.n_tokens;
    cfg.attrs = attr; cfg.numAttrs = blocks <= 200 ? 2 : 1;
    cfg.gridDim = dim3(CL, a.n_kv_heads * a.q_blocks * a.n_splits, a.n_tokens); cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = dt_smem<HD, KEYS>(); cfg.stream = a.stream;
    return cudaLaunchKernelEx(&cfg, decode_attention_tma_kernel<HD, KEYS, CL>, *a.mkv, (const bf16*)a.q, (bf16*)a.out, a.tables,
                              a.tok_seg, a.pos, a.status, a.n_heads, a.n_kv_heads, a.q_blocks, a.page_size, a.box_rows,
                              a.max_blocks, a.window, a.scale2, a.n_splits, a.min_split_tiles, a.part, a.kv_box);
}
template <int HD>
static cudaError_t dt_dispatch(const DtArgs& a, int keys, int cl) {
    if (keys == 32) return dt_launch<HD, 32, DEC_CLUSTER>(a);
    switch (cl) {
        case 8: return dt_launch<HD, 16, 8>(a);
        case 4: return dt_launch<HD, 16, 4>(a);
        case 2: return dt_launch<HD, 16, 2>(a);
        default: return dt_launch<HD, 16, 1>(a);
    }
}

// How a step's decode attention is laid out: tiles of 32 or 16 keys, blocks per cluster, clusters per (request,
// key/value head).
//   A (request, key/value head) is one unit of work.  Few units: clusters of eight blocks share a unit's keys, in
//   tiles of 32 keys while all clusters fit on the device at once, else of 16 (two blocks to an SM).  More units
//   fill the device by themselves: the cluster is then the largest of 8, 4, 2, 1 with which all blocks still run
//   at once, so that a block's fixed cost (start, merge of its warps, cluster exchange) is spread over more keys.
//   Measured at 1,100 cached tokens, 4 key/value heads: 48 requests 47 us with clusters of 8, 25 us with single
//   blocks; 16 requests 15 us with 8, 10 us with 4.
//   Very few units with long contexts leave most of the device idle (one request of 2 key/value heads and 32,768
//   tokens: 16 blocks, 0.8 TB/s): then several clusters share a unit, each taking at least DT_SPLIT_KEYS keys, as
//   far as the longest context of the step (max_kv_len) and the free SMs allow, and a second kernel adds their
//   parts.  That second kernel costs a step of 28 layers about 0.07 ms even when no request is long enough to be
//   shared (measured: 1.25 -> 1.32 ms at 8 requests), so a launch whose max_kv_len stays below DT_SPLIT_FROM plans
//   none; one request of 8,192 tokens: 1.43 ms a step with clusters of 4,096 keys, 1.27 with clusters of 1,024.
#define DT_MAX_SPLITS 16
struct DtPlan { int keys, cl, splits, min_split_tiles; };
static int dt_plan(DtPlan* p, int n_tokens, int n_kv_heads, int q_blocks, int head_dim, int max_kv_len) {
    const long long units = (long long)n_kv_heads * q_blocks * n_tokens;
    const int fit32 = head_dim == 128 ? dt_max_clusters<128, 32>() : dt_max_clusters<64, 32>();
    static int slots = 0;                                         // blocks of the 16-key form that run at once: two to an SM
    if (slots == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        slots = 2 * (sms > 0 ? sms : 1);
    }
    int cl = 8;
    while (cl > 1 && units * cl > slots) cl >>= 1;
    long long splits = max_kv_len < DT_SPLIT_FROM ? 1 : max_kv_len / DT_SPLIT_KEYS;
    if (splits > slots / (units * cl)) splits = slots / (units * cl);
    if (splits > DT_MAX_SPLITS) splits = DT_MAX_SPLITS;
    if (splits < 2) splits = 1;
    p->keys = (fit32 > 0 && units * splits <= fit32) ? 32 : 16;
    p->cl = cl;
    p->splits = (int)splits;
    p->min_split_tiles = DT_SPLIT_KEYS / p->keys;
    return 0;
}

// The number of cached tokens from which a launch may let several clusters share a request (and then runs the
// kernel that adds their parts): a caller that knows its requests stay below passes a smaller max_kv_len.
ZI_EXPORT int zi_decode_attention_tma_split_from() { return DT_SPLIT_FROM; }

// Floats of scratch a call needs for the parts of clusters that share a request (0: none).
ZI_EXPORT long long zi_decode_attention_tma_part_floats(int n_tokens, int n_heads, int n_kv_heads, int head_dim, int max_kv_len) {
    if (n_tokens <= 0 || n_heads <= 0 || n_kv_heads <= 0 || (head_dim != 64 && head_dim != 128) || tc_init()) return 0;
    DtPlan p;
    dt_plan(&p, n_tokens, n_kv_heads, (n_heads / n_kv_heads + 15) / 16, head_dim, max_kv_len);
    return p.splits > 1 ? (long long)n_tokens * n_heads * p.splits * (head_dim + 2) : 0;
}

// max_kv_len: an upper bound of the cached tokens of the step's requests (decides how many clusters may share one
// request); part / part_floats: scratch as zi_decode_attention_tma_part_floats says, may be null when that is 0.
ZI_EXPORT int zi_decode_attention_tma(const void* q, const void* cache, void* out, const int* tables, const int* tok_seg,
                                      const int* pos, int* status, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                      int page_size, int max_blocks, long long n_pages, long long page_stride,
                                      long long kv_stride, int window, float scale, int max_kv_len, float* part,
                                      long long part_floats, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (check_common("decode_attention_tma", n_heads, n_kv_heads, head_dim, page_size, max_blocks)) return 1;
    if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1))) return zi_fail("decode_attention_tma: page size %d is not a power of two from 8 to 128", page_size);
    if (n_tokens > 65535) return zi_fail("decode_attention_tma: %d tokens are more than one launch takes (65535)", n_tokens);
    if (((uintptr_t)q | (uintptr_t)cache) & 15) return zi_fail("decode_attention_tma: q and cache must be 16-byte aligned");
    if ((page_stride | kv_stride) & 7) return zi_fail("decode_attention_tma: cache strides must be multiples of 8 elements");
    if (!status) return zi_fail("decode_attention_tma: a status word is required");
    const int group = n_heads / n_kv_heads, q_blocks = (group + 15) / 16;
    if (tc_init()) return 1;
    DtPlan plan;
    dt_plan(&plan, n_tokens, n_kv_heads, q_blocks, head_dim, max_kv_len);
    if (plan.splits > 1) {
        const long long need = (long long)n_tokens * n_heads * plan.splits * (head_dim + 2);
        if (!part || part_floats < need) return zi_fail("decode_attention_tma: %d clusters share a request and need %lld floats of scratch, got %lld", plan.splits, need, part ? part_floats : 0LL);
    }
    if ((long long)n_kv_heads * q_blocks * plan.splits > 65535) return zi_fail("decode_attention_tma: too many head blocks for one launch");
    const int keys = plan.keys;
    const int box_rows = page_size < keys ? page_size : keys;
    const int kv_box = box_rows == keys ? 1 : 0;                  // a tile lies in one page: keys and values in one box
    CUtensorMap mkv;
    if (tc_map_kv_pages(&mkv, cache, head_dim, page_size, n_kv_heads, n_pages, page_stride, kv_stride, box_rows, kv_box ? 2 : 1)) return 1;
    DtArgs a = {&mkv, q, out, tables, tok_seg, pos, status, n_tokens, n_heads, n_kv_heads, q_blocks, page_size, box_rows,
                max_blocks, window, scale * LOG2E, stream, plan.splits, plan.min_split_tiles, part, kv_box};
    cudaError_t e = head_dim == 128 ? dt_dispatch<128>(a, keys, plan.cl) : dt_dispatch<64>(a, keys, plan.cl);
    if (e != cudaSuccess) { cudaGetLastError(); return zi_fail("decode_attention_tma: launch failed: %s", cudaGetErrorString(e)); }
    if (plan.splits > 1) {
        const dim3 grid(n_tokens, n_heads);
        if (head_dim == 128) decode_attention_merge_kernel<128><<<grid, 128, 0, stream>>>(part, (bf16*)out, pos, n_heads, window, keys, plan.splits, plan.min_split_tiles);
        else decode_attention_merge_kernel<64><<<grid, 64, 0, stream>>>(part, (bf16*)out, pos, n_heads, window, keys, plan.splits, plan.min_split_tiles);
    }
    return zi_check_launch("decode_attention_tma");
}

ZI_EXPORT int zi_prefill_attention(const void* q, const void* cache, void* out, const int* tables, const int* tiles,
                                   const int* pos, int n_tiles, int n_heads, int n_kv_heads, int head_dim,
                                   int page_size, int max_blocks, long long page_stride, long long kv_stride,
                                   int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (check_common("prefill_attention", n_heads, n_kv_heads, head_dim, page_size, max_blocks)) return 1;
    if (n_heads > 65535) return zi_fail("prefill_attention: %d heads are more than one launch takes", n_heads);
    dim3 grid(2 * n_tiles, n_heads);          // two 64-row halves per tile of the list
    const float scale2 = scale * LOG2E;
    const int shift = page_shift_of(page_size);
    if (head_dim == 128) {
        const size_t smem = 5 * TILE_KEYS * 128 * 2;
        if (set_smem(prefill_attention_kernel<128>, smem, "prefill_attention")) return 1;
        prefill_attention_kernel<128><<<grid, ATT_THREADS, smem, stream>>>(
            (const bf16*)q, (const bf16*)cache, (bf16*)out, tables, tiles, pos, n_heads, n_kv_heads, page_size, shift,
            max_blocks, page_stride, kv_stride, window, scale2);
    } else {
        const size_t smem = 5 * TILE_KEYS * 64 * 2;
        if (set_smem(prefill_attention_kernel<64>, smem, "prefill_attention")) return 1;
        prefill_attention_kernel<64><<<grid, ATT_THREADS, smem, stream>>>(
            (const bf16*)q, (const bf16*)cache, (bf16*)out, tables, tiles, pos, n_heads, n_kv_heads, page_size, shift,
            max_blocks, page_stride, kv_stride, window, scale2);
    }
    return zi_check_launch("prefill_attention");
}
