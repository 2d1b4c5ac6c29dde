// C[M,N] = X[M,K] . W[N,K]^T (+ bias[N]) for few rows (M <= 16: decode steps), bfloat16 operands,
// float32 accumulation on the tensor cores (mma.sync m16n8k16), output bfloat16 or float32.
//
// The product is bound by reading W once.  Roles are swapped: 16 rows of W are the "A" tile of the
// MMA and 8 tokens its "N" side, so a decode batch of 8 fills an instruction exactly.  Weights go
// from global memory straight into MMA fragments, no shared memory in between: a thread loads 16
// contiguous bytes (8 k-values) of weight rows g and g+8 and treats them as the k-slots its lane owns
// in two consecutive k16 steps; the activations are loaded with the same assignment, and since a dot
// product does not care in which order k is walked, the result is the plain product.  Per 32
// k-values a warp reads 64 contiguous bytes of each of its 16 rows.
//
// One thread block owns 16 output columns (rows of W) over all of K; its 8 warps take interleaved
// k-steps (warp w: steps w, w+8, ...) and their partial sums are added in warp order through shared
// memory: no atomics, the same bits every time, and a token's result does not depend on the batch.
//
// ACT_SILU_MUL variant: W holds gate rows and up rows ([2*I, K], gate first); the block computes
// both for its 16 columns and writes up * gate / (1 + exp(-gate)): the feed-forward's activation
// never makes a round trip through memory.
#define ZI_PDL_BIT 2
#include "zi_common.cuh"
#include <cooperative_groups.h>

ZI_DEFINE_LAST_ERROR(gemm_smallm)

#define GS_WARPS 8
#define GS_THREADS (GS_WARPS * 32)
#define GS_UNROLL 4

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {
    // weights are read once: do not keep them in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Accumulate 16 rows of W (starting at `row0`, clamped to n_rows) against NT*8 tokens over this warp's k-steps.
// first_pass: the first weight loads are issued before pdl_wait(), so that they overlap with the tail of the
// kernel that produces X.
template <int NT>
__device__ __forceinline__ void accumulate_rows(float (&acc)[NT][4], const bf16* __restrict__ W, const bf16* __restrict__ X,
                                                int row0, int n_rows, int M, int step_begin, int step_end,
                                                long long ldw, long long ldx, int warp, int lane, bool first_pass,
                                                int pair = 8) {
    // pair: distance between the two groups of 8 weight rows a block works on (8: sixteen consecutive rows)
    const int g = lane >> 2, tq = lane & 3;
    const int r0 = min(row0 + g, n_rows - 1), r1 = min(row0 + g + pair, n_rows - 1);
    const bf16* w0 = W + (long long)r0 * ldw + tq * 8;
    const bf16* w1 = W + (long long)r1 * ldw + tq * 8;
    const bf16* xp[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xp[nt] = X + (long long)min(nt * 8 + g, M - 1) * ldx + tq * 8;
    const int steps = step_end;
    int s = step_begin + warp;
    bool waited = !first_pass;
    for (; s + (GS_UNROLL - 1) * GS_WARPS < steps; s += GS_UNROLL * GS_WARPS) {
        uint4 a[GS_UNROLL], b[GS_UNROLL];
#pragma unroll
        for (int u = 0; u < GS_UNROLL; ++u) {
            const int k = (s + u * GS_WARPS) * 32;
            a[u] = ldg_stream(w0 + k);
            b[u] = ldg_stream(w1 + k);
        }
        if (!waited) { pdl_wait(); waited = true; }
        if constexpr (NT == 1) {
            // The activations of the whole batch are asked for before the first product needs one: a load that
            // stands only where its value is used puts an L2 round trip in front of every pair of products, during
            // which the warp has no weight load in flight.  Measured at 8 rows: the 7B-class gate/up product
            // 50 -> 45 us, its down product 35 -> 29 us.  (With 16 tokens the same change made it slower.)
            uint4 x[GS_UNROLL];
#pragma unroll
            for (int u = 0; u < GS_UNROLL; ++u) x[u] = ld_dep16(xp[0] + (s + u * GS_WARPS) * 32);
#pragma unroll
            for (int u = 0; u < GS_UNROLL; ++u) {
                mma_bf16_16816(acc[0], a[u].x, b[u].x, a[u].y, b[u].y, x[u].x, x[u].y);
                mma_bf16_16816(acc[0], a[u].z, b[u].z, a[u].w, b[u].w, x[u].z, x[u].w);
            }
        } else {
#pragma unroll
            for (int u = 0; u < GS_UNROLL; ++u) {
                const int k = (s + u * GS_WARPS) * 32;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 x = ld_dep16(xp[nt] + k);
                    mma_bf16_16816(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, x.x, x.y);
                    mma_bf16_16816(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, x.z, x.w);
                }
            }
        }
    }
    if constexpr (NT == 1) {
        // the up to GS_UNROLL - 1 steps that are left go as one batch too: one trip to memory, not one per step
        if (s < steps) {
            uint4 a[GS_UNROLL - 1], b[GS_UNROLL - 1], x[GS_UNROLL - 1];
#pragma unroll
            for (int u = 0; u < GS_UNROLL - 1; ++u) {
                if (s + u * GS_WARPS < steps) {
                    const int k = (s + u * GS_WARPS) * 32;
                    a[u] = ldg_stream(w0 + k);
                    b[u] = ldg_stream(w1 + k);
                }
            }
            if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
            for (int u = 0; u < GS_UNROLL - 1; ++u)
                if (s + u * GS_WARPS < steps) x[u] = ld_dep16(xp[0] + (s + u * GS_WARPS) * 32);
#pragma unroll
            for (int u = 0; u < GS_UNROLL - 1; ++u) {
                if (s + u * GS_WARPS < steps) {
                    mma_bf16_16816(acc[0], a[u].x, b[u].x, a[u].y, b[u].y, x[u].x, x[u].y);
                    mma_bf16_16816(acc[0], a[u].z, b[u].z, a[u].w, b[u].w, x[u].z, x[u].w);
                }
            }
        }
    } else {
        for (; s < steps; s += GS_WARPS) {
            const int k = s * 32;
            const uint4 a = ldg_stream(w0 + k), b = ldg_stream(w1 + k);
            if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 x = ld_dep16(xp[nt] + k);
                mma_bf16_16816(acc[nt], a.x, b.x, a.y, b.y, x.x, x.y);
                mma_bf16_16816(acc[nt], a.z, b.z, a.w, b.w, x.z, x.w);
            }
        }
    }
    if (!waited) pdl_wait();
}

// Fragment bookkeeping: a thread's 16 bytes of row g are e0..e7.  First MMA: a0 = (e0,e1) = .x for row g,
// a1 = .x of row g+8, a2 = (e2,e3) = .y for row g, a3 = .y of row g+8; b0 = x.x, b1 = x.y.  Second MMA: .z/.w.
// Slot (tq*2, tq*2+1) of A meets slot (tq*2, tq*2+1) of B and slot (tq*2+8, +9) meets (tq*2+8, +9): each
// pairs weight and activation of the same k.

template <int NT, typename TC, bool SILU_MUL>
__global__ void __launch_bounds__(GS_THREADS, NT == 1 ? 4 : 3)
gemm_smallm_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                   TC* __restrict__ C, float* __restrict__ part, int* __restrict__ counters, int M, int N, int K,
                   long long ldx, long long ldw, long long ldc, int cluster_reduce) {
    // N: number of output columns.  With SILU_MUL, W has 2*N rows (gate rows, then up rows).
    // gridDim.y > 1: K is cut into gridDim.y ranges, one block each; the blocks of a column tile leave their
    // sums in `part` [gridDim.y][16][N] and the last one to arrive adds them in range order.
    __shared__ float red[SILU_MUL ? 2 : 1][GS_WARPS][16][NT * 8 + 1];
    __shared__ int is_last;
    __shared__ float tile_sum[16][NT * 8 + 1];      // cluster_reduce: this block's sums, read by the first block of the cluster
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = blockIdx.x * 16;
    const int ksplit = gridDim.y, ks = blockIdx.y;
    const int steps = K / 32, per = (steps + ksplit - 1) / ksplit;
    const int step_begin = ks * per, step_end = min(steps, step_begin + per);
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    pdl_trigger_early();
    accumulate_rows<NT>(acc, W, X, row0, N, M, step_begin, step_end, ldw, ldx, warp, lane, true);
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[0][warp][g][nt * 8 + tq * 2] = acc[nt][0];
        red[0][warp][g][nt * 8 + tq * 2 + 1] = acc[nt][1];
        red[0][warp][g + 8][nt * 8 + tq * 2] = acc[nt][2];
        red[0][warp][g + 8][nt * 8 + tq * 2 + 1] = acc[nt][3];
    }
    if (SILU_MUL) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        accumulate_rows<NT>(acc, W + (long long)N * ldw, X, row0, N, M, step_begin, step_end, ldw, ldx, warp, lane, false);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[SILU_MUL ? 1 : 0][warp][g][nt * 8 + tq * 2] = acc[nt][0];
            red[SILU_MUL ? 1 : 0][warp][g][nt * 8 + tq * 2 + 1] = acc[nt][1];
            red[SILU_MUL ? 1 : 0][warp][g + 8][nt * 8 + tq * 2] = acc[nt][2];
            red[SILU_MUL ? 1 : 0][warp][g + 8][nt * 8 + tq * 2 + 1] = acc[nt][3];
        }
    }
    pdl_trigger_late();
    __syncthreads();
    namespace cg = cooperative_groups;
    if (ksplit > 1 && cluster_reduce) {
        // The blocks of a column tile are one thread-block cluster (launched so): each leaves its sums in its own
        // shared memory, and the first adds them in range order through distributed shared memory.  Against the way
        // through global memory below this saves a fence, an atomic round trip and a read back from L2.
        for (int i = threadIdx.x; i < 16 * NT * 8; i += GS_THREADS) {
            const int r = i % 16, m = i / 16;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) v += red[0][w][r][m];
            tile_sum[r][m] = v;
        }
        cg::this_cluster().sync();
        if (ks != 0) {
            cg::this_cluster().sync();                  // stay until the first block has read
            return;
        }
    } else if (ksplit > 1) {
        // leave this block's sums, then find out whether it is the last of its column tile
        for (int i = threadIdx.x; i < 16 * NT * 8; i += GS_THREADS) {
            const int r = i % 16, m = i / 16;
            if (row0 + r >= N || m >= M) continue;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) v += red[0][w][r][m];
            part[((size_t)ks * 16 + m) * N + row0 + r] = v;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int prev = atomicAdd(&counters[blockIdx.x], 1);
            is_last = (prev == ksplit - 1);
            if (is_last) counters[blockIdx.x] = 0;          // ready for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
    }
    for (int i = threadIdx.x; i < 16 * NT * 8; i += GS_THREADS) {
        const int r = i % 16, m = i / 16;             // consecutive threads -> consecutive output columns
        const int n = row0 + r;
        if (n >= N || m >= M) continue;
        float v = 0.0f;
        if (ksplit > 1 && cluster_reduce) {
            for (int k2 = 0; k2 < ksplit; ++k2) v += cg::this_cluster().map_shared_rank(&tile_sum[0][0], k2)[r * (NT * 8 + 1) + m];
        } else if (ksplit > 1) {
            for (int k2 = 0; k2 < ksplit; ++k2) v += ld_l2(part + ((size_t)k2 * 16 + m) * N + n);
        } else {
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) v += red[0][w][r][m];
        }
        if (SILU_MUL) {
            float u = 0.0f;
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) u += red[SILU_MUL ? 1 : 0][w][r][m];
            // the unfused path rounds gate and up to bfloat16 before the activation; do the same
            const float gr = __bfloat162float(__float2bfloat16_rn(v)), ur = __bfloat162float(__float2bfloat16_rn(u));
            v = ur * gr / (1.0f + expf(-gr));
        } else if (bias) {
            v += __bfloat162float(bias[n]);
        }
        C[(long long)m * ldc + n] = from_f32<TC>(v);
    }
    if (ksplit > 1 && cluster_reduce) cg::this_cluster().sync();
}

template <int NT, typename TC, bool SILU>
static void launch(const void* X, const void* W, const void* bias, void* C, float* part, int* counters, int ksplit,
                   int M, int N, int K, long long ldx, long long ldw, long long ldc, cudaStream_t stream,
                   bool through_clusters = true) {
    if (through_clusters && ksplit > 1 && ksplit <= 8) {
        // the K ranges of a column tile as one cluster along y: their sums meet in distributed shared memory
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((N + 15) / 16, ksplit);
        cfg.blockDim = dim3(GS_THREADS);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = ksplit; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, gemm_smallm_kernel<NT, TC, SILU>, (const bf16*)X, (const bf16*)W, (const bf16*)bias, (TC*)C,
                               part, counters, M, N, K, ldx, ldw, ldc, 1) == cudaSuccess) return;
        cudaGetLastError();                             // no cluster of that shape here: the way through global memory
    }
    zi_launch(gemm_smallm_kernel<NT, TC, SILU>, dim3((N + 15) / 16, ksplit), dim3(GS_THREADS), 0, stream,
              (const bf16*)X, (const bf16*)W, (const bf16*)bias, (TC*)C, part, counters, M, N, K, ldx, ldw, ldc, 0);
}

// How many ranges K is cut into: a function of the weight's shape only.  Few column tiles (narrow outputs)
// would leave most of the GPU idle, so their K is shared out until about two blocks per SM exist.
ZI_EXPORT int zi_gemm_smallm_ksplit(int N, int K, int silu_mul) {
    const int tiles = (N + 15) / 16, steps = K / 32;
    if (silu_mul || tiles >= 296) return 1;
    int ks = (296 + tiles - 1) / tiles;
    if (ks > 8) ks = 8;
    // a split costs a cluster exchange: keep 6 k-steps per warp (K = 1,536 stays whole: 3.9 us against 4.4 us cut in
    // two; K = 3,584 is cut in two: 7.6 us against 8.5 us whole)
    while (ks > 1 && steps / ks < 6 * GS_WARPS) --ks;
    return ks < 1 ? 1 : ks;
}

// Scratch the split needs: floats of `part` and ints of `counters` (zero before the first launch; the
// kernel leaves them zero).
ZI_EXPORT long long zi_gemm_smallm_part_floats(int N, int K, int silu_mul) {
    const int ks = zi_gemm_smallm_ksplit(N, K, silu_mul);
    return ks > 1 ? (long long)ks * 16 * N : 0;
}
ZI_EXPORT int zi_gemm_smallm_counter_ints(int N) { return (N + 15) / 16; }

ZI_EXPORT int zi_gemm_smallm_max_rows() { return 16; }

// silu_mul != 0: W is [2*N, K] (gate rows then up rows), C[m, n] = up * silu(gate); bias must be null.
ZI_EXPORT int zi_gemm_smallm(const void* X, const void* W, const void* bias, void* C, int c_dtype, float* part,
                             int* counters, int M, int N, int K, long long ldx, long long ldw, long long ldc,
                             int silu_mul, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16) return zi_fail("gemm_smallm: M=%d rows; this kernel takes at most 16", M);
    if (K <= 0 || K % 32 != 0) return zi_fail("gemm_smallm: K=%d must be a positive multiple of 32", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_smallm: row strides (%lld, %lld) must be multiples of 8 elements", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_smallm: operands must be 16-byte aligned");
    if (silu_mul && bias) return zi_fail("gemm_smallm: the fused activation takes no bias");
    if (c_dtype != ZI_F32 && c_dtype != ZI_BF16) return zi_fail("gemm_smallm: unknown output dtype %d", c_dtype);
    const bool f32 = c_dtype == ZI_F32;
    const int ksplit = zi_gemm_smallm_ksplit(N, K, silu_mul);
    if (ksplit > 1 && (!part || !counters)) return zi_fail("gemm_smallm: N=%d K=%d is split %d ways and needs scratch", N, K, ksplit);
    if (silu_mul) {
        if (M <= 8) { if (f32) launch<1, float, true>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); else launch<1, bf16, true>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); }
        else        { if (f32) launch<2, float, true>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); else launch<2, bf16, true>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); }
    } else {
        if (M <= 8) { if (f32) launch<1, float, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); else launch<1, bf16, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); }
        else        { if (f32) launch<2, float, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); else launch<2, bf16, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream); }
    }
    return zi_check_launch("gemm_smallm");
}

// ---------------------------------------------------------------------------------------------------------
// The q/k/v product of a decode step with the rotation by position and the append to the cache in its
// epilogue: the projected q, k and v never make a round trip through memory and the step has one kernel less.
//   W [(n_heads + 2 n_kv_heads) * head_dim, K]: q heads, then k heads, then v heads.
// A block takes 8 dimensions d..d+7 of one head and the 8 that pair with them under rotate-half (d + half ..):
// its sixteen weight rows are two groups of eight, `half` apart.  cs [M, head_dim] holds cos (first half) and sin
// (second half) of every token's angles, made once per step for all layers.  The sums are rounded to bfloat16
// before the rotation, as the separate kernels do, and the rotation uses the same explicit roundings, so both
// ways give the same bits.
// ---------------------------------------------------------------------------------------------------------
struct RopeOut {
    const float* cs;
    bf16* q_out;
    bf16* cache;
    const int* tables;
    const int* tok_seg;
    const int* pos;
    int n_heads, n_kv_heads, head_dim, page_size, max_blocks;
    long long page_stride, kv_stride;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}

template <int NT>
__global__ void __launch_bounds__(GS_THREADS, NT == 1 ? 4 : 3)
gemm_smallm_rope_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                        const RopeOut ro, int M, int K, long long ldx, long long ldw) {
    __shared__ float red[GS_WARPS][16][NT * 8 + 1];
    __shared__ int s_page[NT * 8], s_off[NT * 8];
    __shared__ __align__(16) float s_cs[NT * 8][16];         // per token: cos of this block's 8 columns | sin of them
    __shared__ __align__(16) bf16 s_bias[2][8];              // bias of the 8 columns and of the 8 that pair with them
    // The decode attention kernel that follows may start now: it keeps away from what this kernel writes until it
    // has waited for it to finish (dependent_wait() there).  Without such a successor this does nothing.
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int half = ro.head_dim >> 1, tiles_per_head = half >> 3;
    const int head = blockIdx.x / tiles_per_head, d0 = (blockIdx.x - head * tiles_per_head) * 8;
    const int row0 = head * ro.head_dim + d0;
    const int n_rows = (ro.n_heads + 2 * ro.n_kv_heads) * ro.head_dim;
    if (threadIdx.x < M) {          // where each token's k and v go: asked for now, needed after the product
        const int p = ro.pos[threadIdx.x];
        s_page[threadIdx.x] = ro.tables[(size_t)ro.tok_seg[threadIdx.x] * ro.max_blocks + p / ro.page_size];
        s_off[threadIdx.x] = p % ro.page_size;
    }
    // So are the angles and the bias of this block's columns: copied into shared memory behind the product's back
    // (16 bytes a copy) instead of being fetched when the sums are ready, one more trip to memory at the kernel's end.
    {
        const int t = (int)threadIdx.x - 64;                // warps 2 and up: the first two ask for pages above
        if (t >= 0 && t < M * 4) {
            const int m = t >> 2, part = t & 3;             // cos low, cos high, sin low, sin high
            const float* src = ro.cs + (size_t)m * ro.head_dim + (part < 2 ? 0 : half) + d0 + (part & 1) * 4;
            cp_async16(&s_cs[m][part * 4], src);
        } else if (bias && t >= M * 4 && t < M * 4 + 2) {
            const int which = t - M * 4;
            cp_async16(&s_bias[which][0], bias + row0 + (which ? half : 0));
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    accumulate_rows<NT>(acc, W, X, row0, n_rows, M, 0, K / 32, ldw, ldx, warp, lane, false, half);
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][nt * 8 + tq * 2] = acc[nt][0];
        red[warp][g][nt * 8 + tq * 2 + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + tq * 2] = acc[nt][2];
        red[warp][g + 8][nt * 8 + tq * 2 + 1] = acc[nt][3];
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    for (int i = threadIdx.x; i < 8 * NT * 8; i += GS_THREADS) {
        const int rr = i & 7, m = i >> 3;
        if (m >= M) continue;
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) { a += red[w][rr][m]; b += red[w][rr + 8][m]; }
        const int d = d0 + rr;
        if (bias) { a += __bfloat162float(s_bias[0][rr]); b += __bfloat162float(s_bias[1][rr]); }
        a = __bfloat162float(__float2bfloat16_rn(a));
        b = __bfloat162float(__float2bfloat16_rn(b));
        float lo = a, hi = b;
        if (head < ro.n_heads + ro.n_kv_heads) {
            const float c = s_cs[m][rr], sn = s_cs[m][8 + rr];
            lo = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            hi = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
        }
        bf16* dst;
        if (head < ro.n_heads) {
            dst = ro.q_out + ((size_t)m * ro.n_heads + head) * ro.head_dim;
        } else {
            const bool is_v = head >= ro.n_heads + ro.n_kv_heads;
            const int kh = head - ro.n_heads - (is_v ? ro.n_kv_heads : 0);
            dst = ro.cache + (size_t)s_page[m] * ro.page_stride + (is_v ? ro.kv_stride : 0) +
                  ((size_t)kh * ro.page_size + s_off[m]) * ro.head_dim;
        }
        dst[d] = __float2bfloat16_rn(lo);
        dst[d + half] = __float2bfloat16_rn(hi);
    }
}

// cs: float32 [M, head_dim] (cos | sin per token, see zi_rope_table); tables [segments, max_blocks]; the cache is one
// call's slice of the pool.  bias may be null.
ZI_EXPORT int zi_gemm_smallm_rope(const void* X, const void* W, const void* bias, const float* cs, void* q_out, void* cache,
                                  const int* tables, const int* tok_seg, const int* pos, int M, int K, long long ldx,
                                  long long ldw, int n_heads, int n_kv_heads, int head_dim, int page_size, int max_blocks,
                                  long long page_stride, long long kv_stride, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (M > 16) return zi_fail("gemm_smallm_rope: M=%d rows; this kernel takes at most 16", M);
    if (K <= 0 || K % 32 != 0) return zi_fail("gemm_smallm_rope: K=%d must be a positive multiple of 32", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_smallm_rope: row strides (%lld, %lld) must be multiples of 8 elements", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_smallm_rope: operands must be 16-byte aligned");
    if (head_dim <= 0 || head_dim % 16) return zi_fail("gemm_smallm_rope: head_dim=%d must be a positive multiple of 16", head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || max_blocks <= 0) return zi_fail("gemm_smallm_rope: bad head counts, page size or table width");
    if (!cs || !q_out || !cache || !tables || !tok_seg || !pos) return zi_fail("gemm_smallm_rope: a null pointer among cs, q_out, cache, tables, tok_seg, pos");
    RopeOut ro;
    ro.cs = cs; ro.q_out = (bf16*)q_out; ro.cache = (bf16*)cache; ro.tables = tables; ro.tok_seg = tok_seg; ro.pos = pos;
    ro.n_heads = n_heads; ro.n_kv_heads = n_kv_heads; ro.head_dim = head_dim; ro.page_size = page_size; ro.max_blocks = max_blocks;
    ro.page_stride = page_stride; ro.kv_stride = kv_stride;
    if (((uintptr_t)cs & 15) || ((uintptr_t)bias & 15)) return zi_fail("gemm_smallm_rope: cs and bias must be 16-byte aligned (they are copied 16 bytes at a time)");
    const long long tiles = (long long)(n_heads + 2 * n_kv_heads) * (head_dim / 16);
    if (tiles > 0x7fffffffLL) return zi_fail("gemm_smallm_rope: too many tiles");
    if (M <= 8) gemm_smallm_rope_kernel<1><<<(unsigned)tiles, GS_THREADS, 0, stream>>>((const bf16*)X, (const bf16*)W, (const bf16*)bias, ro, M, K, ldx, ldw);
    else gemm_smallm_rope_kernel<2><<<(unsigned)tiles, GS_THREADS, 0, stream>>>((const bf16*)X, (const bf16*)W, (const bf16*)bias, ro, M, K, ldx, ldw);
    return zi_check_launch("gemm_smallm_rope");
}

// ---------------------------------------------------------------------------------------------------------
// The same product with built-in scratch, for callers that must not allocate (see gemm_smallm_noalloc.h).
// ---------------------------------------------------------------------------------------------------------
#include "gemm_smallm_noalloc.h"

// Partial sums of the K ranges, then the arrival counters.  In host code this name is only a handle for
// cudaGetSymbolAddress; the kernel receives the device address that call returns.
static __device__ __align__(256) unsigned char zi_noalloc_scratch[ZI_NOALLOC_SCRATCH_BYTES];

#define ZI_NOALLOC_MAX_DEVICES 64
static void* zi_noalloc_base[ZI_NOALLOC_MAX_DEVICES];      // device address of the array, per device ordinal

// Set-up, once per device, with that device current: resolve the array's address on this device.
static int zi_noalloc_setup(int device, void** base) {
    if (device < 0 || device >= ZI_NOALLOC_MAX_DEVICES) return zi_fail("gemm_smallm_noalloc: device ordinal %d out of range", device);
    if (!zi_noalloc_base[device]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&ptr, zi_noalloc_scratch);
        if (e != cudaSuccess || !ptr) {
            cudaGetLastError();
            return zi_fail("gemm_smallm_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        }
        zi_noalloc_base[device] = ptr;
    }
    *base = zi_noalloc_base[device];
    return 0;
}

// 0 (default): the K ranges of a column tile meet in distributed shared memory where a cluster of that shape can be
// launched, and the array only serves where it cannot.  1: the sums always go through the array (partial sums
// written to it, counted, and added by the block that arrives last).  Both give the same bits.  Returns the
// setting it replaces.  Process-wide; not meant to be flipped while calls are in flight on another thread.
static int zi_noalloc_through_array = 0;
ZI_EXPORT int zi_gemm_smallm_noalloc_reduction(int through_array) {
    const int before = zi_noalloc_through_array;
    zi_noalloc_through_array = through_array ? 1 : 0;
    return before;
}

ZI_EXPORT int zi_gemm_smallm_noalloc(const void* X, const void* W, const void* bias, void* C, int c_dtype, int M, int N,
                                     int K, long long ldx, long long ldw, long long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16) return zi_fail("gemm_smallm_noalloc: M=%d rows; this kernel takes at most 16", M);
    if (K <= 0 || K % 32 != 0) return zi_fail("gemm_smallm_noalloc: K=%d must be a positive multiple of 32", K);
    if (ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_smallm_noalloc: row strides (%lld, %lld) must be multiples of 8 elements", ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_smallm_noalloc: operands must be 16-byte aligned");
    if (c_dtype != ZI_F32 && c_dtype != ZI_BF16) return zi_fail("gemm_smallm_noalloc: unknown output dtype %d", c_dtype);
    const int ksplit = zi_gemm_smallm_ksplit(N, K, 0);
    const int tiles = (N + 15) / 16;
    float* part = nullptr;
    int* counters = nullptr;
    if (ksplit > 1) {
        const long long need = (long long)ksplit * 16 * N;
        if (need > ZI_NOALLOC_PART_FLOATS || tiles > ZI_NOALLOC_COUNTER_INTS)
            return zi_fail("gemm_smallm_noalloc: N=%d, K=%d is cut into %d K ranges whose sums take %lld floats (and %d counters); "
                           "the built-in array holds %d floats and %d counters", N, K, ksplit, need, tiles,
                           ZI_NOALLOC_PART_FLOATS, ZI_NOALLOC_COUNTER_INTS);
        int device = -1;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return zi_fail("gemm_smallm_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
        void* base = nullptr;
        if (zi_noalloc_setup(device, &base)) return 1;
        part = reinterpret_cast<float*>(base);
        counters = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(base) + (size_t)ZI_NOALLOC_PART_FLOATS * 4);
        // the counters must start at zero whatever an earlier (possibly aborted) call left behind
        e = cudaMemsetAsync(counters, 0, (size_t)tiles * sizeof(int), stream);
        if (e != cudaSuccess) return zi_fail("gemm_smallm_noalloc: clearing the counters failed: %s", cudaGetErrorString(e));
    }
    const bool f32 = c_dtype == ZI_F32, cl = !zi_noalloc_through_array;
    if (M <= 8) { if (f32) launch<1, float, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream, cl); else launch<1, bf16, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream, cl); }
    else        { if (f32) launch<2, float, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream, cl); else launch<2, bf16, false>(X, W, bias, C, part, counters, ksplit, M, N, K, ldx, ldw, ldc, stream, cl); }
    return zi_check_launch("gemm_smallm_noalloc");
}
