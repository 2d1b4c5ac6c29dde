// Fused kernels of a decode step (at most 16 tokens, bfloat16): the weight-streaming product of
// gemm_smallm.cu with the neighbouring element-wise work folded into its prologue and epilogue, so that a
// layer is five launches instead of nine and the activations between them never make a round trip.
//
//   prologue X_NORM   : the operand is RMSNorm(h) computed on the fly.  h is the float32 residual stream;
//                       the sum of squares of each row arrives as partial sums (one per column tile of the
//                       kernel that last wrote h) and is added up in a fixed order; the fragment fed to the
//                       tensor cores is bfloat16((w_norm * h) * rstd), the value the stand-alone norm writes.
//   epilogue RESIDUAL : h[m, n] += product (float32, every element owned by one block), and the block's share
//                       of sum(h_new^2) per row is left for the next X_NORM prologue.
//   epilogue SILU     : gate and up rows of one weight; writes up * gate / (1 + exp(-gate)).
//   epilogue ROPE     : the stacked q/k/v projection.  A block owns dims k .. k+7 and k+half .. k+half+7 of one
//                       head (MMA rows g and g+8), so both halves of a rotation pair meet in one thread: bias,
//                       rotate-half RoPE by the token's position, then q goes to the query buffer and k, v to
//                       the token's cache page.
//
// The product itself is the one of gemm_smallm.cu: 16 weight rows per block, 8 warps on interleaved k-steps,
// weights from global memory straight into mma.sync fragments with the k-permutation trick, partial sums of
// the warps added in warp order; optional split of K over blocks with a last-block reduction.
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(decode_fused)

#define DF_WARPS 8
#define DF_THREADS (DF_WARPS * 32)
#define DF_UNROLL 4

enum { X_BF16 = 0, X_NORM = 1 };
enum { EPI_PLAIN = 0, EPI_SILU = 1, EPI_RESIDUAL = 2, EPI_ROPE = 3 };

__device__ __forceinline__ void df_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 df_ldg_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t df_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct DfParams {
    // operand
    const bf16* X; long long ldx;                                   // X_BF16
    const float* h; const bf16* w_norm; const float* ssq_in; int n_part; float eps;   // X_NORM: h is [M, K]
    // weight
    const bf16* W; long long ldw; const bf16* bias;
    int M, N, K;
    // outputs
    void* C; long long ldc; int c_is_f32;                           // PLAIN, SILU
    float* h_out; float* ssq_out;                                   // RESIDUAL: h_out is [M, N]; ssq_out [tiles][16]
    float* part; int* counters;                                     // split of K over blocks
    // ROPE
    bf16* q_out; bf16* cache; const int* tables; const int* tok_seg; const int* pos; const float* inv_freq;
    int n_heads, n_kv_heads, head_dim, page_size, max_blocks, write_kv;
    long long page_stride, kv_stride;
};

// The activation fragment of one k-step (32 k-values from k) for token row `m`: this lane's 8 values k + tq*8 ..
template <int XMODE>
__device__ __forceinline__ uint4 df_x_fragment(const DfParams& p, int m, int k, int tq, float rstd) {
    if (XMODE == X_BF16) {
        return ld_dep16(p.X + (long long)m * p.ldx + k + tq * 8);
    } else {
        const float* hp = p.h + (long long)m * p.K + k + tq * 8;
        const float4 h0 = *reinterpret_cast<const float4*>(hp), h1 = *reinterpret_cast<const float4*>(hp + 4);
        const uint4 wr = *reinterpret_cast<const uint4*>(p.w_norm + k + tq * 8);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
        const float2 w01 = __bfloat1622float2(w2[0]), w23 = __bfloat1622float2(w2[1]);
        const float2 w45 = __bfloat1622float2(w2[2]), w67 = __bfloat1622float2(w2[3]);
        uint4 x;
        x.x = df_pack((w01.x * h0.x) * rstd, (w01.y * h0.y) * rstd);
        x.y = df_pack((w23.x * h0.z) * rstd, (w23.y * h0.w) * rstd);
        x.z = df_pack((w45.x * h1.x) * rstd, (w45.y * h1.y) * rstd);
        x.w = df_pack((w67.x * h1.z) * rstd, (w67.y * h1.w) * rstd);
        return x;
    }
}

template <int NT, int XMODE>
__device__ __forceinline__ void df_accumulate(float (&acc)[NT][4], const DfParams& p, const bf16* w0, const bf16* w1,
                                              int step_begin, int step_end, int warp, int g, int tq, const float* rstd_s) {
    int mrow[NT];
    float rs[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mrow[nt] = min(nt * 8 + g, p.M - 1);
        rs[nt] = XMODE == X_NORM ? rstd_s[mrow[nt]] : 1.0f;
    }
    int s = step_begin + warp;
    for (; s + (DF_UNROLL - 1) * DF_WARPS < step_end; s += DF_UNROLL * DF_WARPS) {
        uint4 a[DF_UNROLL], b[DF_UNROLL];
#pragma unroll
        for (int u = 0; u < DF_UNROLL; ++u) {
            const int k = (s + u * DF_WARPS) * 32;
            a[u] = df_ldg_stream(w0 + k);
            b[u] = df_ldg_stream(w1 + k);
        }
#pragma unroll
        for (int u = 0; u < DF_UNROLL; ++u) {
            const int k = (s + u * DF_WARPS) * 32;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 x = df_x_fragment<XMODE>(p, mrow[nt], k, tq, rs[nt]);
                df_mma(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, x.x, x.y);
                df_mma(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, x.z, x.w);
            }
        }
    }
    for (; s < step_end; s += DF_WARPS) {
        const int k = s * 32;
        const uint4 a = df_ldg_stream(w0 + k), b = df_ldg_stream(w1 + k);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 x = df_x_fragment<XMODE>(p, mrow[nt], k, tq, rs[nt]);
            df_mma(acc[nt], a.x, b.x, a.y, b.y, x.x, x.y);
            df_mma(acc[nt], a.z, b.z, a.w, b.w, x.z, x.w);
        }
    }
}

template <int NT>
__device__ __forceinline__ void df_store_red(float (*red)[16][NT * 8 + 1], const float (&acc)[NT][4], int warp, int g, int tq) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][nt * 8 + tq * 2] = acc[nt][0];
        red[warp][g][nt * 8 + tq * 2 + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + tq * 2] = acc[nt][2];
        red[warp][g + 8][nt * 8 + tq * 2 + 1] = acc[nt][3];
    }
}

template <int NT, int XMODE, int EPI>
__global__ void __launch_bounds__(DF_THREADS)
decode_fused_kernel(const DfParams p) {
    __shared__ float red[EPI == EPI_SILU ? 2 : 1][DF_WARPS][16][NT * 8 + 1];
    __shared__ float rstd_s[16];
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, tq = lane & 3;
    const int tile = blockIdx.x;
    const int ksplit = gridDim.y, ks = blockIdx.y;
    const int steps = p.K / 32, per = (steps + ksplit - 1) / ksplit;
    const int step_begin = ks * per, step_end = min(steps, step_begin + per);

    // the two weight rows behind MMA rows g and g+8
    int rA, rB, head = 0, sub = 0;
    if (EPI == EPI_ROPE) {
        const int tph = p.head_dim / 16;                       // blocks per head
        head = tile / tph;
        sub = tile - head * tph;
        if (!p.write_kv && head >= p.n_heads) return;          // this call only needs the queries
        rA = head * p.head_dim + sub * 8 + g;
        rB = rA + p.head_dim / 2;
    } else {
        rA = min(tile * 16 + g, p.N - 1);
        rB = min(tile * 16 + g + 8, p.N - 1);
    }
    const bf16* w0 = p.W + (long long)rA * p.ldw + tq * 8;
    const bf16* w1 = p.W + (long long)rB * p.ldw + tq * 8;

    if (XMODE == X_NORM) {
        // rstd[m] from the partial sums of squares, added in a fixed order: 16 threads per row
        const int m = threadIdx.x >> 4, sl = threadIdx.x & 15;
        float s = 0.0f;
        for (int i = sl; i < p.n_part; i += 16) s += p.ssq_in[i * 16 + m];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o, 16);
        if (sl == 0) rstd_s[m] = 1.0f / sqrtf(s / (float)p.K + p.eps);
        __syncthreads();
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
    df_accumulate<NT, XMODE>(acc, p, w0, w1, step_begin, step_end, warp, g, tq, rstd_s);
    df_store_red<NT>(red[0], acc, warp, g, tq);
    if (EPI == EPI_SILU) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        df_accumulate<NT, XMODE>(acc, p, w0 + (long long)p.N * p.ldw, w1 + (long long)p.N * p.ldw, step_begin, step_end,
                                 warp, g, tq, rstd_s);
        df_store_red<NT>(red[EPI == EPI_SILU ? 1 : 0], acc, warp, g, tq);
    }
    __syncthreads();

    if (ksplit > 1) {
        for (int i = threadIdx.x; i < 16 * NT * 8; i += DF_THREADS) {
            const int r = i % 16, m = i / 16;
            if (tile * 16 + r >= p.N || m >= p.M) continue;
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < DF_WARPS; ++w) v += red[0][w][r][m];
            p.part[((size_t)ks * 16 + m) * p.N + tile * 16 + r] = v;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int prev = atomicAdd(&p.counters[tile], 1);
            is_last = (prev == ksplit - 1);
            if (is_last) p.counters[tile] = 0;
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
    }

    if (EPI == EPI_ROPE) {
        // pairs (k, k + half): value j of MMA row j and of row j + 8, for token m
        const int half = p.head_dim / 2;
        for (int i = threadIdx.x; i < 8 * NT * 8; i += DF_THREADS) {
            const int j = i & 7, m = i >> 3;
            if (m >= p.M) continue;
            float a = 0.0f, b = 0.0f;
#pragma unroll
            for (int w = 0; w < DF_WARPS; ++w) { a += red[0][w][j][m]; b += red[0][w][j + 8][m]; }
            const int k = sub * 8 + j;
            const int ra = head * p.head_dim + k;
            if (p.bias) { a += __bfloat162float(p.bias[ra]); b += __bfloat162float(p.bias[ra + half]); }
            // the projection's output is stored in bfloat16 before it is rotated, as in the separate kernels
            a = __bfloat162float(__float2bfloat16_rn(a));
            b = __bfloat162float(__float2bfloat16_rn(b));
            const int pm = p.pos[m];
            bf16* dst;
            bool rotate = true;
            if (head < p.n_heads) {
                dst = p.q_out + ((size_t)m * p.n_heads + head) * p.head_dim;
            } else {
                const int kvh = (head - p.n_heads) % p.n_kv_heads;
                const bool is_v = (head - p.n_heads) >= p.n_kv_heads;
                const int page = p.tables[(size_t)p.tok_seg[m] * p.max_blocks + pm / p.page_size];
                const int off = pm % p.page_size;
                dst = p.cache + (size_t)page * p.page_stride + (is_v ? p.kv_stride : 0) +
                      ((size_t)kvh * p.page_size + off) * p.head_dim;
                rotate = !is_v;
            }
            if (rotate) {
                float sn, cs;
                sincosf((float)pm * p.inv_freq[k], &sn, &cs);
                dst[k] = __float2bfloat16_rn(a * cs - b * sn);
                dst[k + half] = __float2bfloat16_rn(b * cs + a * sn);
            } else {
                dst[k] = __float2bfloat16_rn(a);
                dst[k + half] = __float2bfloat16_rn(b);
            }
        }
        return;
    }

    for (int i = threadIdx.x; i < 16 * NT * 8; i += DF_THREADS) {
        const int r = i % 16, m = i / 16;             // consecutive threads -> consecutive output columns
        const int n = tile * 16 + r;
        const bool live = n < p.N && m < p.M;
        float v = 0.0f;
        if (live) {
            if (ksplit > 1) {
                for (int k2 = 0; k2 < ksplit; ++k2) v += ld_l2(p.part + ((size_t)k2 * 16 + m) * p.N + n);
            } else {
#pragma unroll
                for (int w = 0; w < DF_WARPS; ++w) v += red[0][w][r][m];
            }
        }
        if (EPI == EPI_SILU) {
            if (!live) continue;
            float u = 0.0f;
#pragma unroll
            for (int w = 0; w < DF_WARPS; ++w) u += red[EPI == EPI_SILU ? 1 : 0][w][r][m];
            const float gr = __bfloat162float(__float2bfloat16_rn(v)), ur = __bfloat162float(__float2bfloat16_rn(u));
            const float y = ur * gr / (1.0f + expf(-gr));
            if (p.c_is_f32) reinterpret_cast<float*>(p.C)[(long long)m * p.ldc + n] = y;
            else reinterpret_cast<bf16*>(p.C)[(long long)m * p.ldc + n] = __float2bfloat16_rn(y);
        } else if (EPI == EPI_PLAIN) {
            if (!live) continue;
            if (p.bias) v += __bfloat162float(p.bias[n]);
            if (p.c_is_f32) reinterpret_cast<float*>(p.C)[(long long)m * p.ldc + n] = v;
            else reinterpret_cast<bf16*>(p.C)[(long long)m * p.ldc + n] = __float2bfloat16_rn(v);
        } else {   // EPI_RESIDUAL
            float hn = 0.0f;
            if (live) {
                if (p.bias) v += __bfloat162float(p.bias[n]);
                // the branch output is stored in bfloat16 before it is added, as in the separate kernels
                v = __bfloat162float(__float2bfloat16_rn(v));
                float* hp = p.h_out + (long long)m * p.N + n;
                hn = *hp + v;
                *hp = hn;
            }
            // this block's share of sum(h_new^2) of row m: the 16 threads of a row add up (16 | 32, rows never straddle a warp)
            float sq = hn * hn;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o, 16);
            if (r == 0) p.ssq_out[(size_t)tile * 16 + m] = sq;
        }
    }
}

// ---- entry points ----------------------------------------------------------------------------------------
static int df_ksplit(int N, int K) {
    const int tiles = (N + 15) / 16, steps = K / 32;
    if (tiles >= 296) return 1;
    int ks = (296 + tiles - 1) / tiles;
    if (ks > 8) ks = 8;
    while (ks > 1 && steps / ks < 8 * DF_WARPS) --ks;
    return ks < 1 ? 1 : ks;
}

static int df_check(const char* what, int M, int K, long long ldw, const void* W) {
    if (M > 16) return zi_fail("%s: M=%d rows; the fused decode kernels take at most 16", what, M);
    if (K <= 0 || K % 32 != 0) return zi_fail("%s: K=%d must be a positive multiple of 32", what, K);
    if (ldw % 8 != 0 || ((uintptr_t)W & 15)) return zi_fail("%s: weight rows must be 16-byte aligned", what);
    return 0;
}

template <int XMODE, int EPI>
static void df_launch(const DfParams& p, int tiles, int ksplit, cudaStream_t stream) {
    if (p.M <= 8) decode_fused_kernel<1, XMODE, EPI><<<dim3(tiles, ksplit), DF_THREADS, 0, stream>>>(p);
    else decode_fused_kernel<2, XMODE, EPI><<<dim3(tiles, ksplit), DF_THREADS, 0, stream>>>(p);
}

// C = RMSNorm(h; w_norm, ssq_in) . W^T (+ bias), or with silu_mul the gated activation of W = [gate rows; up rows].
ZI_EXPORT int zi_fused_norm_gemm(const float* h, const float* ssq_in, int n_part, const void* w_norm, float eps,
                                 const void* W, const void* bias, void* C, int c_dtype, int M, int N, int K,
                                 long long ldw, long long ldc, int silu_mul, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (df_check("fused_norm_gemm", M, K, ldw, W)) return 1;
    if (n_part <= 0 || !ssq_in) return zi_fail("fused_norm_gemm: the sums of squares of h are missing");
    if (((uintptr_t)h | (uintptr_t)w_norm) & 15) return zi_fail("fused_norm_gemm: h and the norm weight must be 16-byte aligned");
    if (silu_mul && bias) return zi_fail("fused_norm_gemm: the fused activation takes no bias");
    DfParams p;
    memset(&p, 0, sizeof(p));
    p.h = h; p.w_norm = (const bf16*)w_norm; p.ssq_in = ssq_in; p.n_part = n_part; p.eps = eps;
    p.W = (const bf16*)W; p.ldw = ldw; p.bias = (const bf16*)bias; p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc; p.c_is_f32 = c_dtype == ZI_F32;
    const int tiles = (N + 15) / 16;
    if (silu_mul) df_launch<X_NORM, EPI_SILU>(p, tiles, 1, stream);
    else df_launch<X_NORM, EPI_PLAIN>(p, tiles, 1, stream);
    return zi_check_launch("fused_norm_gemm");
}

// q, k, v = RMSNorm(h) . Wqkv^T + b; q and k rotated by position; q -> q_out [M, n_heads, head_dim], k and v -> cache pages.
ZI_EXPORT int zi_fused_norm_qkv_rope(const float* h, const float* ssq_in, int n_part, const void* w_norm, float eps,
                                     const void* W, const void* bias, void* q_out, void* cache, const int* tables,
                                     const int* tok_seg, const int* pos, const float* inv_freq, int M, int K,
                                     long long ldw, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                     int max_blocks, long long page_stride, long long kv_stride, int write_kv,
                                     cudaStream_t stream) {
    if (M <= 0) return 0;
    if (df_check("fused_norm_qkv_rope", M, K, ldw, W)) return 1;
    if (head_dim <= 0 || head_dim % 16 != 0) return zi_fail("fused_norm_qkv_rope: head_dim=%d must be a multiple of 16", head_dim);
    if (n_part <= 0 || !ssq_in) return zi_fail("fused_norm_qkv_rope: the sums of squares of h are missing");
    if (((uintptr_t)h | (uintptr_t)w_norm) & 15) return zi_fail("fused_norm_qkv_rope: h and the norm weight must be 16-byte aligned");
    DfParams p;
    memset(&p, 0, sizeof(p));
    p.h = h; p.w_norm = (const bf16*)w_norm; p.ssq_in = ssq_in; p.n_part = n_part; p.eps = eps;
    p.W = (const bf16*)W; p.ldw = ldw; p.bias = (const bf16*)bias; p.M = M; p.K = K;
    p.N = (n_heads + 2 * n_kv_heads) * head_dim;
    p.q_out = (bf16*)q_out; p.cache = (bf16*)cache; p.tables = tables; p.tok_seg = tok_seg; p.pos = pos; p.inv_freq = inv_freq;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.page_size = page_size; p.max_blocks = max_blocks;
    p.write_kv = write_kv; p.page_stride = page_stride; p.kv_stride = kv_stride;
    const int tiles = (n_heads + 2 * n_kv_heads) * (head_dim / 16);
    df_launch<X_NORM, EPI_ROPE>(p, tiles, 1, stream);
    return zi_check_launch("fused_norm_qkv_rope");
}

ZI_EXPORT int zi_gemm_residual_ksplit(int N, int K) { return df_ksplit(N, K); }

// h[M, N] += X . W^T (+ bias); ssq_out[tile][16] receives each column tile's share of sum(h_new^2) per row.
// part / counters: scratch of the K split (ksplit * 16 * N floats, ceil(N/16) ints that are zero and stay zero).
ZI_EXPORT int zi_gemm_residual(const void* X, const void* W, const void* bias, float* h, float* ssq_out, float* part,
                               int* counters, int M, int N, int K, long long ldx, long long ldw, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (df_check("gemm_residual", M, K, ldw, W)) return 1;
    if (ldx % 8 != 0 || ((uintptr_t)X & 15)) return zi_fail("gemm_residual: X rows must be 16-byte aligned");
    const int ksplit = df_ksplit(N, K);
    if (ksplit > 1 && (!part || !counters)) return zi_fail("gemm_residual: N=%d K=%d is split %d ways and needs scratch", N, K, ksplit);
    DfParams p;
    memset(&p, 0, sizeof(p));
    p.X = (const bf16*)X; p.ldx = ldx; p.W = (const bf16*)W; p.ldw = ldw; p.bias = (const bf16*)bias;
    p.M = M; p.N = N; p.K = K; p.h_out = h; p.ssq_out = ssq_out; p.part = part; p.counters = counters;
    df_launch<X_BF16, EPI_RESIDUAL>(p, (N + 15) / 16, ksplit, stream);
    return zi_check_launch("gemm_residual");
}
