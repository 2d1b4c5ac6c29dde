// Row-wise and element-wise kernels: embedding gather, RMSNorm (plain, and fused with the
// residual add), rotate-half RoPE fused with the append to the paged cache, SiLU-mul, cast.
// All arithmetic is float32; storage types are float32 or bfloat16 per tensor.
#define ZI_PDL_BIT 1
#include "zi_common.cuh"

ZI_DEFINE_LAST_ERROR(elementwise)

// ---------------------------------------------------------------------------------------
// Embedding: out[n, :] = table[ids[n], :]
// ---------------------------------------------------------------------------------------
template <typename TT, typename TO>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 TO* __restrict__ out, int hidden, int vocab) {
    const int n = blockIdx.x;
    pdl_trigger_early();
    pdl_wait();
    pdl_trigger_late();
    int id = ld_dep(ids + n);
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);   // the host refuses ids outside the table
    const TT* src = table + (size_t)id * hidden;
    TO* dst = out + (size_t)n * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = from_f32<TO>(to_f32<TT>(src[j]));
}

ZI_EXPORT int zi_embedding(const void* table, int table_dtype, const int* ids, void* out, int out_dtype,
                           int n_tokens, int hidden, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return zi_fail("embedding: hidden=%d vocab=%d must be positive", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    ZI_DISPATCH(table_dtype, TT, ZI_DISPATCH(out_dtype, TO, {
        zi_launch(embedding_kernel<TT, TO>, dim3(n_tokens), dim3(threads), 0, stream, (const TT*)table, ids, (TO*)out, hidden, vocab);
    }););
    return zi_check_launch("embedding");
}

// ---------------------------------------------------------------------------------------
// RMSNorm.  y = (w * x) * rstd, rstd = 1/sqrt(mean(x^2) + eps), all in float32.
//   delta != null : x = residual[row] + delta[row] (float32 add); written back to residual
//                   when write_residual is set.
//   row_idx != null : output row r reads input row row_idx[r] (used for the rows whose
//                   logits are wanted); the residual is then never written.
// One block per output row, a fixed block size, so the sum's order is a function of the
// width alone.
// ---------------------------------------------------------------------------------------
#define NORM_THREADS 256
// Up to this many rows (decode steps) a norm asks for its weight together with the row instead of after the sum: one
// trip to memory less in a kernel that is nothing else (20 us of a 28-layer step of 1.36 ms).  With many rows the
// extra registers cost more than the trip.
#define NORM_FEW_ROWS 64
#ifndef NORM_KEEP_ROWS
#define NORM_KEEP_ROWS 256
#endif
__device__ __forceinline__ void load8_hint(const float* p, float* out, uint64_t policy) {
    asm volatile("ld.global.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3]) : "l"(p), "l"(policy));
    asm volatile("ld.global.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=f"(out[4]), "=f"(out[5]), "=f"(out[6]), "=f"(out[7]) : "l"(p + 4), "l"(policy));
}
__device__ __forceinline__ void store8_hint(float* p, const float* v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;\n"
                 ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "l"(policy) : "memory");
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;\n"
                 ::"l"(p + 4), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "l"(policy) : "memory");
}
template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const TW* __restrict__ w,
               TO* __restrict__ out, const int* __restrict__ row_idx, float eps, int hidden,
               int write_residual) {
    extern __shared__ float row[];           // hidden floats
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    pdl_trigger_early();
    pdl_wait();
    const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* res = residual + src * hidden;
    const TD* d = delta ? delta + src * hidden : nullptr;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += NORM_THREADS) {
        float x = ld_dep(res + j);
        if (d) x = x + ld_dep_f32<TD>(d + j);
        row[j] = x;
        ss = fmaf(x, x, ss);
    }
    ss = block_sum(ss, scratch);
    pdl_trigger_late();
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    const bool wb = d && write_residual && !row_idx;
    TO* o = out + (size_t)r * hidden;
    for (int j = threadIdx.x; j < hidden; j += NORM_THREADS) {
        const float x = row[j];
        if (wb) res[j] = x;
        o[j] = from_f32<TO>((to_f32<TW>(w[j]) * x) * rstd);
    }
}

// The same with 8 elements per thread and access (16-byte loads and stores for bfloat16, 32-byte for float32):
// taken whenever the width is a multiple of 8 and the rows are aligned, whatever the number of rows, so a row's
// sum has one order however the step was cut.
template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec8_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const TW* __restrict__ w,
                    TO* __restrict__ out, const int* __restrict__ row_idx, float eps, int hidden,
                    int write_residual) {
    extern __shared__ float row[];           // hidden floats
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    pdl_trigger_early();
    pdl_wait();
    const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* res = residual + src * hidden;
    const TD* d = delta ? delta + src * hidden : nullptr;
    const bool wb = d && (write_residual & 1) && !row_idx;
    // Many rows (a prompt portion): the residual stream is read again by the next norm, some 80 us and 150 MB of
    // other traffic later; it asks L2 to let go of it last.
    const bool keep = gridDim.x >= NORM_KEEP_ROWS;
    uint64_t policy = 0;
    if (keep) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(policy));
    float ss = 0.0f;
    if ((write_residual & 2) && hidden <= NORM_THREADS * 8) {
        // Few rows (a decode step), one piece of the row per thread: the weight is asked for together with the row,
        // not after the sum (one trip to memory instead of two in a kernel that is nothing but trips to memory).
        const int j = threadIdx.x * 8;
        float x[8], wv[8];
        const bool mine = j < hidden;
        if (mine) {
            load8(res + j, x);
            load8(w + j, wv);
            if (d) {
                float dv[8];
                load8(d + j, dv);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = x[i] + dv[i];
                if (wb) store8(res + j, x);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        }
        ss = block_sum(ss, scratch);
        pdl_trigger_late();
        const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
        if (mine) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = (wv[i] * x[i]) * rstd;
            store8(out + (size_t)r * hidden + j, x);
        }
        return;
    }
    for (int j = threadIdx.x * 8; j < hidden; j += NORM_THREADS * 8) {
        float x[8];
        if (keep) load8_hint(res + j, x, policy); else load8(res + j, x);
        if (d) {
            float dv[8];
            load8(d + j, dv);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[i] + dv[i];
            if (wb) { if (keep) store8_hint(res + j, x, policy); else store8(res + j, x); }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        store8(row + j, x);
    }
    ss = block_sum(ss, scratch);
    pdl_trigger_late();
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int j = threadIdx.x * 8; j < hidden; j += NORM_THREADS * 8) {
        float x[8], wv[8];
        load8(row + j, x);
        load8(w + j, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (wv[i] * x[i]) * rstd;
        store8(o + j, x);
    }
}

// The branch output as partial sums: delta = parts[0] + parts[1] + ... (float32 [n_parts][rows][hidden], the
// ranges of K of a product that was cut for more parallelism), added in that order and rounded to the output's type,
// as the uncut product would have rounded its result; then as above.  hidden % 8 == 0, 32-byte aligned rows.
template <typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_parts_vec8_kernel(float* __restrict__ residual, const float* __restrict__ parts, int n_parts, long long part_stride,
                          const TW* __restrict__ w, TO* __restrict__ out, const int* __restrict__ row_idx, float eps,
                          int hidden, int write_residual) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
    float* res = residual + src * hidden;
    const float* d = parts + src * hidden;
    const bool wb = (write_residual & 1) && !row_idx;
    float ss = 0.0f;
    if ((write_residual & 2) && hidden <= NORM_THREADS * 8 && n_parts <= 4) {
        // Few rows, one piece of the row per thread: the row, every partial sum and the weight are asked for
        // together (one trip to memory; the loop below makes one per partial sum and one more for the weight).
        const int j = threadIdx.x * 8;
        float x[8], wv[8], dv[4][8];
        const bool mine = j < hidden;
        if (mine) {
            load8(res + j, x);
            load8(w + j, wv);
#pragma unroll
            for (int p = 0; p < 4; ++p)
                if (p < n_parts) load8(d + (size_t)p * part_stride + j, dv[p]);
#pragma unroll
            for (int p = 1; p < 4; ++p) {
                if (p < n_parts) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) dv[0][i] += dv[p][i];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[i] + to_f32<TO>(from_f32<TO>(dv[0][i]));
            if (wb) store8(res + j, x);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
        if (mine) {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = (wv[i] * x[i]) * rstd;
            store8(out + (size_t)r * hidden + j, x);
        }
        return;
    }
    for (int j = threadIdx.x * 8; j < hidden; j += NORM_THREADS * 8) {
        float x[8], dv[8];
        load8(res + j, x);
        load8(d + j, dv);
        for (int p = 1; p < n_parts; ++p) {
            float more[8];
            load8(d + (size_t)p * part_stride + j, more);
#pragma unroll
            for (int i = 0; i < 8; ++i) dv[i] += more[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = x[i] + to_f32<TO>(from_f32<TO>(dv[i]));
        if (wb) store8(res + j, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
        store8(row + j, x);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int j = threadIdx.x * 8; j < hidden; j += NORM_THREADS * 8) {
        float x[8], wv[8];
        load8(row + j, x);
        load8(w + j, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = (wv[i] * x[i]) * rstd;
        store8(o + j, x);
    }
}

// Plain norm of a tensor that is not the float32 residual (used by parts tested alone).
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_plain_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out, float eps,
                     int hidden) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const TX* xr = x + (size_t)blockIdx.x * hidden;
    pdl_trigger_early();
    pdl_wait();
    float ss = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += NORM_THREADS) {
        const float v = ld_dep_f32<TX>(xr + j);
        row[j] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)blockIdx.x * hidden;
    for (int j = threadIdx.x; j < hidden; j += NORM_THREADS)
        o[j] = from_f32<TO>((to_f32<TW>(w[j]) * row[j]) * rstd);
}

static int norm_smem_ok(int hidden, const void* fn) {
    const size_t bytes = (size_t)hidden * sizeof(float);
    if (bytes > 200 * 1024) return zi_fail("rmsnorm: width %d needs %zu bytes of shared memory (limit 200 KiB)", hidden, bytes);
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return zi_fail("rmsnorm: cannot reserve %zu bytes of shared memory: %s", bytes, cudaGetErrorString(e));
    }
    return 0;
}

// residual: float32 [*, hidden] (in/out).  delta: nullable, [*, hidden] of delta_dtype.
ZI_EXPORT int zi_add_rmsnorm(void* residual, const void* delta, int delta_dtype, const void* w, int w_dtype,
                             void* out, int out_dtype, const int* row_idx, int rows, int hidden, float eps,
                             int write_residual, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return zi_fail("rmsnorm: width %d must be positive", hidden);
    const size_t smem = (size_t)hidden * sizeof(float);
    const bool vec = hidden % 8 == 0 && (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 31) == 0;
    ZI_DISPATCH(delta_dtype, TD, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(out_dtype, TO, {
        auto fn = vec ? rmsnorm_vec8_kernel<TD, TW, TO> : rmsnorm_kernel<TD, TW, TO>;
        if (norm_smem_ok(hidden, (const void*)fn)) return 1;
        zi_launch(fn, dim3(rows), dim3(NORM_THREADS), smem, stream, (float*)residual, (const TD*)delta, (const TW*)w,
                  (TO*)out, row_idx, eps, hidden, (write_residual ? 1 : 0) | ((vec && rows <= NORM_FEW_ROWS) ? 2 : 0));
    });););
    return zi_check_launch("add_rmsnorm");
}

// parts: float32 [n_parts][part_rows][hidden] (part_stride = part_rows * hidden elements); see rmsnorm_parts_vec8_kernel.
ZI_EXPORT int zi_add_rmsnorm_parts(void* residual, const float* parts, int n_parts, long long part_stride, const void* w,
                                   int w_dtype, void* out, int out_dtype, const int* row_idx, int rows, int hidden, float eps,
                                   int write_residual, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden % 8) return zi_fail("rmsnorm: partial sums need a width that is a positive multiple of 8, got %d", hidden);
    if (n_parts < 1 || !parts) return zi_fail("rmsnorm: %d partial sums", n_parts);
    if ((((uintptr_t)residual | (uintptr_t)parts | (uintptr_t)w | (uintptr_t)out) & 31) || (part_stride & 7))
        return zi_fail("rmsnorm: partial sums, residual, weight and output must be 32-byte aligned");
    const size_t smem = (size_t)hidden * sizeof(float);
    ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(out_dtype, TO, {
        auto fn = rmsnorm_parts_vec8_kernel<TW, TO>;
        if (norm_smem_ok(hidden, (const void*)fn)) return 1;
        fn<<<rows, NORM_THREADS, smem, stream>>>((float*)residual, parts, n_parts, part_stride, (const TW*)w, (TO*)out, row_idx,
                                                  eps, hidden, (write_residual ? 1 : 0) | (rows <= NORM_FEW_ROWS ? 2 : 0));
    }););
    return zi_check_launch("add_rmsnorm_parts");
}

ZI_EXPORT int zi_rmsnorm(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                         int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return zi_fail("rmsnorm: width %d must be positive", hidden);
    const size_t smem = (size_t)hidden * sizeof(float);
    ZI_DISPATCH(x_dtype, TX, ZI_DISPATCH(w_dtype, TW, ZI_DISPATCH(out_dtype, TO, {
        auto fn = rmsnorm_plain_kernel<TX, TW, TO>;
        if (norm_smem_ok(hidden, (const void*)fn)) return 1;
        zi_launch(fn, dim3(rows), dim3(NORM_THREADS), smem, stream, (const TX*)x, (const TW*)w, (TO*)out, eps, hidden);
    });););
    return zi_check_launch("rmsnorm");
}

// ---------------------------------------------------------------------------------------
// RoPE (rotate-half over the whole head) on q and k, fused with the append of k and v
// to the paged cache.
//   qkv      [n_tokens, row_stride]: q heads, then k heads, then v heads, head_dim each
//   q_out    [n_tokens, n_heads, head_dim]
//   cache    one call's slice of the pool: element (page, kv, kvh, off, d) is at
//            cache + page*page_stride + kv*kv_stride + (kvh*page_size + off)*head_dim + d
//   tables   [n_segments, max_blocks] page ids;  tok_seg[n] = segment of token n
//   pos[n]   absolute position of token n;  inv_freq[head_dim/2] float32
// angle = float(pos) * inv_freq[k]; y[k] = a*c - b*s; y[k+half] = b*c + a*s.
// ---------------------------------------------------------------------------------------
// grid (n_tokens, ceil(heads / heads_per_block)), heads = n_heads + 2*n_kv_heads: q heads and k heads are rotated,
// v heads copied.  Few tokens (decode): one head per block, so that the step's handful of tokens still fills
// the GPU.  Many tokens (prefill): all heads of a token in one block, cos/sin computed once per token.
template <typename T>
__global__ void rope_append_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ cache,
                                   const int* __restrict__ tables, const int* __restrict__ tok_seg,
                                   const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                   int row_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                   int max_blocks, long long page_stride, long long kv_stride, int write_kv,
                                   int heads_per_block) {
    extern __shared__ float cs[];            // cos[half], sin[half]
    const int n = blockIdx.x;
    const int half = head_dim >> 1;
    const int total_heads = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int h_begin = blockIdx.y * heads_per_block;
    const int h_end = min(h_begin + heads_per_block, total_heads);
    pdl_trigger_early();
    if (h_begin >= h_end) return;
    pdl_wait();
    pdl_trigger_late();
    const int p = ld_dep(pos + n);
    for (int k = threadIdx.x; k < half; k += blockDim.x) {
        float s, c;
        sincosf((float)p * inv_freq[k], &s, &c);
        cs[k] = c;
        cs[half + k] = s;
    }
    __syncthreads();
    T* page_base = nullptr;
    if (h_end > n_heads) {
        const int seg = tok_seg[n];
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        page_base = cache + (size_t)page * page_stride + (size_t)(p % page_size) * head_dim;
    }
    const T* row = qkv + (size_t)n * row_stride;
    for (int idx = threadIdx.x; idx < (h_end - h_begin) * half; idx += blockDim.x) {
        const int hh = idx / half, k = idx - hh * half;
        const int h = h_begin + hh;
        const T* src = row + (size_t)h * head_dim;
        if (h < n_heads + n_kv_heads) {
            T* dst = h < n_heads ? q_out + ((size_t)n * n_heads + h) * head_dim
                                 : page_base + (size_t)(h - n_heads) * page_size * head_dim;
            const float a = ld_dep_f32<T>(src + k), b = ld_dep_f32<T>(src + k + half);
            const float c = cs[k], sn = cs[half + k];
            // explicit roundings: this kernel and the 8-wide one below must agree to the bit
            dst[k] = from_f32<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
            dst[k + half] = from_f32<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn)));
        } else {
            T* dst = page_base + kv_stride + (size_t)(h - n_heads - n_kv_heads) * page_size * head_dim;
            dst[k] = ld_dep(src + k);
            dst[k + half] = ld_dep(src + k + half);
        }
    }
}

// Few tokens with the step's table of angles (cs [n_tokens, head_dim]: cos | sin, from rope_table_kernel, the same
// sincosf of the same angle): one block per (token, head), a thread per pair of elements.  Everything that does not
// depend on anything else (position, segment, the pair, its cosine and sine) is asked for at once; only the page number
// waits for position and segment.  Two trips to memory instead of four, and no sincosf per layer.
template <typename T>
__global__ void rope_append_few_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ cache,
                                       const int* __restrict__ tables, const int* __restrict__ tok_seg,
                                       const int* __restrict__ pos, const float* __restrict__ cs,
                                       int row_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                       int max_blocks, long long page_stride, long long kv_stride) {
    const int n = blockIdx.x, h = blockIdx.y;
    const int half = head_dim >> 1;
    const int k = threadIdx.x;
    if (k >= half) return;
    const T* src = qkv + (size_t)n * row_stride + (size_t)h * head_dim;
    const int p = pos[n], seg = tok_seg[n];
    const float a = to_f32<T>(src[k]), b = to_f32<T>(src[k + half]);
    const float c = cs[(size_t)n * head_dim + k], sn = cs[(size_t)n * head_dim + half + k];
    T* dst;
    if (h < n_heads) {
        dst = q_out + ((size_t)n * n_heads + h) * head_dim;
    } else {
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        const bool is_v = h >= n_heads + n_kv_heads;
        dst = cache + (size_t)page * page_stride + (is_v ? kv_stride : 0) +
              ((size_t)(h - n_heads - (is_v ? n_kv_heads : 0)) * page_size + (size_t)(p % page_size)) * head_dim;
    }
    if (h < n_heads + n_kv_heads) {
        dst[k] = from_f32<T>(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
        dst[k + half] = from_f32<T>(__fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn)));
    } else {
        dst[k] = from_f32<T>(a);
        dst[k + half] = from_f32<T>(b);
    }
}

// The same for many tokens with 8 elements per access: one block per token, a thread takes 8 consecutive
// elements of a head's first half and the 8 that pair with them in its second half.  The arithmetic per element is
// the one above, so both kernels give the same bits.
template <typename T>
__global__ void __launch_bounds__(128)
rope_append_vec8_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ cache,
                        const int* __restrict__ tables, const int* __restrict__ tok_seg,
                        const int* __restrict__ pos, const float* __restrict__ inv_freq,
                        int row_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                        int max_blocks, long long page_stride, long long kv_stride, int write_kv) {
    // One block per token, 128 threads.  What does not depend on anything else is asked for first and together: the
    // token's position and segment, and each thread's first pieces of the row; the page number needs both of the
    // former, the rotation the position.  (Three trips to memory one after another, with half of 256 threads idle,
    // took 7.3 us for 2,048 tokens of 16 heads; the data would pass in 2.6.)
    extern __shared__ float cs[];            // cos[half], sin[half]
    const int n = blockIdx.x;
    const int half = head_dim >> 1, half8 = half >> 3;
    const int total_heads = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int items = total_heads * half8;
    const T* row = qkv + (size_t)n * row_stride;
    const int p = pos[n];
    const int seg = write_kv ? tok_seg[n] : 0;
    float a0[8], b0[8];                      // the thread's first item, on its way while the angles are computed
    const int idx0 = threadIdx.x;
    if (idx0 < items) {
        const int h = idx0 / half8, k = (idx0 - h * half8) * 8;
        load8(row + (size_t)h * head_dim + k, a0);
        load8(row + (size_t)h * head_dim + k + half, b0);
    }
    for (int k = threadIdx.x; k < half; k += blockDim.x) {
        float sn, c;
        sincosf((float)p * inv_freq[k], &sn, &c);
        cs[k] = c;
        cs[half + k] = sn;
    }
    T* page_base = nullptr;
    if (write_kv) {
        const int page = tables[(size_t)seg * max_blocks + p / page_size];
        page_base = cache + (size_t)page * page_stride + (size_t)(p % page_size) * head_dim;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int h = idx / half8, k = (idx - h * half8) * 8;
        float a[8], b[8];
        if (idx == idx0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) { a[i] = a0[i]; b[i] = b0[i]; }
        } else {
            const T* src = row + (size_t)h * head_dim;
            load8(src + k, a);
            load8(src + k + half, b);
        }
        if (h < n_heads + n_kv_heads) {
            T* dst = h < n_heads ? q_out + ((size_t)n * n_heads + h) * head_dim
                                 : page_base + (size_t)(h - n_heads) * page_size * head_dim;
            float lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float c = cs[k + i], sn = cs[half + k + i];
                lo[i] = __fsub_rn(__fmul_rn(a[i], c), __fmul_rn(b[i], sn));
                hi[i] = __fadd_rn(__fmul_rn(b[i], c), __fmul_rn(a[i], sn));
            }
            store8(dst + k, lo);
            store8(dst + k + half, hi);
        } else {
            T* dst = page_base + kv_stride + (size_t)(h - n_heads - n_kv_heads) * page_size * head_dim;
            store8(dst + k, a);
            store8(dst + k + half, b);
        }
    }
}

// cs: null, or the step's table of angles [n_tokens, head_dim] (zi_rope_table of these positions and inv_freq); few
// tokens then take their cosines and sines from it.
ZI_EXPORT int zi_rope_append(const void* qkv, void* q_out, void* cache, int dtype, const int* tables,
                             const int* tok_seg, const int* pos, const float* inv_freq, int n_tokens,
                             int row_stride, int n_heads, int n_kv_heads, int head_dim, int page_size,
                             int max_blocks, long long page_stride, long long kv_stride, int write_kv,
                             const float* cs, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || (head_dim & 1)) return zi_fail("rope: head_dim=%d must be positive and even", head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0 || page_size <= 0) return zi_fail("rope: bad head counts or page size");
    const int total_heads = n_heads + 2 * n_kv_heads;
    if (total_heads > 65535) return zi_fail("rope: too many heads for one launch");
    if (cs && n_tokens <= 64 && head_dim <= 2048) {
        const int heads = n_heads + (write_kv ? 2 * n_kv_heads : 0);
        const int threads = ((head_dim / 2 + 31) / 32) * 32;
        ZI_DISPATCH(dtype, T, {
            rope_append_few_kernel<T><<<dim3(n_tokens, heads), threads, 0, stream>>>((const T*)qkv, (T*)q_out, (T*)cache, tables,
                tok_seg, pos, cs, row_stride, n_heads, n_kv_heads, head_dim, page_size, max_blocks, page_stride, kv_stride);
        });
        return zi_check_launch("rope_append");
    }
    const int hpb = n_tokens <= 64 ? 1 : total_heads;
    const int vec_align = dtype == ZI_BF16 ? 15 : 31;
    if (hpb != 1 && head_dim % 16 == 0 && row_stride % 8 == 0 && page_stride % 8 == 0 && kv_stride % 8 == 0 &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)cache) & vec_align) == 0) {
        const size_t smem8 = (size_t)head_dim * sizeof(float);
        ZI_DISPATCH(dtype, T, {
            rope_append_vec8_kernel<T><<<n_tokens, 128, smem8, stream>>>((const T*)qkv, (T*)q_out, (T*)cache, tables, tok_seg, pos,
                inv_freq, row_stride, n_heads, n_kv_heads, head_dim, page_size, max_blocks, page_stride, kv_stride, write_kv);
        });
        return zi_check_launch("rope_append");
    }
    dim3 grid(n_tokens, (total_heads + hpb - 1) / hpb);
    const int threads = hpb == 1 ? (head_dim >= 128 ? 64 : 32) : 256;
    const size_t smem = (size_t)head_dim * sizeof(float);
    ZI_DISPATCH(dtype, T, {
        zi_launch(rope_append_kernel<T>, grid, dim3(threads), smem, stream, (const T*)qkv, (T*)q_out, (T*)cache, tables,
                  tok_seg, pos, inv_freq, row_stride, n_heads, n_kv_heads, head_dim, page_size, max_blocks,
                  page_stride, kv_stride, write_kv, hpb);
    });
    return zi_check_launch("rope_append");
}

// cos and sin of every token's angles, once per step for all layers: out[n, k] = cos(pos[n] * inv_freq[k]),
// out[n, half + k] = sin(...), the same sincosf of the same float32 angle as the kernels above.
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq, float* __restrict__ out,
                                  int n_tokens, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    const int n = i / half, k = i - n * half;
    float s, c;
    sincosf((float)pos[n] * inv_freq[k], &s, &c);
    out[(size_t)n * 2 * half + k] = c;
    out[(size_t)n * 2 * half + half + k] = s;
}

ZI_EXPORT int zi_rope_table(const int* pos, const float* inv_freq, float* out, int n_tokens, int head_dim, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || (head_dim & 1)) return zi_fail("rope_table: head_dim=%d must be positive and even", head_dim);
    const int total = n_tokens * (head_dim / 2);
    rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(pos, inv_freq, out, n_tokens, head_dim / 2);
    return zi_check_launch("rope_table");
}

// ---------------------------------------------------------------------------------------
// SiLU-mul: out[n, j] = up * gate / (1 + exp(-gate)),  gate = x[n, j], up = x[n, inter + j]
// (src/backend/ops/swiglu/cpu/swiglu_cpu.cpp:13-20)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter, j = i - n * inter;
        const float g = to_f32<T>(x[n * 2 * inter + j]);
        const float u = to_f32<T>(x[n * 2 * inter + inter + j]);
        out[i] = from_f32<T>(u * g / (1.0f + expf(-g)));
    }
}

// 8 elements per thread with 16-byte loads and stores (inter % 8 == 0, 16-byte aligned rows).
template <typename T>
__global__ void silu_mul_vec8_kernel(const T* __restrict__ x, T* __restrict__ out, int inter8, size_t total8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / inter8, j = (i - n * inter8) * 8;
        const size_t inter = (size_t)inter8 * 8;
        float g[8], u[8], r[8];
        load8(x + n * 2 * inter + j, g);
        load8(x + n * 2 * inter + inter + j, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) r[e] = u[e] * g[e] / (1.0f + expf(-g[e]));
        store8(out + n * inter + j, r);
    }
}

ZI_EXPORT int zi_silu_mul(const void* gate_up, void* out, int dtype, int rows, int inter, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0) return zi_fail("silu_mul: width %d must be positive", inter);
    const size_t total = (size_t)rows * inter;
    const int threads = 256;
    if (inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 31) == 0) {
        const size_t total8 = total / 8;
        const size_t want = (total8 + threads - 1) / threads;
        const int nblocks = (int)(want > 148 * 32 ? 148 * 32 : want);
        ZI_DISPATCH(dtype, T, { silu_mul_vec8_kernel<T><<<nblocks, threads, 0, stream>>>((const T*)gate_up, (T*)out, inter / 8, total8); });
        return zi_check_launch("silu_mul");
    }
    const int blocks = (int)((total + threads - 1) / threads > 148 * 16 ? 148 * 16 : (total + threads - 1) / threads);
    ZI_DISPATCH(dtype, T, { silu_mul_kernel<T><<<blocks, threads, 0, stream>>>((const T*)gate_up, (T*)out, inter, total); });
    return zi_check_launch("silu_mul");
}

// ---------------------------------------------------------------------------------------
// Cast between float32 and bfloat16 (round to nearest even).
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}

ZI_EXPORT int zi_cast(const void* in, int in_dtype, void* out, int out_dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    ZI_DISPATCH(in_dtype, TI, ZI_DISPATCH(out_dtype, TO, {
        cast_kernel<TI, TO><<<blocks, threads, 0, stream>>>((const TI*)in, (TO*)out, (size_t)total);
    }););
    return zi_check_launch("cast");
}

// ---------------------------------------------------------------------------------------
// out = a + b, elementwise, in float32 with one rounding (src/backend/ops/add/cpu/add_cpu.cpp; the reference's GPU
// kernel adds in the storage type).  The engine folds its residual adds into the norm that follows them; this
// stands alone for callers of the op.
// ---------------------------------------------------------------------------------------
template <typename TA, typename TB, typename TO>
__global__ void add_kernel(const TA* __restrict__ a, const TB* __restrict__ b, TO* __restrict__ out, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32<TA>(a[i]) + to_f32<TB>(b[i]));
}

ZI_EXPORT int zi_add(const void* a, int a_dtype, const void* b, int b_dtype, void* out, int out_dtype, long long total,
                     cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    const long long want = (total + threads - 1) / threads;
    const int blocks = (int)(want > 148 * 16 ? 148 * 16 : want);
    ZI_DISPATCH(a_dtype, TA, ZI_DISPATCH(b_dtype, TB, ZI_DISPATCH(out_dtype, TO, {
        add_kernel<TA, TB, TO><<<blocks, threads, 0, stream>>>((const TA*)a, (const TB*)b, (TO*)out, (size_t)total);
    });););
    return zi_check_launch("add");
}
