// C[M,N] = X[M,K] . W[N,K]^T (+ bias[N]) for bfloat16 operands on the 5th-generation tensor cores:
// tcgen05.mma issued by one thread per CTA, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), the float32 accumulator in tensor memory (TMEM), read back
// with tcgen05.ld for the epilogue.  cta_group::1, no multicast.
//
// One CTA computes one 128 x BN tile of D = A . B^T, A and B both K-major ([rows, K] row-major):
//   normal  : A = X (tokens), B = W (outputs);  D[m, n] = C[m, n]                    (prefill, many rows)
//   swapped : A = W (outputs), B = X (tokens);  D[n, m] = C[m, n], written transposed (decode, few rows:
//             the 128-row side of the MMA is filled by weights, the narrow side by 16..256 tokens)
//
// Warp roles (6 warps): warp 0 issues TMA loads into a ring of STAGES buffers, warp 1 allocates TMEM and
// issues the MMAs, warps 2..5 are the epilogue (each reads the 32 TMEM lanes of its quadrant).
// Barriers: full[s] (TMA bytes landed), empty[s] (MMAs that read stage s retired, by tcgen05.commit),
// accum (all MMAs retired).  Every wait is bounded: after WAIT_LIMIT polls a role records where it gave
// up in `status`, the CTA skips what is left, frees its TMEM and returns.
//
// K is walked in blocks of 64 (one 128-byte swizzle atom per row); a tail of K % 64 is covered by the
// tensor map, which fills what lies outside the tensor with zeros, as it does for rows beyond M or N.
#include "zi_common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

ZI_DEFINE_LAST_ERROR(gemm_tcgen05)

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_WAIT_LIMIT (1u << 24)

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: true when the phase with `parity` completed; false after TC_WAIT_LIMIT polls (a fraction of a
// second), or as soon as another role of the CTA has given up.  test_wait never suspends the thread.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 1023) == 1023 && *gave_up) return false;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16), stored as TMA
// writes it with 128-byte swizzle: groups of 8 rows are 1024 bytes apart (stride byte offset), the leading
// byte offset is unused for swizzled K-major layouts (1), descriptor version 1, layout type 2 = SWIZZLE_128B.
// Fields: start address >> 4 in bits 0-13, LBO >> 4 in 16-29, SBO >> 4 in 32-45, version in 46-47, layout 61-63.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9 and 10-12 = 1), both K-major
// (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcParams {
    void* C;
    const bf16* bias;
    int* status;
    long long ldc;
    int rows_a, rows_b, K;      // rows of the A operand (128 per CTA), of the B operand (BN per CTA)
    int c_is_f32, swapped;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;                 // power of two >= 32 (BN is 16, 32, 64, 128 or 256)
    // the dynamic window starts 1024-aligned (checked on the host side by the alignment attribute above)
    unsigned char* stages = tc_smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + (size_t)STAGES * STAGE_BYTES);   // full[S], empty[S], accum
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * TC_BM, b0 = blockIdx.y * BN;
    const int k_blocks = (p.K + TC_BK - 1) / TC_BK;
    const uint32_t full0 = tc_smem_u32(bars), empty0 = tc_smem_u32(bars + STAGES), accum = tc_smem_u32(bars + 2 * STAGES);

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !mbar_wait(empty0 + 8 * s, ((kb / STAGES) - 1) & 1, &gave_up)) { atomicExch(p.status, 1); gave_up = 1; break; }
                const uint32_t sa = tc_smem_u32(stages + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d(sa, &map_a, kb * TC_BK, a0, full0 + 8 * s);
                tma_load_2d(sb, &map_b, kb * TC_BK, b0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(full0 + 8 * s, (kb / STAGES) & 1, &gave_up)) { atomicExch(p.status, 2); gave_up = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t sa = tc_smem_u32(stages + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)       // 16 k-values = 32 bytes further along the swizzled row
                    umma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);               // stage s may be refilled once these MMAs have read it
            }
            umma_commit(accum);                            // arrives when every MMA above has retired (at once if none ran)
        }
    } else {
        // epilogue: warp w owns TMEM lanes 32*(w % 4) .. +31, i.e. rows a0 + 32*(w % 4) + lane of the tile
        const int quad = warp & 3;
        const bool ok = __all_sync(0xffffffffu, mbar_wait(accum, 0, &gave_up));      // the same answer for the whole warp
        if (!ok && lane == 0) { atomicExch(p.status, 3); gave_up = 1; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const int ra = a0 + quad * 32 + lane;              // row of the A operand this thread holds
        if (ok && k_blocks > 0) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                tmem_ld16(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)c, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (ra >= p.rows_a) continue;
                if (!p.swapped) {
                    // D[m = ra][n = b0 + c + j]
                    const long long base = (long long)ra * p.ldc + b0 + c;
                    if (!p.c_is_f32 && b0 + c + 16 <= p.rows_b && (p.ldc & 7) == 0 &&
                        ((uintptr_t)p.C & 15) == 0) {             // a full group: two 16-byte stores
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]) + (p.bias ? __bfloat162float(p.bias[b0 + c + j]) : 0.0f);
                        store8(reinterpret_cast<bf16*>(p.C) + base, v);
                        store8(reinterpret_cast<bf16*>(p.C) + base + 8, v + 8);
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int n = b0 + c + j;
                        if (n >= p.rows_b) break;
                        float v = __uint_as_float(r[j]);
                        if (p.bias) v += __bfloat162float(p.bias[n]);
                        if (p.c_is_f32) reinterpret_cast<float*>(p.C)[base + j] = v;
                        else reinterpret_cast<bf16*>(p.C)[base + j] = __float2bfloat16_rn(v);
                    }
                } else {
                    // D[n = ra][m = b0 + c + j] -> C[m][n]; a warp writes 32 consecutive n for each m
                    const float bv = p.bias ? __bfloat162float(p.bias[ra]) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = b0 + c + j;
                        if (m >= p.rows_b) break;
                        const float v = __uint_as_float(r[j]) + bv;
                        if (p.c_is_f32) reinterpret_cast<float*>(p.C)[(long long)m * p.ldc + ra] = v;
                        else reinterpret_cast<bf16*>(p.C)[(long long)m * p.ldc + ra] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 tc_encode = nullptr;

static int tc_init() {
    if (tc_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return zi_fail("gemm_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    tc_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    return 0;
}

// [rows, K] row-major bfloat16 with row stride ld (elements); box = 64 k-values x box_rows rows, 128-byte swizzle.
static int tc_make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = tc_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return zi_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, ld %lld, box %d)", (int)r, rows, K, ld, box_rows);
    return 0;
}

template <int BN, int STAGES>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int tiles_a, int tiles_b, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return zi_fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    kernel<<<dim3(tiles_a, tiles_b), TC_THREADS, smem, stream>>>(ma, mb, p);
    return zi_check_launch("gemm_tcgen05");
}

// status: one int of device memory, zero before the launch; non-zero afterwards means a bounded wait ran out
// (1 = producer, 2 = MMA issuer, 3 = epilogue) and the output is not valid.
ZI_EXPORT int zi_gemm_tcgen05(const void* X, const void* W, const void* bias, void* C, int c_dtype, int* status, int M, int N,
                              int K, long long ldx, long long ldw, long long ldc, int swapped, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return zi_fail("gemm_tcgen05: K=%d must be positive", K);
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_tcgen05: K and the row strides must be multiples of 8 elements (16 bytes) for TMA; got K=%d ldx=%lld ldw=%lld", K, ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_tcgen05: operands must be 16-byte aligned");
    if (c_dtype != ZI_F32 && c_dtype != ZI_BF16) return zi_fail("gemm_tcgen05: unknown output dtype %d", c_dtype);
    if (!status) return zi_fail("gemm_tcgen05: a status word is required");
    if (tc_init()) return 1;
    TcParams p;
    p.C = C; p.bias = (const bf16*)bias; p.status = status; p.ldc = ldc; p.K = K;
    p.c_is_f32 = c_dtype == ZI_F32; p.swapped = swapped;
    const void* a_ptr = swapped ? W : X;
    const void* b_ptr = swapped ? X : W;
    const long long a_ld = swapped ? ldw : ldx, b_ld = swapped ? ldx : ldw;
    p.rows_a = swapped ? N : M;
    p.rows_b = swapped ? M : N;
    int bn;
    if (swapped) {
        if (M > 256) return zi_fail("gemm_tcgen05: the swapped form takes at most 256 rows of X, got %d", M);
        bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    } else {
        bn = N >= 128 ? 128 : N > 32 ? 64 : N > 16 ? 32 : 16;
    }
    CUtensorMap ma, mb;
    if (tc_make_map(&ma, a_ptr, p.rows_a, K, a_ld, TC_BM)) return 1;
    if (tc_make_map(&mb, b_ptr, p.rows_b, K, b_ld, bn)) return 1;
    const int tiles_a = (p.rows_a + TC_BM - 1) / TC_BM, tiles_b = (p.rows_b + bn - 1) / bn;
    if (tiles_b > 65535) return zi_fail("gemm_tcgen05: too many column tiles (%d)", tiles_b);
    switch (bn) {
        case 16: return tc_launch<16, 8>(ma, mb, p, tiles_a, tiles_b, stream);
        case 32: return tc_launch<32, 8>(ma, mb, p, tiles_a, tiles_b, stream);
        case 64: return tc_launch<64, 6>(ma, mb, p, tiles_a, tiles_b, stream);
        case 128: return tc_launch<128, 6>(ma, mb, p, tiles_a, tiles_b, stream);
        default: return tc_launch<256, 4>(ma, mb, p, tiles_a, tiles_b, stream);
    }
}
