// C[M,N] = X[M,K] . W[N,K]^T (+ bias[N]) for bfloat16 operands on the 5th-generation tensor cores:
// tcgen05.mma issued by one thread per CTA, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), the float32 accumulator in tensor memory (TMEM), read back
// with tcgen05.ld for the epilogue.  Single CTAs (cta_group::1) in the first two entry points, pairs of SMs
// (cta_group::2) in the third; no load uses cluster multicast.
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
#include "tcgen05.cuh"

ZI_DEFINE_LAST_ERROR(gemm_tcgen05)

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

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
        for (int kb = 0; kb < k_blocks; ++kb) {
            const int s = kb % STAGES;
            if (kb >= STAGES && !mbar_wait_warp(empty0 + 8 * s, ((kb / STAGES) - 1) & 1, &gave_up)) { if (lane == 0) { atomicExch(p.status, 1); gave_up = 1; } break; }
            if (elect_one()) {
                const uint32_t sa = tc_smem_u32(stages + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d(sa, &map_a, kb * TC_BK, a0, full0 + 8 * s);
                tma_load_2d(sb, &map_b, kb * TC_BK, b0, full0 + 8 * s);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
            const int s = kb % STAGES;
            if (!mbar_wait_warp(full0 + 8 * s, (kb / STAGES) & 1, &gave_up)) { if (lane == 0) { atomicExch(p.status, 2); gave_up = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (elect_one()) {
                const uint32_t sa = tc_smem_u32(stages + (size_t)s * STAGE_BYTES), sb = sa + A_BYTES;
                const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)       // 16 k-values = 32 bytes further along the swizzled row
                    umma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);               // stage s may be refilled once these MMAs have read it
            }
            __syncwarp();
        }
        if (elect_one()) umma_commit(accum);               // arrives when every MMA above has retired (at once if none ran)
        __syncwarp();
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

// ---- the persistent form for many rows -----------------------------------------------------------------
// One CTA per SM walks over 128 x BN tiles of C (BN a multiple of 16 up to 256, chosen per call).  The
// accumulator is double-buffered in TMEM (2 x 256 columns): while the epilogue warps read tile i out of
// one buffer, the MMA warp already fills the other with tile i+1, and the TMA ring runs on across tile
// borders.  Tiles are numbered with the row tile fastest, so the CTAs of one wave share a few column
// tiles of W (read once from HBM, then from L2) and all of X.
//
// The B operand of a tile is loaded as two boxes of BN/2 rows.  plain: rows n0.. and n0+BN/2.. of W.
// silu_mul: W = [gate; up] stacked, rows n0.. of the gate half and the same rows of the up half, so the
// accumulator holds gate in columns [0, BN/2) and up in [BN/2, BN) for the same BN/2 outputs, and the
// epilogue writes silu(gate) * up without the two halves ever reaching memory.
#define TP_STAGES 4
#define TP_A_BYTES (TC_BM * TC_BK * 2)
#define TP_B_BYTES (256 * TC_BK * 2)
#define TP_STAGE_BYTES (TP_A_BYTES + TP_B_BYTES)
#define TP_SMEM ((size_t)TP_STAGES * TP_STAGE_BYTES + (2 * TP_STAGES + 4) * 8 + 16)

struct TpParams {
    void* C;
    const bf16* bias;
    int* status;
    long long ldc;
    int M, N, K;                // N: columns of C (silu_mul: the intermediate size)
    int c_is_f32, silu_mul;
    int bn;                     // accumulator columns per tile
    int up_row0;                // silu_mul: first row of the up half in W
    int tiles_m, tiles_n;
};

__device__ __forceinline__ void tp_store16(const TpParams& p, long long base, int n, const float (&v)[16]) {
    // 16 consecutive columns n .. n+15 of one row of C
    if (!p.c_is_f32 && n + 16 <= p.N && ((base & 7) == 0) && (((uintptr_t)p.C & 15) == 0)) {
        store8(reinterpret_cast<bf16*>(p.C) + base, v);
        store8(reinterpret_cast<bf16*>(p.C) + base + 8, v + 8);
        return;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (n + j >= p.N) break;
        if (p.c_is_f32) reinterpret_cast<float*>(p.C)[base + j] = v[j];
        else reinterpret_cast<bf16*>(p.C)[base + j] = __float2bfloat16_rn(v[j]);
    }
}

// The epilogue of one tile for one thread: row m of C, accumulator columns at taddr.  A tcgen05.ld takes
// several hundred clocks while the MMAs of the next tile keep TMEM busy, so the loads of 64 columns are
// issued together before one wait, not 16 by 16.
__device__ __forceinline__ void tp_epilogue_row(const TpParams& p, uint32_t taddr, int m, int nt) {
    const int half = p.bn >> 1;
    if (p.silu_mul) {
        const int n0 = nt * half;
#pragma unroll 1
        for (int c0 = 0; c0 < half; c0 += 32) {
            uint32_t g[1][32], u[1][32];
#pragma unroll
            for (int q = 0; q < 1; ++q)
                if (c0 + 32 * q < half) { tmem_ld32(taddr + (uint32_t)(c0 + 32 * q), g[q]); tmem_ld32(taddr + (uint32_t)(half + c0 + 32 * q), u[q]); }
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (m >= p.M) continue;
#pragma unroll
            for (int q = 0; q < 1; ++q) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = c0 + 32 * q + 16 * h;
                    if (c >= half || n0 + c >= p.N) continue;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float gv = __uint_as_float(g[q][16 * h + j]);
                        v[j] = __fdividef(gv, 1.0f + __expf(-gv)) * __uint_as_float(u[q][16 * h + j]);
                    }
                    tp_store16(p, (long long)m * p.ldc + n0 + c, n0 + c, v);
                }
            }
        }
    } else {
        const int n0 = nt * p.bn;
#pragma unroll 1
        for (int c0 = 0; c0 < p.bn; c0 += 64) {
            uint32_t r[2][32];
#pragma unroll
            for (int q = 0; q < 2; ++q)
                if (c0 + 32 * q < p.bn) tmem_ld32(taddr + (uint32_t)(c0 + 32 * q), r[q]);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            if (m >= p.M) continue;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = c0 + 32 * q + 16 * h;
                    if (c >= p.bn || n0 + c >= p.N) continue;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        v[j] = __uint_as_float(r[q][16 * h + j]) + ((p.bias && n0 + c + j < p.N) ? __bfloat162float(p.bias[n0 + c + j]) : 0.0f);
                    tp_store16(p, (long long)m * p.ldc + n0 + c, n0 + c, v);
                }
            }
        }
    }
}

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TpParams p) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    unsigned char* stages = tc_smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + (size_t)TP_STAGES * TP_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TP_STAGES + 4);
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.K + TC_BK - 1) / TC_BK;
    const int n_tiles = p.tiles_m * p.tiles_n;
    const int half = p.bn >> 1;
    const uint32_t full0 = tc_smem_u32(bars), empty0 = tc_smem_u32(bars + TP_STAGES);
    const uint32_t tfull0 = tc_smem_u32(bars + 2 * TP_STAGES), tempty0 = tc_smem_u32(bars + 2 * TP_STAGES + 2);

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < TP_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        const uint32_t stage_tx = TP_A_BYTES + (uint32_t)p.bn * TC_BK * 2;
        uint32_t kbg = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile % p.tiles_m) * TC_BM, nt = tile / p.tiles_m;
            const int row_b0 = p.silu_mul ? nt * half : nt * p.bn;
            const int row_b1 = p.silu_mul ? p.up_row0 + nt * half : nt * p.bn + half;
            for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                const uint32_t s = kbg % TP_STAGES;
                if (kbg >= TP_STAGES && !mbar_wait_warp(empty0 + 8 * s, ((kbg / TP_STAGES) - 1) & 1, &gave_up)) {
                    if (lane == 0) { atomicExch(p.status, 1); gave_up = 1; }
                    ok = false; break;
                }
                if (elect_one()) {
                    const uint32_t sa = tc_smem_u32(stages + (size_t)s * TP_STAGE_BYTES), sb = sa + TP_A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, stage_tx);
                    tma_load_2d(sa, &map_a, kb * TC_BK, m0, full0 + 8 * s);
                    tma_load_2d(sb, &map_b, kb * TC_BK, row_b0, full0 + 8 * s);
                    tma_load_2d(sb + (uint32_t)half * TC_BK * 2, &map_b, kb * TC_BK, row_b1, full0 + 8 * s);
                }
                __syncwarp();
            }
        }
        if (!ok || gave_up) {
            // copies that were started but never consumed: let them land before the CTA's memory goes away
            const uint32_t last = kbg < TP_STAGES ? kbg : TP_STAGES;
            for (uint32_t i = 0; i < last; ++i) {
                const uint32_t g = kbg - 1 - i, s = g % TP_STAGES;
                mbar_wait(full0 + 8 * s, (g / TP_STAGES) & 1, nullptr);
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc = umma_idesc_bf16(TC_BM, p.bn);
        uint32_t kbg = 0;
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
            const uint32_t buf = it & 1;
            if (it >= 2 && !mbar_wait_warp(tempty0 + 8 * buf, ((it >> 1) - 1) & 1, &gave_up)) {
                if (lane == 0) { atomicExch(p.status, 4); gave_up = 1; }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t tmem_d = tmem_base + buf * 256u;
            for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                const uint32_t s = kbg % TP_STAGES;
                if (!mbar_wait_warp(full0 + 8 * s, (kbg / TP_STAGES) & 1, &gave_up)) {
                    if (lane == 0) { atomicExch(p.status, 2); gave_up = 1; }
                    ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (elect_one()) {
                    const uint32_t sa = tc_smem_u32(stages + (size_t)s * TP_STAGE_BYTES), sb = sa + TP_A_BYTES;
                    const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                    if (kb == k_blocks - 1) umma_commit(tfull0 + 8 * buf);
                }
                __syncwarp();
            }
        }
    } else {
        const int quad = warp & 3;
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            const uint32_t buf = it & 1;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, (it >> 1) & 1, &gave_up));
            if (!ok) { if (lane == 0) { atomicExch(p.status, 3); gave_up = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int m = (tile % p.tiles_m) * TC_BM + quad * 32 + lane, nt = tile / p.tiles_m;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256u;
            tp_epilogue_row(p, taddr, m, nt);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tempty0 + 8 * buf) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- the persistent form on pairs of SMs (cta_group::2) -------------------------------------------------
// Two CTAs of a cluster work on one 256 x BN tile: each loads its own 128 rows of X and only HALF of the
// tile's rows of W (BN/2), the MMA issued by the first CTA of the pair reads both halves out of both
// shared memories, and each CTA ends up with its 128 rows of the accumulator in its own TMEM.  A CTA thus
// pulls 32 KB instead of 48 KB from L2 for the same 128 x 256 x 64 products, which is what bounds the
// single-CTA form, and the ring holds six stages instead of four.
//   silu_mul: the first CTA loads the tile's gate rows, the second its up rows.
// Barriers: the TMA loads of both CTAs complete on the first CTA's full[s]; tcgen05.commit signals
// empty[s] and tmem_full[b] in both CTAs; the epilogue warps of both arrive on the first CTA's tmem_empty[b].
#define TQ_STAGES 6
#define TQ_STAGE_BYTES (2 * TP_A_BYTES)
#define TQ_SMEM ((size_t)TQ_STAGES * TQ_STAGE_BYTES + (2 * TQ_STAGES + 4) * 8 + 16)

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TpParams p) {
    extern __shared__ __align__(1024) unsigned char tc_smem[];
    unsigned char* stages = tc_smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + (size_t)TQ_STAGES * TQ_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TQ_STAGES + 4);
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int first_tile = (int)cluster_id_x(), tile_step = (int)cluster_count_x();
    const int k_blocks = (p.K + TC_BK - 1) / TC_BK;
    const int n_tiles = p.tiles_m * p.tiles_n;             // tiles_m counts 256-row tiles here
    const int half = p.bn >> 1;
    const uint32_t full0 = tc_smem_u32(bars), empty0 = tc_smem_u32(bars + TQ_STAGES);
    const uint32_t tfull0 = tc_smem_u32(bars + 2 * TQ_STAGES), tempty0 = tc_smem_u32(bars + 2 * TQ_STAGES + 2);

    if (threadIdx.x == 0) {
        gave_up = 0;
        for (int s = 0; s < TQ_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {       // one warp of each CTA of the pair takes part; both get the same columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                    // the peer's barriers exist before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        const uint32_t stage_tx = TP_A_BYTES + (uint32_t)half * TC_BK * 2;      // per CTA
        uint32_t kbg = 0;
        bool ok = true;
        for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step) {
            const int m0 = (tile % p.tiles_m) * 256 + (int)rank * TC_BM, nt = tile / p.tiles_m;
            const int row_b = p.silu_mul ? (rank == 0 ? nt * half : p.up_row0 + nt * half) : nt * p.bn + (int)rank * half;
            for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                const uint32_t s = kbg % TQ_STAGES;
                if (kbg >= TQ_STAGES && !mbar_wait_warp(empty0 + 8 * s, ((kbg / TQ_STAGES) - 1) & 1, &gave_up)) {
                    if (lane == 0) { atomicExch(p.status, 1); gave_up = 1; }
                    ok = false; break;
                }
                if (elect_one()) {
                    const uint32_t sa = tc_smem_u32(stages + (size_t)s * TQ_STAGE_BYTES), sb = sa + TP_A_BYTES;
                    const uint32_t lead_full = mapa_shared(full0 + 8 * s, 0);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * stage_tx);
                    tma_load_2d_pair(sa, &map_a, kb * TC_BK, m0, lead_full);
                    tma_load_2d_pair(sb, &map_b, kb * TC_BK, row_b, lead_full);
                }
                __syncwarp();
            }
        }
        if (rank == 0 && (!ok || gave_up)) {
            // copies of either CTA that were started but never consumed: let them land before the pair leaves
            const uint32_t last = kbg < TQ_STAGES ? kbg : TQ_STAGES;
            for (uint32_t i = 0; i < last; ++i) {
                const uint32_t g = kbg - 1 - i, s = g % TQ_STAGES;
                mbar_wait(full0 + 8 * s, (g / TQ_STAGES) & 1, nullptr);
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            const uint32_t idesc = umma_idesc_bf16(256, p.bn);
            uint32_t kbg = 0;
            bool ok = true;
            int it = 0;
            for (int tile = first_tile; tile < n_tiles && ok; tile += tile_step, ++it) {
                const uint32_t buf = it & 1;
                if (it >= 2 && !mbar_wait_warp(tempty0 + 8 * buf, ((it >> 1) - 1) & 1, &gave_up)) {
                    if (lane == 0) { atomicExch(p.status, 4); gave_up = 1; }
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * 256u;
                for (int kb = 0; kb < k_blocks; ++kb, ++kbg) {
                    const uint32_t s = kbg % TQ_STAGES;
                    if (!mbar_wait_warp(full0 + 8 * s, (kbg / TQ_STAGES) & 1, &gave_up)) {
                        if (lane == 0) { atomicExch(p.status, 2); gave_up = 1; }
                        ok = false; break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    if (elect_one()) {
                        const uint32_t sa = tc_smem_u32(stages + (size_t)s * TQ_STAGE_BYTES), sb = sa + TP_A_BYTES;
                        const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sb);
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)
                            umma_bf16_pair(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        umma_commit_pair(empty0 + 8 * s);
                        if (kb == k_blocks - 1) umma_commit_pair(tfull0 + 8 * buf);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        const int quad = warp & 3;
        int it = 0;
        for (int tile = first_tile; tile < n_tiles; tile += tile_step, ++it) {
            const uint32_t buf = it & 1;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * buf, (it >> 1) & 1, &gave_up));
            if (!ok) { if (lane == 0) { atomicExch(p.status, 3); gave_up = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int m = (tile % p.tiles_m) * 256 + (int)rank * TC_BM + quad * 32 + lane, nt = tile / p.tiles_m;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * 256u;
            tp_epilogue_row(p, taddr, m, nt);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(mapa_shared(tempty0 + 8 * buf, 0)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                    // neither CTA's memory goes away while the other may read it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------------
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

// Cost of one 16-deep MMA step of a 128 x bn tile in SM clocks: the tensor pipe needs bn / 2, shared memory
// has to deliver the A (4 KB) and B (32 bn bytes) operands at 128 bytes a clock.
static int tp_step_cost(int bn) { const int pipe = bn / 2, smem = 32 + bn / 4; return pipe > smem ? pipe : smem; }

// C[M,N] = X[M,K] . W^T with the persistent kernel.  epilogue 0: W is [N,K], optional bias[N].
// epilogue 1 (silu_mul): W is [2N,K] = [gate; up], C = silu(X.gate^T) * (X.up^T), no bias.
// bn_hint: 0 lets the call choose the tile width; else a multiple of 16 (32 for silu_mul) up to 256.
ZI_EXPORT int zi_gemm_tcgen05_tiles(const void* X, const void* W, const void* bias, void* C, int c_dtype, int* status, int M, int N,
                                    int K, long long ldx, long long ldw, long long ldc, int epilogue, int bn_hint, int num_sms,
                                    cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return zi_fail("gemm_tcgen05: K=%d must be positive", K);
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_tcgen05: K and the row strides must be multiples of 8 elements (16 bytes) for TMA; got K=%d ldx=%lld ldw=%lld", K, ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_tcgen05: operands must be 16-byte aligned");
    if (c_dtype != ZI_F32 && c_dtype != ZI_BF16) return zi_fail("gemm_tcgen05: unknown output dtype %d", c_dtype);
    if (epilogue != 0 && epilogue != 1) return zi_fail("gemm_tcgen05: unknown epilogue %d", epilogue);
    if (epilogue == 1 && bias) return zi_fail("gemm_tcgen05: the silu_mul epilogue takes no bias");
    if (!status) return zi_fail("gemm_tcgen05: a status word is required");
    if (num_sms <= 0) return zi_fail("gemm_tcgen05: num_sms=%d must be positive", num_sms);
    if (tc_init()) return 1;
    const int step = epilogue == 1 ? 32 : 16;              // silu_mul: both halves are multiples of 16 columns
    const int tiles_m = (M + TC_BM - 1) / TC_BM;
    int bn = bn_hint;
    if (bn == 0) {
        long long best = -1;
        for (int cand = 256; cand >= step; cand -= step) {
            const int cols = epilogue == 1 ? cand / 2 : cand;
            const long long tiles = (long long)tiles_m * ((N + cols - 1) / cols);
            const long long cost = ((tiles + num_sms - 1) / num_sms) * tp_step_cost(cand);
            if (best < 0 || cost < best) { best = cost; bn = cand; }
        }
    }
    if (bn < step || bn > 256 || bn % step) return zi_fail("gemm_tcgen05: tile width %d must be a multiple of %d up to 256", bn, step);
    TpParams p;
    p.C = C; p.bias = (const bf16*)bias; p.status = status; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.c_is_f32 = c_dtype == ZI_F32; p.silu_mul = epilogue; p.bn = bn; p.up_row0 = N;
    p.tiles_m = tiles_m;
    const int cols = epilogue == 1 ? bn / 2 : bn;
    p.tiles_n = (N + cols - 1) / cols;
    const long long n_tiles = (long long)p.tiles_m * p.tiles_n;
    if (n_tiles > 0x7fffffffLL) return zi_fail("gemm_tcgen05: too many tiles");
    CUtensorMap ma, mb;
    if (tc_make_map(&ma, X, M, K, ldx, TC_BM)) return 1;
    if (tc_make_map(&mb, W, epilogue == 1 ? 2LL * N : N, K, ldw, bn / 2)) return 1;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TP_SMEM);
        if (e != cudaSuccess) return zi_fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", TP_SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    const int grid = (int)(n_tiles < num_sms ? n_tiles : num_sms);
    gemm_tcgen05_persistent_kernel<<<grid, TC_THREADS, TP_SMEM, stream>>>(ma, mb, p);
    return zi_check_launch("gemm_tcgen05_persistent");
}

static int tq_step_cost(int bn) { const int pipe = bn / 2, smem = 32 + bn / 8; return pipe > smem ? pipe : smem; }

// The same product on pairs of SMs (256-row tiles).  Arguments as zi_gemm_tcgen05_tiles, without num_sms:
// the number of pairs that fit on the device at once is asked of the runtime.
ZI_EXPORT int zi_gemm_tcgen05_pairs(const void* X, const void* W, const void* bias, void* C, int c_dtype, int* status, int M, int N,
                                    int K, long long ldx, long long ldw, long long ldc, int epilogue, int bn_hint, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return zi_fail("gemm_tcgen05: K=%d must be positive", K);
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return zi_fail("gemm_tcgen05: K and the row strides must be multiples of 8 elements (16 bytes) for TMA; got K=%d ldx=%lld ldw=%lld", K, ldx, ldw);
    if (((uintptr_t)X | (uintptr_t)W) & 15) return zi_fail("gemm_tcgen05: operands must be 16-byte aligned");
    if (c_dtype != ZI_F32 && c_dtype != ZI_BF16) return zi_fail("gemm_tcgen05: unknown output dtype %d", c_dtype);
    if (epilogue != 0 && epilogue != 1) return zi_fail("gemm_tcgen05: unknown epilogue %d", epilogue);
    if (epilogue == 1 && bias) return zi_fail("gemm_tcgen05: the silu_mul epilogue takes no bias");
    if (!status) return zi_fail("gemm_tcgen05: a status word is required");
    if (tc_init()) return 1;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(TC_THREADS); cfg.dynamicSmemBytes = TQ_SMEM; cfg.stream = stream; cfg.attrs = attr; cfg.numAttrs = 1;
    static int max_pairs = 0;
    if (max_pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TQ_SMEM);
        if (e != cudaSuccess) return zi_fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", TQ_SMEM, cudaGetErrorString(e));
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cfg.gridDim = dim3(sms > 1 ? sms & ~1 : 2);
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel, &cfg);
        if (e != cudaSuccess || n <= 0) return zi_fail("gemm_tcgen05: no pair of CTAs of this kernel fits on the device (%s)", cudaGetErrorString(e));
        max_pairs = n;
    }
    const int step = epilogue == 1 ? 32 : 16;
    const int tiles_m = (M + 255) / 256;
    int bn = bn_hint;
    if (bn == 0) {
        long long best = -1;
        for (int cand = 256; cand >= step; cand -= step) {
            const int cols = epilogue == 1 ? cand / 2 : cand;
            const long long tiles = (long long)tiles_m * ((N + cols - 1) / cols);
            const long long cost = ((tiles + max_pairs - 1) / max_pairs) * tq_step_cost(cand);
            if (best < 0 || cost < best) { best = cost; bn = cand; }
        }
    }
    if (bn < step || bn > 256 || bn % step) return zi_fail("gemm_tcgen05: tile width %d must be a multiple of %d up to 256", bn, step);
    TpParams p;
    p.C = C; p.bias = (const bf16*)bias; p.status = status; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.c_is_f32 = c_dtype == ZI_F32; p.silu_mul = epilogue; p.bn = bn; p.up_row0 = N;
    p.tiles_m = tiles_m;
    const int cols = epilogue == 1 ? bn / 2 : bn;
    p.tiles_n = (N + cols - 1) / cols;
    const long long n_tiles = (long long)p.tiles_m * p.tiles_n;
    if (n_tiles > 0x7fffffffLL) return zi_fail("gemm_tcgen05: too many tiles");
    CUtensorMap ma, mb;
    if (tc_make_map(&ma, X, M, K, ldx, TC_BM)) return 1;
    if (tc_make_map(&mb, W, epilogue == 1 ? 2LL * N : N, K, ldw, bn / 2)) return 1;
    cfg.gridDim = dim3(2 * (unsigned)(n_tiles < max_pairs ? n_tiles : max_pairs));
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, ma, mb, p);
    if (e != cudaSuccess) return zi_fail("gemm_tcgen05_pairs: launch failed: %s", cudaGetErrorString(e));
    return zi_check_launch("gemm_tcgen05_pairs");
}
