// Causal attention of portions of prompts over the paged cache on the 5th-generation tensor cores
// (bfloat16, head size 64 or 128, pages of a power of two from 8 to 128 tokens).
//
// One CTA takes 128 consecutive query rows of one portion and one head and walks over the keys in tiles of 128:
//   S = Q . K^T      tcgen05.mma, 128 x 128; Q sits in TMEM (A operand), K in shared memory; S in TMEM, two buffers
//   P = exp2(S - m)  four warps, one thread per query row: tcgen05.ld the row, running maximum and sum in
//                    registers, P written back to TMEM as bfloat16 pairs (tcgen05.st), the A operand of the next product.
//                    This is what a tile's time goes to (about 1,900 clocks against 1,024 for its two products):
//                    three-input maxima, packed float32 pairs, and a quarter of the exponentials by arithmetic
//                    instead of the special-function unit keep it as short as the schedulers allow.  Two threads
//                    per row (eight warps) were measured and are no faster: the two warps of a scheduler are in
//                    the same phase at the same time and share its pipes.
//   O += P . V       tcgen05.mma, 128 x head size, V straight from its pages as an MN-major operand, O in TMEM
// With both A operands in TMEM, shared memory only takes the K and V tiles from TMA and feeds them to the
// tensor core once each; with A operands in shared memory as well its bandwidth, not the tensor pipe, set the pace.
// K and V tiles come page by page through one 5-d tensor map of the layer's cache (128-byte swizzle): the lanes
// of the producer warp each issue one page-half, the block table gives the page.
//
// O stays in TMEM for the whole row of tiles.  Its rescaling when the maximum grows is done lazily: only when
// a row's maximum exceeds the value in use by more than 2^8, the four warps multiply their O rows in TMEM
// (tcgen05.ld / st) and their sums by 2^(old - new); otherwise P is simply computed against the older maximum,
// which changes no result, since sum and O share it and the final division cancels it.
//
// Order of the MMAs: QK(0), QK(1), QK(2), PV(0), QK(3), PV(1), ...: the scores of a tile are asked for as soon as
// the buffer of the tile two before is free, so they are there when the softmax warps finish the tile between.
// Barriers (all waits bounded, as in the matrix product): q_full, k_full/k_empty[3], v_full/v_empty[3],
// s_full/s_empty[2], p_full, pv_done.
//
// Keys a row must not see (beyond its position, before its window) get probability 0.  Cache slots that hold
// nothing yet are multiplied by 0 as well, so the pool must never hold NaN bit patterns: it is allocated
// zeroed, and pages that are used again hold finite values.
#include "tcgen05.cuh"

ZI_DEFINE_LAST_ERROR(attention_tcgen05)

#define FA_ROWS 128
#define FA_KEYS 128
#define FA_THREADS 256           // warps: 0, 6 and 7 load, 1 issues the MMAs, 2..5 are the softmax
#define FA_LAZY_LOG2 8.0f
#define FA_KSTAGES 3
#define FA_VSTAGES 3
#define FA_NBARS (1 + 2 * FA_KSTAGES + 2 * FA_VSTAGES + 6)
// shared memory: the K and V stages, the barriers and the TMEM address, then (128-byte aligned) the stage of Q / O rows
#define FA_STAGE_OFFSET(hd) ((((FA_KSTAGES + FA_VSTAGES) * FA_KEYS * (hd) * 2 + FA_NBARS * 8 + 16) + 127) / 128 * 128)

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float fa_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 in one 64-bit register and the packed arithmetic of sm_100 on them: one instruction for two values.
__device__ __forceinline__ uint64_t f2_pack(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) { uint64_t d; asm("sub.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b)); return d; }
// The exponentials of a tile set the pace of its softmax.  Measured on one scheduler of an SM (32 rows x 128
// keys): the special-function unit takes 8 clocks for a warp's ex2, and the instructions around it (scale, sum,
// maximum, conversion) do not hide behind it: 1,580 clocks a tile with scalar arithmetic, against 1,024 for the
// tile's two products.  With packed arithmetic and every FA_POLY_MOD-th pair of exponentials computed without
// that unit it is 1,220.  2^x by arithmetic: round x to the nearest integer n by adding 1.5 * 2^23 (n is then in
// the low mantissa bits), a cubic for 2^f on f = x - n in [-0.5, 0.5] (relative error 7.5e-5, a fiftieth of what
// rounding P to bfloat16 adds), and n added into the exponent field.  x is held at -125 from below, so a masked
// key gets 2^-125 instead of 0 there: nothing beside a row's other terms.
#ifndef FA_POLY_MOD
#define FA_POLY_MOD 4
#endif
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// MN-major operand (V: rows are keys, the head dimension is contiguous), 128-byte swizzle: groups of 8 keys are
// 1024 bytes apart (stride offset); the two 64-wide halves of a 128-wide head are 128 keys x 128 bytes apart
// (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lead_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)(lead_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// A operand in TMEM: row m in lane m, elements 2c and 2c+1 of a row in column c; 16 elements of K = 8 columns.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

struct FaParams {
    const bf16* q;
    bf16* out;
    const int* tables;
    const int* tiles;
    const int* pos;
    int* status;
    int n_heads, n_kv_heads, page_size, max_blocks, window;
    float scale2;                  // softmax scale x log2(e)
};

// TMEM columns of a CTA: two score buffers, the output, and the two A operands (bfloat16 pairs, one row per lane)
#define FA_COL_S 0
#define FA_COL_O 256
#define FA_COL_Q 384
#define FA_COL_P 448

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_kv, const FaParams p) {
    constexpr int HH = HD / 64;                               // 64-wide halves of a head
    constexpr int SUB = FA_KEYS * 128;                        // bytes of one [128 rows x 128 bytes] sub-tile
    constexpr int TILE_BYTES = FA_KEYS * HD * 2;              // one K or V tile
    extern __shared__ __align__(1024) unsigned char fa_smem[];
    unsigned char* sK = fa_smem;                              // FA_KSTAGES stages
    unsigned char* sV = sK + FA_KSTAGES * TILE_BYTES;         // FA_VSTAGES stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + FA_VSTAGES * TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FA_NBARS);
    // Rows of Q on their way in and rows of O on their way out: a thread owns a row, but memory wants a warp on
    // consecutive bytes (a thread reading or writing its own row 16 bytes at a time touches 32 lines with every
    // instruction: 2,000 clocks for Q and 3,200 for O, a quarter of a 16-tile CTA's time).  16-byte chunk c of row
    // r sits at chunk c ^ (r & 7), so both ways of walking it are free of bank conflicts.
    constexpr int CH = HD * 2 / 16;                           // 16-byte chunks of a row
    unsigned char* stage = fa_smem + FA_STAGE_OFFSET(HD);
    __shared__ volatile int gave_up;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t b0 = tc_smem_u32(bars);
    const uint32_t q_full = b0, k_full = q_full + 8, k_empty = k_full + 8 * FA_KSTAGES, v_full = k_empty + 8 * FA_KSTAGES,
                   v_empty = v_full + 8 * FA_VSTAGES, s_full = v_empty + 8 * FA_VSTAGES, s_empty = s_full + 16,
                   p_full = s_empty + 16, pv_done = p_full + 8;
    const int tile = gridDim.y - 1 - blockIdx.y;              // heads run fastest, so the heavy tiles of all heads start first
    const int n0 = p.tiles[tile * 3], rows = p.tiles[tile * 3 + 1], seg = p.tiles[tile * 3 + 2];
    const int h = blockIdx.x, kvh = h / (p.n_heads / p.n_kv_heads);
    const int p0 = p.pos[n0], p_last = p0 + rows - 1;         // positions of a tile are consecutive
    const int lo_tile = (p.window > 0 && p0 - p.window + 1 > 0) ? p0 - p.window + 1 : 0;
    const int kt_begin = lo_tile / FA_KEYS, n_kt = p_last / FA_KEYS - kt_begin + 1;

    // the softmax warps ask for their 32 rows of Q before anything else, CH requests a lane in flight together
    uint4 q_in[CH];
    if (warp >= 2 && warp < 6) {
#pragma unroll
        for (int k = 0; k < CH; ++k) {
            const int idx = k * 32 + lane, r = (warp & 3) * 32 + idx / CH, c = idx % CH;
            q_in[k] = r < rows ? *reinterpret_cast<const uint4*>(p.q + ((size_t)(n0 + r) * p.n_heads + h) * HD + c * 8) : make_uint4(0, 0, 0, 0);
        }
    }
    if (threadIdx.x == 0) gave_up = 0;
    if (threadIdx.x < FA_NBARS) {                             // one barrier a thread
        const uint32_t bar = b0 + 8 * threadIdx.x;
        const bool per_warp = bar == q_full || bar == s_empty || bar == s_empty + 8 || bar == p_full;   // one arrival per softmax warp
        mbar_init(bar, per_warp ? 4 : 1);
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

    if (warp == 0 || warp >= 6) {
        // ---- producers: K(0), K(1), K(2), V(0), K(3), V(1), ...: a K tile is asked for two tiles ahead of its V ----
        // A lane's TMA instruction takes some 60 clocks to issue and a warp's lanes issue one after another, so the
        // 16 or 32 page-halves of a tile are dealt to three warps; all of them follow the same barriers.
        const int prod = warp == 0 ? 0 : warp - 5;            // 0..2
        const int* table = p.tables + (size_t)seg * p.max_blocks;
        const int ppt = FA_KEYS / p.page_size;                // pages per tile
        int k_issued = 0, v_issued = 0;
        // one page-half per lane (at most 16 pages x 2 halves).  A tile's page numbers are read from the block table
        // one tile ahead, so that load's latency does not sit between a freed stage and its refill.
        const int my_pg = lane / HH, my_hh = lane - my_pg * HH;
        const bool my_op = lane < ppt * HH && lane % 3 == prod;
        auto page_of = [&](int j) -> int {
            const int blk = (kt_begin + j) * ppt + my_pg;
            return (my_op && j < n_kt && blk < p.max_blocks) ? table[blk] : -1;      // -1: outside the map, reads zeros
        };
        auto load_tile = [&](int j, int kv, int page) {
            const int st = kv ? (j % FA_VSTAGES) : (j % FA_KSTAGES);
            const uint32_t bar = (kv ? v_full : k_full) + 8 * st;
            if (prod == 0 && elect_one()) mbar_expect_tx(bar, TILE_BYTES);
            __syncwarp();
            if (my_op) {
                const uint32_t dst = tc_smem_u32(kv ? sV : sK) + st * TILE_BYTES + my_hh * SUB + my_pg * p.page_size * 128;
                tma_load_5d(dst, &map_kv, my_hh * 64, 0, kvh, kv, page, bar);
            }
            __syncwarp();
        };
        bool ok = true;
        int page_next = page_of(0), page_prev = -1, page_prev2 = -1;
        for (int j = 0; j <= n_kt + 1 && ok; ++j) {
            const int page_cur = page_next;
            page_next = page_of(j + 1);
            if (j < n_kt) {                   // K(j)
                if (j >= FA_KSTAGES && !mbar_wait_warp(k_empty + 8 * (j % FA_KSTAGES), ((j / FA_KSTAGES) - 1) & 1, &gave_up)) { ok = false; break; }
                load_tile(j, 0, page_cur);
                k_issued = j + 1;
            }
            if (j >= 2) {                     // V(j - 2)
                const int jv = j - 2;
                if (jv >= FA_VSTAGES && !mbar_wait_warp(v_empty + 8 * (jv % FA_VSTAGES), ((jv / FA_VSTAGES) - 1) & 1, &gave_up)) { ok = false; break; }
                load_tile(jv, 1, page_prev2);
                v_issued = jv + 1;
            }
            page_prev2 = page_prev;
            page_prev = page_cur;
        }
        if (!ok && lane == 0) { atomicExch(p.status, 11); gave_up = 1; }
        if (gave_up && prod == 0) {      // copies in flight: let them land before the CTA's memory goes away
            for (int j = k_issued > FA_KSTAGES ? k_issued - FA_KSTAGES : 0; j < k_issued; ++j)
                mbar_wait(k_full + 8 * (j % FA_KSTAGES), (j / FA_KSTAGES) & 1, nullptr);
            for (int j = v_issued > FA_VSTAGES ? v_issued - FA_VSTAGES : 0; j < v_issued; ++j)
                mbar_wait(v_full + 8 * (j % FA_VSTAGES), (j / FA_VSTAGES) & 1, nullptr);
        }
    } else if (warp == 1) {
        // ---- MMA issuer: QK(0), QK(1), QK(2), PV(0), QK(3), PV(1), ... --------------------------------------------
        // Both products take their A operand (Q, P) from TMEM, so shared memory serves only K and V.  The loops
        // stay lean (descriptors are a base plus a constant, the lane is elected per instruction): a 128 x 128 x 16
        // product lasts 64 clocks and its issue must not take longer.
        constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_ROWS, FA_KEYS);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_ROWS, HD) | (1u << 16);      // B operand MN-major
        const uint32_t tq = tmem_base + FA_COL_Q, tp = tmem_base + FA_COL_P, to = tmem_base + FA_COL_O;
        const uint64_t dk_base = umma_desc_sw128(tc_smem_u32(sK)), dv_base = umma_desc_mn_sw128(tc_smem_u32(sV), SUB);
        bool ok = mbar_wait_warp(q_full, 0, &gave_up);
        auto issue_qk = [&](int j) -> bool {
            const int st = j & 1, kst = j % FA_KSTAGES;
            if (!mbar_wait_warp(k_full + 8 * kst, (j / FA_KSTAGES) & 1, &gave_up)) return false;
            if (j >= 2 && !mbar_wait_warp(s_empty + 8 * st, ((j >> 1) - 1) & 1, &gave_up)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint64_t dk = dk_base + (uint64_t)(kst * (TILE_BYTES >> 4));
            const uint32_t ts = tmem_base + FA_COL_S + st * 128u;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                if (elect_one()) umma_bf16_ts(ts, tq + ks * 8, dk + (uint64_t)(((ks >> 2) * SUB + (ks & 3) * 32) >> 4), idesc_qk, ks > 0 ? 1u : 0u);
            if (elect_one()) { umma_commit(s_full + 8 * st); umma_commit(k_empty + 8 * kst); }
            __syncwarp();
            return true;
        };
        auto issue_pv = [&](int j) -> bool {
            const int vst = j % FA_VSTAGES;
            if (!mbar_wait_warp(p_full, j & 1, &gave_up)) return false;
            if (!mbar_wait_warp(v_full + 8 * vst, (j / FA_VSTAGES) & 1, &gave_up)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint64_t dv = dv_base + (uint64_t)(vst * (TILE_BYTES >> 4));
#pragma unroll
            for (int ks = 0; ks < FA_KEYS / 16; ++ks)
                if (elect_one()) umma_bf16_ts(to, tp + ks * 8, dv + (uint64_t)((ks * 2048) >> 4), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            if (elect_one()) { umma_commit(pv_done); umma_commit(v_empty + 8 * vst); }
            __syncwarp();
            return true;
        };
        if (ok) ok = issue_qk(0);
        if (ok && n_kt > 1) ok = issue_qk(1);
        for (int j = 0; j < n_kt && ok; ++j) {
            if (j + 2 < n_kt) ok = issue_qk(j + 2);       // as soon as the softmax has taken S(j) out of its buffer
            if (ok) ok = issue_pv(j);
        }
        if (!ok && lane == 0) { atomicExch(p.status, 13); gave_up = 1; }
    } else {
        // ---- softmax: one thread per query row --------------------------------------------------------------------
        const int quad = warp & 3, r = quad * 32 + lane;
        const int qpos = p0 + r;
        const int lo = (p.window > 0 && qpos - p.window + 1 > 0) ? qpos - p.window + 1 : 0;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        {   // the rows of Q go through shared memory into TMEM, two bfloat16 per column; rows beyond the tile are zero
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int idx = k * 32 + lane, rr = quad * 32 + idx / CH, c = idx % CH;
                *reinterpret_cast<uint4*>(stage + rr * (HD * 2) + ((c ^ (rr & 7)) * 16)) = q_in[k];
            }
            __syncwarp();
#pragma unroll
            for (int c = 0; c < HD / 2; c += 32) {
                uint32_t w[32];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + r * (HD * 2) + (((c / 4 + i) ^ (r & 7)) * 16));
                    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
                }
                tmem_st32(lane_base + FA_COL_Q + c, w);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(q_full) : "memory");
        }
        float m_run = -INFINITY, m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        uint32_t s[4][32];
        for (int j = 0; j < n_kt; ++j) {
            const int st = j & 1, key0 = (kt_begin + j) * FA_KEYS;
            if (!mbar_wait_warp(s_full + 8 * st, (j >> 1) & 1, &gave_up)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) tmem_ld32(lane_base + FA_COL_S + st * 128u + q4 * 32, s[q4]);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s_empty + 8 * st) : "memory");
            // keys this row must not see; whole tiles below the diagonal and inside the window need no test
            const bool need_mask = key0 + FA_KEYS - 1 > p0 || (p.window > 0 && key0 < p_last - p.window + 1);
            if (need_mask) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int kp = key0 + q4 * 32 + c;
                        if (kp > qpos || kp < lo) s[q4][c] = __float_as_uint(-INFINITY);
                    }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains of three-input maxima
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    mx[(c >> 1) & 3] = fa_max3(mx[(c >> 1) & 3], __uint_as_float(s[q4][c]), __uint_as_float(s[q4][c + 1]));
            const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float m_new = fmaxf(m_run, m_tile * p.scale2);
            const bool grow = m_new > m_used + FA_LAZY_LOG2;            // false while both are -inf
            const bool any_grow = __any_sync(0xffffffffu, grow);
            const float f = grow ? fa_exp2(m_used - m_new) : 1.0f;      // 0 when nothing was seen before
            if (grow) m_used = m_new;
            m_run = m_new;
            const float mu = m_used == -INFINITY ? 0.0f : m_used;       // nothing seen yet: every p is exp2(-inf) = 0
            uint64_t sums2[2] = {0ull, 0ull};                            // two pairs of partial sums
            uint32_t pk[2][32];                                          // the row of P, two bfloat16 per word
            const uint64_t scale22 = f2_pack(p.scale2, p.scale2), nmu2 = f2_pack(-mu, -mu), magic2 = f2_pack(12582912.0f, 12582912.0f);
            const uint64_t c3 = f2_pack(0.055171459913253784f, 0.055171459913253784f), c2 = f2_pack(0.2426108568906784f, 0.2426108568906784f),
                           c1 = f2_pack(0.6932609677314758f, 0.6932609677314758f), c0 = f2_pack(0.9999281167984009f, 0.9999281167984009f);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    uint64_t x = f2_fma(f2_pack(__uint_as_float(s[q4][2 * i]), __uint_as_float(s[q4][2 * i + 1])), scale22, nmu2);
                    float e0, e1;
                    if (FA_POLY_MOD > 0 && (q4 * 16 + i) % (FA_POLY_MOD > 0 ? FA_POLY_MOD : 1) == 0) {
                        float x0, x1;
                        f2_unpack(x, x0, x1);
                        x = f2_pack(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
                        const uint64_t t = f2_add(x, magic2);
                        const uint64_t f = f2_sub(x, f2_sub(t, magic2));
                        uint64_t q = f2_fma(c3, f, c2);
                        q = f2_fma(q, f, c1);
                        q = f2_fma(q, f, c0);
                        float q0, q1, t0, t1;
                        f2_unpack(q, q0, q1), f2_unpack(t, t0, t1);
                        e0 = __uint_as_float(__float_as_uint(t0) * 0x800000u + __float_as_uint(q0));
                        e1 = __uint_as_float(__float_as_uint(t1) * 0x800000u + __float_as_uint(q1));
                    } else {
                        float x0, x1;
                        f2_unpack(x, x0, x1);
                        e0 = fa_exp2(x0), e1 = fa_exp2(x1);
                    }
                    sums2[i & 1] = f2_add(sums2[i & 1], f2_pack(e0, e1));
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                    pk[q4 >> 1][(q4 & 1) * 16 + i] = *reinterpret_cast<uint32_t*>(&b2);
                }
            float sums[4];
            f2_unpack(sums2[0], sums[0], sums[1]), f2_unpack(sums2[1], sums[2], sums[3]);
            // only now the product of the tile before must be done: it read P and wrote O
            if (j > 0) {
                if (!mbar_wait_warp(pv_done, (j - 1) & 1, &gave_up)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (any_grow) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + FA_COL_O + c, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st32(lane_base + FA_COL_O + c, o);
                    }
                }
            }
            l = l * f + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
            tmem_st32(lane_base + FA_COL_P, pk[0]);
            tmem_st32(lane_base + FA_COL_P + 32, pk[1]);
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(p_full) : "memory");
        }
        if (ok) ok = mbar_wait_warp(pv_done, (n_kt - 1) & 1, &gave_up);
        if (!ok) {
            if (lane == 0) { atomicExch(p.status, 14); gave_up = 1; }
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            // the whole row of O with one wait (the registers of the scores are free now)
#pragma unroll
            for (int c = 0; c < HD; c += 32) tmem_ld32(lane_base + FA_COL_O + c, s[c / 32]);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            __syncwarp();                                     // every lane has read its row of Q from the stage
#pragma unroll
            for (int c = 0; c < HD; c += 8) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(s[c / 32][(c & 31) + k]) * inv;
                store8(reinterpret_cast<bf16*>(stage + r * (HD * 2) + (((c / 8) ^ (r & 7)) * 16)), v);
            }
            __syncwarp();
#pragma unroll
            for (int k = 0; k < CH; ++k) {                    // the warp's 32 rows, consecutive lanes on consecutive bytes
                const int idx = k * 32 + lane, rr = quad * 32 + idx / CH, c = idx % CH;
                if (rr < rows)
                    *reinterpret_cast<uint4*>(p.out + ((size_t)(n0 + rr) * p.n_heads + h) * HD + c * 8) =
                        *reinterpret_cast<const uint4*>(stage + rr * (HD * 2) + ((c ^ (rr & 7)) * 16));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------------------
// tiles: int32 [n_tiles, 3] = (first token, rows <= 128, segment).  status: one int of device memory, zero before;
// non-zero afterwards means a bounded wait ran out (11 producer, 12/13 MMA issuer, 14 softmax).
ZI_EXPORT int zi_prefill_attention_tcgen05(const void* q, const void* cache, void* out, const int* tables, const int* tiles,
                                           const int* pos, int* status, int n_tokens, int n_tiles, int n_heads, int n_kv_heads,
                                           int head_dim, int page_size, int max_blocks, long long n_pages, long long page_stride,
                                           long long kv_stride, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) return zi_fail("prefill_attention_tcgen05: head_dim %d is not 64 or 128", head_dim);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return zi_fail("prefill_attention_tcgen05: %d heads over %d key-value heads", n_heads, n_kv_heads);
    if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1))) return zi_fail("prefill_attention_tcgen05: page size %d is not a power of two from 8 to 128", page_size);
    if (n_tiles > 65535) return zi_fail("prefill_attention_tcgen05: %d tiles are more than one launch takes", n_tiles);
    if (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15) return zi_fail("prefill_attention_tcgen05: q, cache and out must be 16-byte aligned");
    if ((page_stride | kv_stride) & 7) return zi_fail("prefill_attention_tcgen05: cache strides must be multiples of 8 elements");
    if (!status) return zi_fail("prefill_attention_tcgen05: a status word is required");
    if (tc_init()) return 1;
    CUtensorMap mkv;
    if (tc_map_kv_pages(&mkv, cache, head_dim, page_size, n_kv_heads, n_pages, page_stride, kv_stride, page_size)) return 1;
    FaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.tables = tables; p.tiles = tiles; p.pos = pos; p.status = status;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.max_blocks = max_blocks; p.window = window;
    p.scale2 = scale * 1.4426950408889634f;
    const dim3 grid(n_heads, n_tiles);
    const size_t smem = (size_t)FA_STAGE_OFFSET(head_dim) + (size_t)FA_ROWS * head_dim * 2;
    cudaError_t e;
    if (head_dim == 128) {
        e = cudaFuncSetAttribute(prefill_attention_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return zi_fail("prefill_attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        prefill_attention_tcgen05_kernel<128><<<grid, FA_THREADS, smem, stream>>>(mkv, p);
    } else {
        e = cudaFuncSetAttribute(prefill_attention_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return zi_fail("prefill_attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        prefill_attention_tcgen05_kernel<64><<<grid, FA_THREADS, smem, stream>>>(mkv, p);
    }
    return zi_check_launch("prefill_attention_tcgen05");
}
