// Building blocks of the kernels that drive the 5th-generation tensor cores directly: mbarriers with bounded
// waits, TMA tile loads, tcgen05.mma / commit / ld / st wrappers, shared-memory and instruction descriptors, and
// the host side of tensor maps.  Included by the .cu files that use them; everything is static or inline.
#pragma once
#include "zi_common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <map>
#include <mutex>
#include <tuple>

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
        if ((it & 1023) == 1023 && gave_up && *gave_up) return false;
    }
    return false;
}
// One lane of a converged warp.  The issuing roles run their loops with the whole warp and elect the lane per
// instruction: from a divergent branch (if (lane == 0)) every tcgen05.mma took about 100 clocks to issue and
// stalled the issuer, which a 128 x 256 x 16 product (128 clocks) cannot hide.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, gave_up));      // one answer for the whole warp
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
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

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_id_x() { uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;\n" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_count_x() { uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;\n" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have retired
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}


// ---- host side: tensor maps -----------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 tc_encode = nullptr;

static inline int tc_init() {
    if (tc_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return zi_fail("tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    tc_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
    return 0;
}

// [rows, K] row-major bfloat16 with row stride ld (elements); box = 64 k-values x box_rows rows, 128-byte swizzle.
static inline int tc_make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = tc_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return zi_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, ld %lld, box %d)", (int)r, rows, K, ld, box_rows);
    return 0;
}


// A layer's slice of the paged cache as a 5-d tensor: (head_dim, token in page, key-value head, k|v, page), with
// boxes of 64 elements x box_rows tokens, 128-byte swizzle.  Element (page, kv, kvh, off, d) lives at
// cache + page*page_stride + kv*kv_stride + (kvh*page_size + off)*head_dim + d.  A page coordinate outside
// [0, n_pages) reads zeros.  Maps are kept per (pointer, geometry): a layer's cache comes back every step.
typedef std::tuple<const void*, long long, long long, long long, long long, long long> TcMapKey;
static std::map<TcMapKey, CUtensorMap> tc_kv_maps;
static std::mutex tc_kv_maps_lock;

static inline int tc_map_kv_pages(CUtensorMap* out, const void* cache, int head_dim, int page_size, int n_kv_heads, long long n_pages,
                                  long long page_stride, long long kv_stride, int box_rows, int box_kv = 1) {
    // box_kv 2: one box holds the keys and the values of its rows (the keys' rows first)
    std::lock_guard<std::mutex> g(tc_kv_maps_lock);
    const TcMapKey key(cache, head_dim * 1024LL + box_rows + (box_kv == 2 ? 512 : 0), page_size, n_kv_heads * (1LL << 32) + n_pages, page_stride, kv_stride);
    auto it = tc_kv_maps.find(key);
    if (it == tc_kv_maps.end()) {
        if (tc_kv_maps.size() > 4096) tc_kv_maps.clear();
        cuuint64_t dims[5] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, 2, (cuuint64_t)n_pages};
        cuuint64_t strides[4] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2, (cuuint64_t)kv_stride * 2, (cuuint64_t)page_stride * 2};
        cuuint32_t box[5] = {64, (cuuint32_t)box_rows, 1, (cuuint32_t)(box_kv == 2 ? 2 : 1), 1};
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUtensorMap m;
        CUresult r = tc_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(cache), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return zi_fail("paged cache tensor map: cuTensorMapEncodeTiled failed with code %d (head %d, page %d, box rows %d, kv heads %d, pages %lld, strides %lld %lld)",
                           (int)r, head_dim, page_size, box_rows, n_kv_heads, n_pages, page_stride, kv_stride);
        it = tc_kv_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar) : "memory");
}
