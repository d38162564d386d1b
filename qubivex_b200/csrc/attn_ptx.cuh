// PTX wrappers and argument structs shared by the decode-attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qvx_common.cuh"

namespace qvx {

constexpr int TILE = 16;              // positions per tile
constexpr uint32_t NO_PART = 0xffffffffu;
// Polls a bounded wait makes before it gives up (with the back-off below: around a second).  A test build
// makes it small so that a wait can be seen to run out.
#ifndef QVX_WAIT_LIMIT
#define QVX_WAIT_LIMIT (1u << 20)
#endif
constexpr uint32_t WAIT_LIMIT = QVX_WAIT_LIMIT;

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Global -> this CTA's shared memory, completion counted in bytes on `bar`.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
// L2 eviction priorities: the KV stream is read once and should leave the L2 first; what a launch
// writes for its own later use (partial results) should stay.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// bulk_g2s with an L2 eviction priority for the lines it reads.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
// Asks the L2 to fetch `bytes` (a multiple of 16) at `src` (16-byte aligned); nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(__cvta_generic_to_global(src)), "r"(bytes) : "memory");
}
// 16 bytes global -> shared through the L2, asynchronously: no register holds the data meanwhile.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(__cvta_generic_to_global(src)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void st_global_hint(float4* addr, float4 v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(__cvta_generic_to_global(addr)), "f"(v.x),
                 "f"(v.y), "f"(v.z), "f"(v.w), "l"(policy)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after WAIT_LIMIT polls and reports it instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 1024) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
template <int DT>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (DT == QVX_BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}
template <int DT>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if constexpr (DT == QVX_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}
// x = hi + lo with hi the nearest 16-bit value and lo the rounded remainder: two tensor-core
// passes then carry ~16 bits of mantissa instead of 8 (bf16) or 11 (f16).
template <int DT>
__device__ __forceinline__ void split16(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    if constexpr (DT == QVX_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
        float2 hf = __bfloat1622float2(h);
        __nv_bfloat162 l = __floats2bfloat162_rn(x0 - hf.x, x1 - hf.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    } else {
        __half2 h = __floats2half2_rn(x0, x1);
        float2 hf = __half22float2(h);
        __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    }
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- kernel arguments --------------------------------------------------------------------
struct SplitArgs {
    const uint8_t* pool;
    const float* q;             // [token][head][d]
    float* out;                 // [token][head][d]
    float* partials;            // n_parts x (8*d + 16): acc[8][d], m[8], l[8]
    uint32_t* counters;         // one per split (sequence, group): arrivals so far; zero between launches
    const uint32_t* items;      // n_items x item_words: header, then the item's block ids
    int* status;                // a kernel that gave up a wait leaves a code here
    uint64_t block_bytes;
    uint32_t page_bytes, row_bytes, tiles_per_block, heads, d, item_words;
    float scale_log2;           // (1 / sqrt(d)) * log2(e)
};

struct Item {
    uint32_t seq, tokens, head0, nheads, kv_head, part, part0, nch, counter;
};
__device__ __forceinline__ Item load_item(const uint32_t* w) {
    uint4 a = *reinterpret_cast<const uint4*>(w), b = *reinterpret_cast<const uint4*>(w + 4);
    Item it;
    it.seq = a.x; it.tokens = a.y; it.head0 = a.z; it.nheads = a.w & 0xffffu; it.kv_head = a.w >> 16;
    it.part = b.x; it.part0 = b.y; it.nch = b.z; it.counter = b.w;
    return it;
}


}  // namespace qvx
