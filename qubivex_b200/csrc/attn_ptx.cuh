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

// Plain shared-memory accesses by 32-bit shared address (a pointer kept in a struct loses its address space and
// turns into generic loads, which wait on the long scoreboard).  Volatile: kept in order with the barrier waits.
__device__ __forceinline__ float4 lds128(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, float2 v) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}

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

// ---- one tile of 16 positions for one group of <= 8 query heads (one warp) ----------------------
// The arithmetic both 16-bit decode-attention kernels share, so that the streaming kernel and the fixed-scratch
// one cannot drift apart.  `kt` / `vt`: shared-memory addresses of the tile's key rows and value rows (the
// pool's native layout: rows of D 16-bit elements, 16-byte chunks XORed with (row & 7)); `vt_rows`: the value
// rows again as a generic pointer; `valid` <= 16 positions of the tile are filled.  qf / ql: the queries as
// B-operand fragments, value and remainder (this lane: head lane >> 2, dims 16 ks + 2 (lane & 3) + {0,1,8,9}).
// State per lane: o = O^T fragments (dims 16 mt + lane >> 2 (+8), heads 2 (lane & 3) (+1)), running maxima
// m0 / m1 (base 2, scaled) and row sums l0 / l1 of heads 2t and 2t + 1 over the positions this lane has seen.
// PASSES: bit 0 = the queries go through the tensor cores as value + remainder, bit 1 = the probabilities do.
// The caller orders its own accesses to the stage (wait before, release after); the rows cleared here are made
// visible to the bulk copy that reuses the stage (fence.proxy.async) before the function returns.
#ifndef QVX_LAZY_RESCALE
#define QVX_LAZY_RESCALE 1
#endif
template <int DT, int D, int PASSES>
__device__ __forceinline__ void attend_tile(uint32_t kt, uint32_t vt, uint8_t* vt_rows, uint32_t valid, uint32_t lane,
                                            const uint32_t (&qf)[D / 16][2], const uint32_t (&ql)[D / 16][2], float scale_log2,
                                            float (&o)[D / 16][4], float& m0, float& m1, float& l0, float& l1) {
    const uint32_t g = lane >> 2;
    const uint32_t mid = lane >> 3, r8 = lane & 7;
    const uint32_t k_row = r8 + 8 * (mid & 1), k_chunk = mid >> 1;  // keys: A = K
    const uint32_t v_row = r8 + 8 * (mid >> 1), v_chunk = mid & 1;  // values: A = V^T (ldmatrix.trans)
    // S^T = K Q^T.  Four accumulators (even and odd 16-dim steps, value and remainder pass): the chains of
    // dependent tensor-core ops are a quarter as long as one accumulator's would be.
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, sr[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < D / 16; ks++) {
        uint32_t af[4];
        ldmatrix_x4(kt + k_row * (D * 2) + (((2 * ks + k_chunk) ^ (k_row & 7)) << 4), af);
        mma_16816<DT>(sc[ks & 1], af, qf[ks][0], qf[ks][1]);
        if constexpr ((PASSES & 1) != 0) mma_16816<DT>(sr[ks & 1], af, ql[ks][0], ql[ks][1]);
    }
    float s[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        s[i] = sc[0][i] + sc[1][i];
        if constexpr ((PASSES & 1) != 0) s[i] += sr[0][i] + sr[1][i];
    }
    if (valid < TILE) {
        // The tail of the last block: unwritten slots hold whatever the pool held before.
        if (g >= valid) { s[0] = -INFINITY; s[1] = -INFINITY; }
        if (g + 8 >= valid) { s[2] = -INFINITY; s[3] = -INFINITY; }
        // 0 * NaN is NaN: clear the value rows no probability reaches.
        for (uint32_t c = valid * (D * 2 / 16) + lane; c < TILE * (D * 2 / 16); c += 32)
            *reinterpret_cast<uint4*>(vt_rows + c * 16) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();  // these generic writes precede the bulk copy that reuses the stage
        __syncwarp();
    }
    // Online softmax in base 2; this lane sees heads 2t, 2t+1 at positions g, g+8.
    float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
    }
    const float mn0 = fmaxf(m0, mx0 * scale_log2), mn1 = fmaxf(m1, mx1 * scale_log2);
    const float al0 = ex2(m0 - mn0), al1 = ex2(m1 - mn1);
    m0 = mn0; m1 = mn1;
    const float p0 = ex2(fmaf(s[0], scale_log2, -mn0)), p1 = ex2(fmaf(s[1], scale_log2, -mn1));
    const float p2 = ex2(fmaf(s[2], scale_log2, -mn0)), p3 = ex2(fmaf(s[3], scale_log2, -mn1));
    l0 = fmaf(l0, al0, p0 + p2);
    l1 = fmaf(l1, al1, p1 + p3);
    // P^T as the B operand: (position g; heads 2t,2t+1) -> (head g; positions 2t,2t+1).
    uint32_t ph0, pl0, ph1, pl1;
    split16<DT>(p0, p1, ph0, pl0);
    split16<DT>(p2, p3, ph1, pl1);
    const uint32_t pb0 = movmatrix_trans(ph0), pb1 = movmatrix_trans(ph1);
    uint32_t pc0 = 0, pc1 = 0;
    if constexpr ((PASSES & 2) != 0) { pc0 = movmatrix_trans(pl0); pc1 = movmatrix_trans(pl1); }
    // O^T = O^T * alpha + V^T P^T.  The running maxima settle after a sequence's first tiles: when no lane's
    // moved, every factor is 1 and the multiplications are left out (x * 1.0f is x: the bits are the same).
    const bool rescale = QVX_LAZY_RESCALE ? __any_sync(0xffffffffu, al0 != 1.0f || al1 != 1.0f) : true;
#pragma unroll
    for (int mt = 0; mt < D / 16; mt++) {
        if (rescale) { o[mt][0] *= al0; o[mt][1] *= al1; o[mt][2] *= al0; o[mt][3] *= al1; }
        uint32_t vf[4];
        ldmatrix_x4_trans(vt + v_row * (D * 2) + (((2 * mt + v_chunk) ^ (v_row & 7)) << 4), vf);
        mma_16816<DT>(o[mt], vf, pb0, pb1);
        if constexpr ((PASSES & 2) != 0) mma_16816<DT>(o[mt], vf, pc0, pc1);
    }
}

// ---- the chunks of one (sequence, group) merged by one CTA, in chunk order ---------------------------
// p0: nch partial results, each acc[8][d], m[8], l[8] (8 d + 16 floats); out: the group's rows [nheads][d] of the
// output; scratch: (16 nch + 8) floats of shared memory; every thread of the CTA (nthreads of them) calls it,
// after a fence that makes the partials visible.  The merge is latency bound (a few KiB from the L2), so it is
// two rounds of independent loads: every chunk's (m, l) into shared memory, then the weighted sums with 16-byte
// loads, eight chunks in flight per thread.
__device__ __forceinline__ void merge_chunks_in_order(const float* p0, uint32_t nch, uint32_t nheads, uint32_t d, float* out,
                                                      float* scratch, uint32_t nthreads) {
    const uint32_t stride = 8 * d + 16;
    float* msm = scratch;             // [nch][8] maxima, then weights
    float* lsm = scratch + nch * 8;   // [nch][8] row sums
    float* Lsm = lsm + nch * 8;       // [8]
    for (uint32_t i = threadIdx.x; i < nch * 16; i += nthreads) {
        const uint32_t c = i >> 4, j = i & 15;
        const float v = __ldcg(p0 + (size_t)c * stride + 8 * d + j);
        if (j < 8) msm[c * 8 + j] = v; else lsm[c * 8 + j - 8] = v;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        const uint32_t h = threadIdx.x;
        float M = -INFINITY, L = 0.f;
        for (uint32_t c = 0; c < nch; c++) M = fmaxf(M, msm[c * 8 + h]);
        for (uint32_t c = 0; c < nch; c++) {
            const float w = ex2(msm[c * 8 + h] - M);
            msm[c * 8 + h] = w;
            L = fmaf(lsm[c * 8 + h], w, L);
        }
        Lsm[h] = L;
    }
    __syncthreads();
    const uint32_t d4 = d >> 2;
    for (uint32_t i = threadIdx.x; i < nheads * d4; i += nthreads) {
        const uint32_t h = i / d4, x = (i % d4) * 4;
        const float* p = p0 + h * d + x;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t c = 0;
        for (; c + 8 <= nch; c += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = __ldcg(reinterpret_cast<const float4*>(p + (size_t)(c + u) * stride));
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float w = msm[(c + u) * 8 + h];
                acc.x = fmaf(v[u].x, w, acc.x); acc.y = fmaf(v[u].y, w, acc.y);
                acc.z = fmaf(v[u].z, w, acc.z); acc.w = fmaf(v[u].w, w, acc.w);
            }
        }
        for (; c < nch; c++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(p + (size_t)c * stride));
            const float w = msm[c * 8 + h];
            acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
            acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
        }
        const float L = Lsm[h];
        *reinterpret_cast<float4*>(out + (size_t)h * d + x) = make_float4(acc.x / L, acc.y / L, acc.z / L, acc.w / L);
    }
}

// ---- a work item's header -----------------------------------------------------------------
struct Item {
    uint32_t seq, tokens, head0, nheads, kv_head, part, part0, nch, counter;
};

}  // namespace qvx
