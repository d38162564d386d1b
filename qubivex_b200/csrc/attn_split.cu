// Paged decode attention, the fast path: GQA-grouped, online (flash-style) softmax, split
// over the context; the CTA that finishes a sequence's last split merges all of them, in
// split order, so the sum order is fixed whichever CTA does it.
//
// Computes what `attn_decode.comp` (crates/qubivex-backend-vulkan/shaders/attn_decode.comp:60-175)
// and the gather + `attend` of the CPU device (crates/qubivex-backend-cpu/src/sim.rs:400-429,
// crates/qubivex-compute/src/math.rs:142-155) compute, in another operation order: results
// agree within a tolerance, not bit for bit (the reference's own audit measured that an
// online softmax cannot be bit-identical, docs/engineering/VULKAN_EXECUTION_AUDIT.md:2031-2061).
//
// Work item (one CTA of 4 warps): one (sequence, kv head, group of <= 8 query heads) and up
// to `chunk` consecutive blocks of that sequence's table.  Chunk boundaries depend on the
// sequence's own length and a constant only, never on the batch or the SM count, so a
// sequence's result is the same whatever else shares the launch.
//
// Data movement: the native pool layout keeps the keys and the values of one (block, kv head)
// as two contiguous pages, rows pre-swizzled (16-byte chunk index XOR (slot & 7)).  Each
// warp streams its own tiles of 16 positions: lane 0 issues two bulk async copies
// (cp.async.bulk, global -> shared, completion on an mbarrier) per tile into the warp's own
// ring of stages, so no warp ever waits for another inside the loop, and a shared-memory
// image read with ldmatrix is bank-conflict free without any repacking.
// The kernel is HBM bound: per position per kv head it reads 2*d*e bytes and does 4*d*G flops.
//
// 16-bit pools: QK^T and PV run on the tensor cores with the roles swapped so nothing is
// padded: S^T[16 positions x 8 heads] = K[16 x d] * Q^T[d x 8] (m16n8k16, K is the A operand
// straight from the page), and O^T[d x 8] = V^T[d x 16] * P^T[16 x 8] (V through
// ldmatrix.trans, P transposed in registers by movmatrix).  f32 pools use the CUDA cores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "qvx_common.cuh"

namespace qvx {

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int TILE = 16;              // positions per tile
constexpr uint32_t NO_PART = 0xffffffffu;
constexpr uint32_t WAIT_LIMIT = 1u << 20;
// Status word values a kernel can leave (0 = fine).
constexpr int STATUS_WAIT_TIMEOUT = 1;

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

// Shared memory per CTA: WARPS rings of `stages` stages (a stage = a key tile then a value
// tile, 16 rows each), the f32 path's query and probability scratch, the mbarriers.  After
// the loop every ring is reused for its warp's result (m[8], l[8], acc[8][d]).
struct SmemPlan {
    uint32_t tile_bytes, stage_bytes, stages, ring_bytes, q_off, p_off, bar_off, total;
};
__host__ __device__ inline SmemPlan smem_plan(uint32_t row_bytes, uint32_t d, bool f32path) {
    SmemPlan p;
    p.tile_bytes = TILE * row_bytes;
    p.stage_bytes = 2 * p.tile_bytes;
    p.stages = 16384 / p.stage_bytes;
    if (p.stages < 2) p.stages = 2;
    if (p.stages > 8) p.stages = 8;
    p.ring_bytes = p.stages * p.stage_bytes;
    uint32_t off = WARPS * p.ring_bytes;
    p.q_off = off;
    if (f32path) off += 8 * d * 4;
    p.p_off = off;
    if (f32path) off += WARPS * TILE * 8 * 4;
    p.bar_off = off;
    off += WARPS * 8 * 8;
    p.total = off;
    return p;
}

// The per-warp stream of tiles of one item.
struct TileStream {
    uint32_t ring, bars, stages, stage_bytes, tile_bytes;  // shared addresses / sizes
    const uint8_t* base;  // pool + kv head offset
    uint64_t block_bytes;
    uint32_t page_bytes, tiles_per_block, my_block;  // my_block: block id of this lane's tile
    uint32_t warp, lane;

    __device__ __forceinline__ void issue(uint32_t it) {
        uint32_t tau = warp + WARPS * it;
        uint32_t blk = __shfl_sync(0xffffffffu, my_block, it & 31);
        if (lane == 0) {
            uint32_t st = it % stages;
            uint32_t bar = bars + st * 8, dst = ring + st * stage_bytes;
            const uint8_t* src = base + (uint64_t)blk * block_bytes + (uint64_t)(tau % tiles_per_block) * tile_bytes;
            fence_proxy_async();
            mbar_expect_tx(bar, stage_bytes);
            bulk_g2s(dst, src, tile_bytes, bar);
            bulk_g2s(dst + tile_bytes, src + page_bytes, tile_bytes, bar);
        }
    }
};

// Merges the four warps' results (left in shared memory) and writes either the final output
// (a sequence that fits one item) or this item's partial result.  The CTA that delivers the
// last partial of a (sequence, group) then merges all of them in chunk order: nobody waits,
// the arrival counter only tells the last one that it is the last.
__device__ __forceinline__ void merge_and_store(const SplitArgs& a, const Item& it, const float* res,
                                                uint32_t res_stride_f, uint32_t d, float* scratch) {
    // res + w * res_stride_f: m[8], l[8], acc[8][d]
    for (uint32_t i = threadIdx.x; i < it.nheads * d; i += THREADS) {
        uint32_t h = i / d, x = i % d;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) M = fmaxf(M, res[w * res_stride_f + h]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            const float* r = res + w * res_stride_f;
            float wgt = ex2(r[h] - M);
            acc = fmaf(r[16 + h * d + x], wgt, acc);
            l = fmaf(r[8 + h], wgt, l);
        }
        if (it.part == NO_PART) {
            a.out[((size_t)it.seq * a.heads + it.head0 + h) * d + x] = acc / l;
        } else {
            float* p = a.partials + (size_t)it.part * (8 * d + 16);
            p[h * d + x] = acc;
            if (x == 0) { p[8 * d + h] = M; p[8 * d + 8 + h] = l; }
        }
    }
    if (it.part == NO_PART) return;
    __shared__ uint32_t s_last;
    __threadfence();  // this thread's partial is visible device-wide before the arrival is counted
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(a.counters + it.counter, 1u) == it.nch - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The merge is latency bound (a few KiB from L2), so it is arranged as two rounds of
    // independent loads: every chunk's (m, l) into shared memory, then the weighted sums with
    // 16-byte loads, eight chunks in flight per thread.
    const uint32_t stride = 8 * d + 16, nch = it.nch;
    const float* p0 = a.partials + (size_t)it.part0 * stride;
    float* msm = scratch;             // [nch][8] maxima, then weights
    float* lsm = scratch + nch * 8;   // [nch][8] row sums
    float* Lsm = lsm + nch * 8;       // [8]
    for (uint32_t i = threadIdx.x; i < nch * 16; i += THREADS) {
        uint32_t c = i >> 4, j = i & 15;
        float v = __ldcg(p0 + (size_t)c * stride + 8 * d + j);
        if (j < 8) msm[c * 8 + j] = v; else lsm[c * 8 + j - 8] = v;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        const uint32_t h = threadIdx.x;
        float M = -INFINITY, L = 0.f;
        for (uint32_t c = 0; c < nch; c++) M = fmaxf(M, msm[c * 8 + h]);
        for (uint32_t c = 0; c < nch; c++) {
            float w = ex2(msm[c * 8 + h] - M);
            msm[c * 8 + h] = w;
            L = fmaf(lsm[c * 8 + h], w, L);
        }
        Lsm[h] = L;
    }
    __syncthreads();
    const uint32_t d4 = d >> 2;
    for (uint32_t i = threadIdx.x; i < it.nheads * d4; i += THREADS) {
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
                float w = msm[(c + u) * 8 + h];
                acc.x = fmaf(v[u].x, w, acc.x); acc.y = fmaf(v[u].y, w, acc.y);
                acc.z = fmaf(v[u].z, w, acc.z); acc.w = fmaf(v[u].w, w, acc.w);
            }
        }
        for (; c < nch; c++) {
            float4 v = __ldcg(reinterpret_cast<const float4*>(p + (size_t)c * stride));
            float w = msm[c * 8 + h];
            acc.x = fmaf(v.x, w, acc.x); acc.y = fmaf(v.y, w, acc.y);
            acc.z = fmaf(v.z, w, acc.z); acc.w = fmaf(v.w, w, acc.w);
        }
        const float L = Lsm[h];
        float4 o = make_float4(acc.x / L, acc.y / L, acc.z / L, acc.w / L);
        *reinterpret_cast<float4*>(a.out + ((size_t)it.seq * a.heads + it.head0 + h) * d + x) = o;
    }
    if (threadIdx.x == 0) a.counters[it.counter] = 0;  // ready for the next launch
}

// ---- 16-bit pools: tensor-core path ------------------------------------------------------
// PRECISE: queries and probabilities go through the tensor cores as value + remainder (two
// passes); needed for bf16's 8-bit mantissa to stay inside the tolerance, not for f16's 11.
template <int DT, int D, bool PRECISE>
__global__ void __launch_bounds__(THREADS, 3) attn_split_mma_kernel(SplitArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const SmemPlan sp = smem_plan(D * 2, D, false);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t* itw = a.items + (size_t)blockIdx.x * a.item_words;
    const Item it = load_item(itw);
    const uint32_t smem_base = smem_u32(smem);

    TileStream ts;
    ts.ring = smem_base + warp * sp.ring_bytes;
    ts.bars = smem_base + sp.bar_off + warp * 64;
    ts.stages = sp.stages; ts.stage_bytes = sp.stage_bytes; ts.tile_bytes = sp.tile_bytes;
    ts.base = a.pool + (uint64_t)it.kv_head * 2u * a.page_bytes;
    ts.block_bytes = a.block_bytes; ts.page_bytes = a.page_bytes; ts.tiles_per_block = a.tiles_per_block;
    ts.warp = warp; ts.lane = lane;

    if (lane == 0) {
        for (uint32_t s = 0; s < sp.stages; s++) mbar_init(ts.bars + s * 8, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncwarp();

    const uint32_t ntiles = (it.tokens + TILE - 1) / TILE;
    const uint32_t n_my = ntiles > warp ? (ntiles - warp + WARPS - 1) / WARPS : 0;
    ts.my_block = 0;
    if (lane < n_my) ts.my_block = itw[QVX_ITEM_HEADER_WORDS + (warp + WARPS * lane) / a.tiles_per_block];
    const uint32_t pre = n_my < sp.stages ? n_my : sp.stages;
    for (uint32_t i = 0; i < pre; i++) ts.issue(i);

    // Q^T fragments (the B operand): this lane holds head g, dims 16*ks + 2t + {0,1,8,9}, as a
    // 16-bit value plus a 16-bit remainder.
    uint32_t qf[D / 16][2], ql[D / 16][2];
    {
        const bool live = g < it.nheads;
        const float* qp = a.q + ((size_t)it.seq * a.heads + it.head0 + (live ? g : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            float2 x0 = make_float2(0.f, 0.f), x1 = x0;
            if (live) {
                x0 = *reinterpret_cast<const float2*>(qp + 16 * ks + 2 * t);
                x1 = *reinterpret_cast<const float2*>(qp + 16 * ks + 2 * t + 8);
            }
            split16<DT>(x0.x, x0.y, qf[ks][0], ql[ks][0]);
            split16<DT>(x1.x, x1.y, qf[ks][1], ql[ks][1]);
        }
    }

    float o[D / 16][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; mt++) { o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // heads 2t and 2t+1
    bool failed = false;

    // ldmatrix row addresses of this lane inside a tile (row stride D*2 bytes, swizzled chunks).
    const uint32_t mid = lane >> 3, r8 = lane & 7;
    const uint32_t k_row = r8 + 8 * (mid & 1), k_chunk = mid >> 1;  // keys: A = K, non-transposed
    const uint32_t v_row = r8 + 8 * (mid >> 1), v_chunk = mid & 1;  // values: A = V^T, transposed

    for (uint32_t i = 0; i < n_my; i++) {
        const uint32_t st = i % sp.stages;
        if (!__all_sync(0xffffffffu, mbar_wait(ts.bars + st * 8, (i / sp.stages) & 1))) { failed = true; break; }
        const uint32_t kt = ts.ring + st * sp.stage_bytes, vt = kt + sp.tile_bytes;
        const uint32_t tau = warp + WARPS * i;
        const uint32_t valid = min((uint32_t)TILE, it.tokens - tau * TILE);

        // S^T = K Q^T
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            uint32_t af[4];
            ldmatrix_x4(kt + k_row * (D * 2) + (((2 * ks + k_chunk) ^ (k_row & 7)) << 4), af);
            mma_16816<DT>(sc, af, qf[ks][0], qf[ks][1]);
            if constexpr (PRECISE) mma_16816<DT>(sc, af, ql[ks][0], ql[ks][1]);
        }
        if (valid < TILE) {
            // The tail of the last block: unwritten slots hold whatever the pool held before.
            if (g >= valid) { sc[0] = -INFINITY; sc[1] = -INFINITY; }
            if (g + 8 >= valid) { sc[2] = -INFINITY; sc[3] = -INFINITY; }
            // 0 * NaN is NaN: clear the value rows no probability reaches.
            uint4 z = make_uint4(0, 0, 0, 0);
            for (uint32_t c = valid * (D * 2 / 16) + lane; c < TILE * (D * 2 / 16); c += 32)
                *reinterpret_cast<uint4*>(smem + (vt - smem_base) + c * 16) = z;
            __syncwarp();
        }
        // Online softmax in base 2; this lane sees heads 2t, 2t+1 at positions g, g+8.
        float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
        }
        const float mn0 = fmaxf(m0, mx0 * a.scale_log2), mn1 = fmaxf(m1, mx1 * a.scale_log2);
        const float al0 = ex2(m0 - mn0), al1 = ex2(m1 - mn1);
        m0 = mn0; m1 = mn1;
        const float p0 = ex2(fmaf(sc[0], a.scale_log2, -mn0)), p1 = ex2(fmaf(sc[1], a.scale_log2, -mn1));
        const float p2 = ex2(fmaf(sc[2], a.scale_log2, -mn0)), p3 = ex2(fmaf(sc[3], a.scale_log2, -mn1));
        l0 = fmaf(l0, al0, p0 + p2);
        l1 = fmaf(l1, al1, p1 + p3);
        // P^T as the B operand: (position g; heads 2t,2t+1) -> (head g; positions 2t,2t+1),
        // again as value + remainder.
        uint32_t ph0, pl0, ph1, pl1;
        split16<DT>(p0, p1, ph0, pl0);
        split16<DT>(p2, p3, ph1, pl1);
        const uint32_t pb0 = movmatrix_trans(ph0), pb1 = movmatrix_trans(ph1);
        const uint32_t pc0 = movmatrix_trans(pl0), pc1 = movmatrix_trans(pl1);
        // O^T = O^T * alpha + V^T P^T
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            o[mt][0] *= al0; o[mt][1] *= al1; o[mt][2] *= al0; o[mt][3] *= al1;
            uint32_t vf[4];
            ldmatrix_x4_trans(vt + v_row * (D * 2) + (((2 * mt + v_chunk) ^ (v_row & 7)) << 4), vf);
            mma_16816<DT>(o[mt], vf, pb0, pb1);
            if constexpr (PRECISE) mma_16816<DT>(o[mt], vf, pc0, pc1);
        }
        __syncwarp();  // every lane is done reading this stage
        if (i + sp.stages < n_my) ts.issue(i + sp.stages);
    }

    // Row sums over the positions held by the other lanes of the same t.
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    if (failed) {
        if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
        // Give the copies still in flight a bounded chance to land before the CTA's shared
        // memory is handed to another one.
        for (uint32_t s = 0; s < sp.stages; s++) mbar_try_wait(ts.bars + s * 8, 0);
    }
    // All rings are quiet: reuse them for the warps' results.  An item any warp gave up on
    // writes nothing (the host sees the status word).
    if (__syncthreads_or(failed)) return;
    const uint32_t res_stride_f = sp.ring_bytes / 4;
    float* res = reinterpret_cast<float*>(smem) + warp * res_stride_f;
    if (g == 0) {
        res[2 * t] = m0; res[2 * t + 1] = m1;
        res[8 + 2 * t] = l0; res[8 + 2 * t + 1] = l1;
    }
#pragma unroll
    for (int mt = 0; mt < D / 16; mt++) {
        res[16 + (2 * t) * D + 16 * mt + g] = o[mt][0];
        res[16 + (2 * t + 1) * D + 16 * mt + g] = o[mt][1];
        res[16 + (2 * t) * D + 16 * mt + g + 8] = o[mt][2];
        res[16 + (2 * t + 1) * D + 16 * mt + g + 8] = o[mt][3];
    }
    __syncthreads();
    merge_and_store(a, it, reinterpret_cast<const float*>(smem), res_stride_f, D, reinterpret_cast<float*>(smem));
}

// ---- f32 pools: CUDA-core path -------------------------------------------------------------
// Scores: lane = (position = lane & 15, half = lane >> 4) computes heads half, half+2, ...;
// values: lane owns output dims lane, lane+32, ... of all NH heads.
template <int D, int NH>
__global__ void __launch_bounds__(THREADS, 2) attn_split_f32_kernel(SplitArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NJ = NH / 2;   // heads per lane in the score phase
    constexpr int DK = D / 32;   // output dims per lane
    const SmemPlan sp = smem_plan(D * 4, D, true);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t* itw = a.items + (size_t)blockIdx.x * a.item_words;
    const Item it = load_item(itw);
    const uint32_t smem_base = smem_u32(smem);

    TileStream ts;
    ts.ring = smem_base + warp * sp.ring_bytes;
    ts.bars = smem_base + sp.bar_off + warp * 64;
    ts.stages = sp.stages; ts.stage_bytes = sp.stage_bytes; ts.tile_bytes = sp.tile_bytes;
    ts.base = a.pool + (uint64_t)it.kv_head * 2u * a.page_bytes;
    ts.block_bytes = a.block_bytes; ts.page_bytes = a.page_bytes; ts.tiles_per_block = a.tiles_per_block;
    ts.warp = warp; ts.lane = lane;
    if (lane == 0) {
        for (uint32_t s = 0; s < sp.stages; s++) mbar_init(ts.bars + s * 8, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncwarp();
    const uint32_t ntiles = (it.tokens + TILE - 1) / TILE;
    const uint32_t n_my = ntiles > warp ? (ntiles - warp + WARPS - 1) / WARPS : 0;
    ts.my_block = 0;
    if (lane < n_my) ts.my_block = itw[QVX_ITEM_HEADER_WORDS + (warp + WARPS * lane) / a.tiles_per_block];
    const uint32_t pre = n_my < sp.stages ? n_my : sp.stages;
    for (uint32_t i = 0; i < pre; i++) ts.issue(i);

    // The group's queries, pre-multiplied by scale * log2(e); heads past the group are zero.
    float* qs = reinterpret_cast<float*>(smem + sp.q_off);
    for (uint32_t i = threadIdx.x; i < NH * D; i += THREADS) {
        uint32_t h = i / D, x = i % D;
        qs[i] = h < it.nheads ? a.q[((size_t)it.seq * a.heads + it.head0 + h) * D + x] * a.scale_log2 : 0.f;
    }
    __syncthreads();
    float* ps = reinterpret_cast<float*>(smem + sp.p_off) + warp * (TILE * 8);  // [position][8]

    const uint32_t tok = lane & 15, half = lane >> 4;
    float m[NH], o[NH][DK], lpart[NJ];
#pragma unroll
    for (int h = 0; h < NH; h++) {
        m[h] = -INFINITY;
#pragma unroll
        for (int k = 0; k < DK; k++) o[h][k] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < NJ; j++) lpart[j] = 0.f;
    bool failed = false;

    for (uint32_t i = 0; i < n_my; i++) {
        const uint32_t st = i % sp.stages;
        if (!__all_sync(0xffffffffu, mbar_wait(ts.bars + st * 8, (i / sp.stages) & 1))) { failed = true; break; }
        const uint8_t* kt = smem + warp * sp.ring_bytes + st * sp.stage_bytes;
        const uint8_t* vt = kt + sp.tile_bytes;
        const uint32_t tau = warp + WARPS * i;
        const uint32_t valid = min((uint32_t)TILE, it.tokens - tau * TILE);

        float s[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) s[j] = 0.f;
        const uint8_t* krow = kt + tok * (D * 4);
#pragma unroll 4
        for (int c = 0; c < D / 4; c++) {
            float4 kv = *reinterpret_cast<const float4*>(krow + ((c ^ (tok & 7)) << 4));
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                float4 qv = *reinterpret_cast<const float4*>(qs + (half + 2 * j) * D + 4 * c);
                s[j] = fmaf(qv.x, kv.x, s[j]); s[j] = fmaf(qv.y, kv.y, s[j]);
                s[j] = fmaf(qv.z, kv.z, s[j]); s[j] = fmaf(qv.w, kv.w, s[j]);
            }
        }
        if (tok >= valid) {
#pragma unroll
            for (int j = 0; j < NJ; j++) s[j] = -INFINITY;
        }
        // Tile maximum per head over the 16 positions, then across the two halves.
        float mx[NH];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            float v = s[j];
#pragma unroll
            for (int sh = 1; sh <= 8; sh <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, sh));
            float other = __shfl_xor_sync(0xffffffffu, v, 16);
            // Head half+2j is mine, head (1-half)+2j the other half's.
            mx[2 * j] = half == 0 ? v : other;
            mx[2 * j + 1] = half == 0 ? other : v;
        }
        float al[NH];
#pragma unroll
        for (int h = 0; h < NH; h++) {
            float mn = fmaxf(m[h], mx[h]);
            al[h] = ex2(m[h] - mn);
            m[h] = mn;
        }
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            float mine = half == 0 ? m[2 * j] : m[2 * j + 1];
            float al_mine = half == 0 ? al[2 * j] : al[2 * j + 1];
            float p = ex2(s[j] - mine);
            lpart[j] = fmaf(lpart[j], al_mine, p);
            ps[tok * 8 + half + 2 * j] = p;
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < NH; h++) {
#pragma unroll
            for (int k = 0; k < DK; k++) o[h][k] *= al[h];
        }
        for (uint32_t p = 0; p < valid; p++) {
            float pv[8];
            *reinterpret_cast<float4*>(pv) = *reinterpret_cast<const float4*>(ps + p * 8);
            if (NH > 4) *reinterpret_cast<float4*>(pv + 4) = *reinterpret_cast<const float4*>(ps + p * 8 + 4);
            const uint8_t* vrow = vt + p * (D * 4);
#pragma unroll
            for (int k = 0; k < DK; k++) {
                uint32_t x = lane + 32 * k;
                float v = *reinterpret_cast<const float*>(vrow + ((((x >> 2) ^ (p & 7)) << 4) | ((x & 3) << 2)));
#pragma unroll
                for (int h = 0; h < NH; h++) o[h][k] = fmaf(pv[h], v, o[h][k]);
            }
        }
        __syncwarp();
        if (i + sp.stages < n_my) ts.issue(i + sp.stages);
    }
    // Row sums: over the 16 positions, then hand each half's heads to the other.
    float l[NH];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        float v = lpart[j];
#pragma unroll
        for (int sh = 1; sh <= 8; sh <<= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
        float other = __shfl_xor_sync(0xffffffffu, v, 16);
        l[2 * j] = half == 0 ? v : other;
        l[2 * j + 1] = half == 0 ? other : v;
    }
    if (failed) {
        if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
        for (uint32_t s = 0; s < sp.stages; s++) mbar_try_wait(ts.bars + s * 8, 0);
    }
    if (__syncthreads_or(failed)) return;
    const uint32_t res_stride_f = sp.ring_bytes / 4;
    float* res = reinterpret_cast<float*>(smem) + warp * res_stride_f;
    if (lane == 0) {
#pragma unroll
        for (int h = 0; h < 8; h++) {
            res[h] = h < NH ? m[h < NH ? h : 0] : -INFINITY;
            res[8 + h] = h < NH ? l[h < NH ? h : 0] : 0.f;
        }
    }
#pragma unroll
    for (int h = 0; h < NH; h++) {
#pragma unroll
        for (int k = 0; k < DK; k++) res[16 + h * D + lane + 32 * k] = o[h][k];
    }
    __syncthreads();
    merge_and_store(a, it, reinterpret_cast<const float*>(smem), res_stride_f, D, reinterpret_cast<float*>(smem));
}

// ---- host side -------------------------------------------------------------------------------
bool attn_split_supported(const Layout& L, size_t heads) {
    if (L.layout != QVX_LAYOUT_NATIVE) return false;
    if (L.B % TILE != 0) return false;
    if (heads % L.kvh != 0) return false;
    if (L.dtype == QVX_F32) return L.d == 64 || L.d == 128;
    return L.d == 64 || L.d == 128 || L.d == 256;
}

size_t attn_partial_floats(const qvx_tables* t) { return t->n_parts * (size_t)(8 * t->L.d + 16); }

template <typename K>
static int32_t launch_one(qvx_device* dev, K kernel, const SplitArgs& a, unsigned grid, uint32_t smem,
                          cudaStream_t s) {
    static thread_local K configured = nullptr;  // one opt-in per kernel instantiation and thread
    if (configured != kernel) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return check_cuda(dev, e, "split attention shared memory");
        configured = kernel;
    }
    kernel<<<grid, THREADS, smem, s>>>(a);
    return check_cuda(dev, cudaGetLastError(), "split attention launch");
}

extern int* device_status_word(qvx_device* dev);

int32_t launch_attn_split(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          float* partials, uint32_t* counters, cudaStream_t s) {
    if (t->n_items == 0) return QVX_OK;
    const Layout& L = t->L;
    SplitArgs a;
    a.pool = (const uint8_t*)pool; a.q = q; a.out = out; a.partials = partials; a.counters = counters;
    a.items = t->d_items; a.status = device_status_word(dev);
    a.block_bytes = L.block_bytes; a.page_bytes = L.page_bytes; a.row_bytes = L.row_bytes;
    a.tiles_per_block = L.B / TILE; a.heads = (uint32_t)t->heads; a.d = L.d; a.item_words = t->item_words;
    a.scale_log2 = (1.0f / sqrtf((float)L.d)) * 1.4426950408889634f;
    const bool f32 = L.dtype == QVX_F32;
    const SmemPlan sp = smem_plan(L.row_bytes, L.d, f32);
    const unsigned grid = (unsigned)t->n_items;
    const size_t group = t->heads / L.kvh;
    int32_t rc = QVX_ERR_UNSUPPORTED;
    LaunchTimer timer(dev, QVX_K_ATTN, s);
    if (f32) {
        const int nh = group >= 8 ? 8 : (group > 2 ? 4 : 2);
#define QVX_F32_CASE(DD, NN) \
    if (L.d == DD && nh == NN) rc = launch_one(dev, attn_split_f32_kernel<DD, NN>, a, grid, sp.total, s);
        QVX_F32_CASE(64, 2) QVX_F32_CASE(64, 4) QVX_F32_CASE(64, 8)
        QVX_F32_CASE(128, 2) QVX_F32_CASE(128, 4) QVX_F32_CASE(128, 8)
#undef QVX_F32_CASE
    } else {
        static const bool one_pass = getenv("QVX_ATTN_ONE_PASS") != nullptr;  // experiments only
        const bool precise = L.dtype == QVX_BF16 && !one_pass;
#define QVX_MMA_CASE(TT, DD, PP) \
    if (L.dtype == TT && L.d == DD && precise == PP) \
        rc = launch_one(dev, attn_split_mma_kernel<TT, DD, PP>, a, grid, sp.total, s);
        QVX_MMA_CASE(QVX_BF16, 64, true) QVX_MMA_CASE(QVX_BF16, 128, true) QVX_MMA_CASE(QVX_BF16, 256, true)
        QVX_MMA_CASE(QVX_BF16, 128, false)
        QVX_MMA_CASE(QVX_F16, 64, false) QVX_MMA_CASE(QVX_F16, 128, false) QVX_MMA_CASE(QVX_F16, 256, false)
#undef QVX_MMA_CASE
    }
    if (rc == QVX_ERR_UNSUPPORTED) return fail(dev, rc, "split attention: no kernel for this geometry");
    return rc;
}

}  // namespace qvx
