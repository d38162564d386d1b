// Paged decode attention over f32 pools (CUDA cores): GQA-grouped, online softmax, split over
// the context; the CTA that delivers a sequence's last split merges all of them in split
// order.  The 16-bit pools' tensor-core kernel is attn_stream.cu; this file also holds the
// dispatch between the two.
//
// Computes what `attn_decode.comp` (crates/qubivex-backend-vulkan/shaders/attn_decode.comp:60-175)
// and the gather + `attend` of the CPU device (crates/qubivex-backend-cpu/src/sim.rs:400-429,
// crates/qubivex-compute/src/math.rs:142-155) compute, in another operation order: results
// agree within 1e-5, not bit for bit (the reference's own audit measured that an online
// softmax cannot be bit-identical, docs/engineering/VULKAN_EXECUTION_AUDIT.md:2031-2061).
//
// Work item (one CTA of 4 warps): one (sequence, kv head, group of <= 8 query heads) and up
// to `chunk` consecutive blocks of that sequence's table.  Chunk boundaries depend on the
// sequence's own length and a constant only, never on the batch or the SM count, so a
// sequence's result is the same whatever else shares the launch.
//
// Each warp streams its own tiles of 16 positions: lane 0 issues two bulk async copies
// (cp.async.bulk, global -> shared, completion on an mbarrier) per tile into the warp's own
// ring of stages; the native layout's pre-swizzled rows make the shared-memory image
// conflict-free to read.  Per position per kv head: 2*d*4 bytes, 4*d*G flops.
#include <algorithm>

#include "attn_ptx.cuh"

namespace qvx {

#ifndef QVX_RING_BYTES
#define QVX_RING_BYTES 16384   // shared memory each warp streams its tiles through
#endif
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;

// Shared memory per CTA: WARPS rings of `stages` stages (a stage = a key tile then a value
// tile, 16 rows each), the query and probability scratch, the mbarriers.  After
// the loop every ring is reused for its warp's result (m[8], l[8], acc[8][d]).
struct SmemPlan {
    uint32_t tile_bytes, stage_bytes, stages, ring_bytes, q_off, p_off, bar_off, total;
};
__host__ __device__ inline SmemPlan smem_plan(uint32_t row_bytes, uint32_t d) {
    SmemPlan p;
    p.tile_bytes = TILE * row_bytes;
    p.stage_bytes = 2 * p.tile_bytes;
    p.stages = QVX_RING_BYTES / p.stage_bytes;
    if (p.stages < 2) p.stages = 2;
    if (p.stages > 8) p.stages = 8;
    p.ring_bytes = p.stages * p.stage_bytes;
    uint32_t off = WARPS * p.ring_bytes;
    p.q_off = off;
    off += 8 * d * 4;
    p.p_off = off;
    off += WARPS * TILE * 8 * 8;   // per warp: [position][8 heads] of (p, p) pairs
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
            const uint64_t stream_policy = l2_policy_evict_first();  // read once: leave the L2 to the partial results
            bulk_g2s_hint(dst, src, tile_bytes, bar, stream_policy);
            bulk_g2s_hint(dst + tile_bytes, src + page_bytes, tile_bytes, bar, stream_policy);
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
    merge_chunks_in_order(a.partials + (size_t)it.part0 * (8 * d + 16), it.nch, it.nheads, d,
                          a.out + ((size_t)it.seq * a.heads + it.head0) * d, scratch, THREADS);
    if (threadIdx.x == 0) a.counters[it.counter] = 0;  // ready for the next launch
}

// ---- f32 pools: CUDA-core path -------------------------------------------------------------
// Scores: lane = (position = lane & 15, half = lane >> 4) computes heads half, half+2, ...;
// values: lane owns output dims 2 lane, 2 lane + 1 (+ 64, ...) of all NH heads.
// The kernel is bound by instruction issue, not by memory (every multiply-add takes operands from shared memory),
// so the multiply-adds go out two at a time (fma.rn.f32x2, a Blackwell instruction): a score is summed as an even
// and an odd half, an output pair (2 lane, 2 lane + 1) takes one instruction per head and position.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra = *reinterpret_cast<unsigned long long*>(&a), rb = *reinterpret_cast<unsigned long long*>(&b),
                       rc = *reinterpret_cast<unsigned long long*>(&c), rd;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    return *reinterpret_cast<float2*>(&rd);
}
template <int D, int NH>
__global__ void __launch_bounds__(THREADS, 2) attn_split_f32_kernel(SplitArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NJ = NH / 2;   // heads per lane in the score phase
    constexpr int DK = D / 64;   // output pairs per lane
    const SmemPlan sp = smem_plan(D * 4, D);
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
    float2* ps = reinterpret_cast<float2*>(smem + sp.p_off) + warp * (TILE * 8);  // [position][8] of (p, p)

    const uint32_t tok = lane & 15, half = lane >> 4;
    float m[NH], lpart[NJ];
    float2 o[NH][DK];
#pragma unroll
    for (int h = 0; h < NH; h++) {
        m[h] = -INFINITY;
#pragma unroll
        for (int k = 0; k < DK; k++) o[h][k] = make_float2(0.f, 0.f);
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

        float2 s2[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) s2[j] = make_float2(0.f, 0.f);
        const uint8_t* krow = kt + tok * (D * 4);
#pragma unroll 4
        for (int c = 0; c < D / 4; c++) {
            const float4 kv = *reinterpret_cast<const float4*>(krow + ((c ^ (tok & 7)) << 4));
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const float4 qv = *reinterpret_cast<const float4*>(qs + (half + 2 * j) * D + 4 * c);
                s2[j] = fma2(make_float2(qv.x, qv.y), make_float2(kv.x, kv.y), s2[j]);
                s2[j] = fma2(make_float2(qv.z, qv.w), make_float2(kv.z, kv.w), s2[j]);
            }
        }
        float s[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) s[j] = s2[j].x + s2[j].y;
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
            ps[tok * 8 + half + 2 * j] = make_float2(p, p);
        }
        __syncwarp();
        bool moved = false;
#pragma unroll
        for (int h = 0; h < NH; h++) moved = moved || al[h] != 1.0f;
        if (moved) {   // (the maxima settle after a chunk's first tiles: x * 1.0f is x, so skipping changes no bit)
#pragma unroll
            for (int h = 0; h < NH; h++) {
#pragma unroll
                for (int k = 0; k < DK; k++) { o[h][k].x *= al[h]; o[h][k].y *= al[h]; }
            }
        }
        // This lane's dims 2 lane, 2 lane + 1 (+ 64 k) of a value row: one 8-byte load in the row's swizzled chunk.
        auto accumulate = [&](uint32_t p) {
            float2 pv[NH];
#pragma unroll
            for (int h = 0; h < NH; h += 2) {
                const float4 two = *reinterpret_cast<const float4*>(ps + p * 8 + h);
                pv[h] = make_float2(two.x, two.y);
                pv[h + 1] = make_float2(two.z, two.w);
            }
            const uint8_t* vrow = vt + p * (D * 4);
#pragma unroll
            for (int k = 0; k < DK; k++) {
                const uint32_t chunk = (lane >> 1) + 16u * k;
                const float2 v = *reinterpret_cast<const float2*>(vrow + (((chunk ^ (p & 7)) << 4) | ((lane & 1u) << 3)));
#pragma unroll
                for (int h = 0; h < NH; h++) o[h][k] = fma2(pv[h], v, o[h][k]);
            }
        };
        if (valid == TILE) {
#pragma unroll
            for (uint32_t p = 0; p < TILE; p++) accumulate(p);
        } else {
            for (uint32_t p = 0; p < valid; p++) accumulate(p);   // (rows past `valid` may hold anything, NaNs included)
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
        for (int k = 0; k < DK; k++) *reinterpret_cast<float2*>(res + 16 + h * D + 2 * lane + 64 * k) = o[h][k];
    }
    __syncthreads();
    merge_and_store(a, it, reinterpret_cast<const float*>(smem), res_stride_f, D, reinterpret_cast<float*>(smem));
}

// ---- host side -------------------------------------------------------------------------------
bool attn_stream_supported(const Layout& L, size_t heads);
int32_t launch_attn_stream(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                           float* partials, uint32_t* counters, uint32_t* queue, const float* k_new, const float* v_new,
                           bool overlap, cudaStream_t s);

bool attn_split_supported(const Layout& L, size_t heads) {
    if (L.layout != QVX_LAYOUT_NATIVE) return false;
    if (L.B % TILE != 0) return false;
    if (heads == 0 || heads % L.kvh != 0) return false;
    if (L.dtype == QVX_F32) return L.d == 64 || L.d == 128;
    return attn_stream_supported(L, heads);
}

size_t attn_stream_partial_floats(uint32_t d);
uint32_t attn_stream_parts(uint32_t nch);
uint32_t attn_stream_counters(uint32_t nch);

// Floats of scratch for the partial results (the 16-bit kernel keeps m and l once per warp).
size_t attn_partial_floats(const qvx_tables* t) {
    size_t one = t->L.dtype == QVX_F32 ? 8 * (size_t)t->L.d + 16 : attn_stream_partial_floats(t->L.d);
    return t->n_parts * one;
}
// Partial slots and arrival counters of one split (sequence, group) of `nch` chunks.
uint32_t attn_parts_per_group(const Layout& L, uint32_t nch) { return L.dtype == QVX_F32 ? nch : attn_stream_parts(nch); }
uint32_t attn_counters_per_group(const Layout& L, uint32_t nch) { return L.dtype == QVX_F32 ? 1u : attn_stream_counters(nch); }

template <typename K>
static int32_t launch_one(qvx_device* dev, K kernel, const SplitArgs& a, unsigned grid, uint32_t smem,
                          cudaStream_t s) {
    // The opt-in belongs to the device's context: once per device for each kernel instantiation
    // (this function is instantiated per kernel type; the caller holds dev->mu, the table has its own lock
    // because two devices' callers may come here together).
    static std::mutex mu;
    static K configured[64] = {};
    {
        std::lock_guard<std::mutex> lk(mu);
        K& done = configured[dev->ordinal & 63];
        if (done != kernel) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return check_cuda(dev, e, "split attention shared memory");
            done = kernel;
        }
    }
    kernel<<<grid, THREADS, smem, s>>>(a);
    return check_cuda(dev, cudaGetLastError(), "split attention launch");
}

extern int* device_status_word(qvx_device* dev);

bool attn_split_fuses_append(const Layout& L, size_t heads) { return attn_stream_supported(L, heads); }

int32_t launch_attn_split(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          float* partials, uint32_t* counters, uint32_t* queue, const float* k_new, const float* v_new,
                          bool overlap, cudaStream_t s) {
    if (t->n_items == 0) return QVX_OK;
    const Layout& L = t->L;
    if (L.dtype != QVX_F32) return launch_attn_stream(dev, t, pool, q, out, partials, counters, queue, k_new, v_new, overlap, s);
    SplitArgs a;
    a.pool = (const uint8_t*)pool; a.q = q; a.out = out; a.partials = partials; a.counters = counters;
    a.items = t->d_items; a.status = device_status_word(dev);
    a.block_bytes = L.block_bytes; a.page_bytes = L.page_bytes; a.row_bytes = L.row_bytes;
    a.tiles_per_block = L.B / TILE; a.heads = (uint32_t)t->heads; a.d = L.d; a.item_words = t->item_words;
    a.scale_log2 = (1.0f / sqrtf((float)L.d)) * 1.4426950408889634f;
    const SmemPlan sp = smem_plan(L.row_bytes, L.d);
    const unsigned grid = (unsigned)t->n_items;
    const size_t group = t->heads / L.kvh;
    int32_t rc = QVX_ERR_UNSUPPORTED;
    LaunchTimer timer(dev, QVX_K_ATTN, s);
    const int nh = group >= 8 ? 8 : (group > 2 ? 4 : 2);
#define QVX_F32_CASE(DD, NN) \
    if (L.d == DD && nh == NN) rc = launch_one(dev, attn_split_f32_kernel<DD, NN>, a, grid, sp.total, s);
    QVX_F32_CASE(64, 2) QVX_F32_CASE(64, 4) QVX_F32_CASE(64, 8)
    QVX_F32_CASE(128, 2) QVX_F32_CASE(128, 4) QVX_F32_CASE(128, 8)
#undef QVX_F32_CASE
    if (rc == QVX_ERR_UNSUPPORTED) return fail(dev, rc, "split attention: no kernel for this geometry");
    return rc;
}

}  // namespace qvx
