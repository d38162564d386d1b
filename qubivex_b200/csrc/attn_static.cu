// qvx_attn_decode_static: paged decode attention for callers that must not allocate.
//
// Who that is.  qubivex's runtime accounts for every byte of device memory in a ledger and
// sizes the KV pool by "what the budget leaves" (crates/qubivex-runtime/src/discrete.rs:429-455);
// a host that has handed the whole remaining device to the pool cannot let a backend call
// cudaMalloc later for its scratch: the call may fail, it is not in the ledger, and cudaMalloc
// and cudaFree synchronise the whole device in the middle of a decode step.  The other entry
// points of this library grow their scratch on demand (the split partials, the block-table
// image); this one owns all the scratch it will ever use, as a file-scope array in device
// memory, and takes everything else from the caller.
//
// The price: the array has a fixed size (STATIC_SCRATCH_BYTES, a little over 16 MiB, held by
// every GPU that loads the library until the process exits), so the op is refused beyond it;
// every call shares the array, so two calls that overlap on the GPU race on it (keep them on
// one stream, or order them with events); and the kernel is the plain one-launch-per-chunk
// variant, without the persistent queue of the main kernel.
//
// Same arithmetic as the main 16-bit kernel: S^T = K Q^T and O^T = V^T P^T on the tensor cores,
// queries and probabilities as value + remainder for bf16, online softmax in base 2, the context
// split into the main kernel's chunks (576 positions in whole blocks; no doubling for long sequences), the chunks of a
// sequence merged in chunk order by the CTA
// that delivers the last one.  There is no counterpart in the reference.
#include "attn_ptx.cuh"

namespace qvx {

constexpr uint32_t STATIC_MAX_COUNTERS = 16384;                       // (sequence, group) pairs per call
constexpr size_t STATIC_PARTIAL_BYTES = 16u << 20;                    // partial results per call
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_PARTIAL_BYTES + STATIC_MAX_COUNTERS * 4;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char qvx_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int SW = 4;                 // warps per CTA, each streaming its own tiles
constexpr int STHREADS = SW * 32;

struct StaticArgs {
    const uint8_t* pool;
    const float* q;
    float* out;
    float* partials;            // in the static array: slots x (8*d + 16): acc[8][d], m[8], l[8]
    uint32_t* counters;         // in the static array: one per (sequence, group); cleared before each launch
    const uint32_t* pos;
    const uint32_t* blocks;
    const uint32_t* table_at;
    int* status;
    uint64_t block_bytes;
    uint32_t page_bytes, tiles_per_block, heads, group, groups_per_kv, ngroups, max_chunks, chunk_blocks, chunk_tokens;
    float scale_log2;
};

template <int D>
struct StaticSmem {
    static constexpr uint32_t tile_bytes = TILE * D * 2;
    static constexpr uint32_t stage_bytes = 2 * tile_bytes;
    static constexpr uint32_t stages = 16384 / stage_bytes < 2 ? 2 : 16384 / stage_bytes;
    static constexpr uint32_t ring_bytes = stages * stage_bytes;   // per warp
    static constexpr uint32_t bar_off = SW * ring_bytes;
    static constexpr uint32_t total = bar_off + SW * stages * 8;
    static_assert(ring_bytes >= (16 + 8 * D) * 4, "a warp's result must fit its ring");
};

// grid: (max_chunks, groups, sequences); a CTA whose chunk lies past its sequence's end leaves at once.
template <int DT, int D, bool PRECISE>
__global__ void __launch_bounds__(STHREADS, 3) attn_static_kernel(StaticArgs a) {
    using SM = StaticSmem<D>;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t s_last;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t chunk = blockIdx.x, grp = blockIdx.y, seq = blockIdx.z;
    const uint32_t len = a.pos[seq] + 1u;
    const uint32_t nch = (len + a.chunk_tokens - 1) / a.chunk_tokens;
    if (chunk >= nch) return;
    if (nch > a.max_chunks) {  // the caller's bound on the positions was too small: refuse, write nothing
        if (threadIdx.x == 0) atomicExch(a.status, STATUS_POSITION_BOUND);
        return;
    }
    const uint32_t tokens = min(a.chunk_tokens, len - chunk * a.chunk_tokens);
    const uint32_t kv_head = grp / a.groups_per_kv, sub = grp % a.groups_per_kv;
    const uint32_t head0 = kv_head * a.group + sub * 8, nheads = min(8u, a.group - sub * 8);
    const uint32_t first = a.table_at[seq] + chunk * a.chunk_blocks;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + warp * SM::ring_bytes, bars = sbase + SM::bar_off + warp * SM::stages * 8;
    const uint8_t* base = a.pool + (uint64_t)kv_head * 2u * a.page_bytes;

    if (lane == 0) {
        for (uint32_t s = 0; s < SM::stages; s++) mbar_init(bars + s * 8, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncwarp();
    const uint32_t ntiles = (tokens + TILE - 1) / TILE;
    const uint32_t n_my = ntiles > warp ? (ntiles - warp + SW - 1) / SW : 0;   // at most 8: 512 / 16 / 4
    uint32_t my_block = 0;
    if (lane < n_my) my_block = a.blocks[first + (warp + SW * lane) / a.tiles_per_block];
    auto issue = [&](uint32_t i) {
        const uint32_t tau = warp + SW * i;
        const uint32_t blk = __shfl_sync(0xffffffffu, my_block, i & 31);
        if (lane == 0) {
            const uint32_t st = i % SM::stages, bar = bars + st * 8, dst = ring + st * SM::stage_bytes;
            const uint8_t* src = base + (uint64_t)blk * a.block_bytes + (uint64_t)(tau % a.tiles_per_block) * SM::tile_bytes;
            fence_proxy_async();
            mbar_expect_tx(bar, SM::stage_bytes);
            const uint64_t stream_policy = l2_policy_evict_first();  // read once: leave the L2 to the partial results
            bulk_g2s_hint(dst, src, SM::tile_bytes, bar, stream_policy);
            bulk_g2s_hint(dst + SM::tile_bytes, src + a.page_bytes, SM::tile_bytes, bar, stream_policy);
        }
    };
    const uint32_t pre = n_my < SM::stages ? n_my : SM::stages;
    for (uint32_t i = 0; i < pre; i++) issue(i);

    uint32_t qf[D / 16][2], ql[D / 16][2];
    {
        const bool live = g < nheads;
        const float* qp = a.q + ((size_t)seq * a.heads + head0 + (live ? g : 0)) * D;
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
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    bool failed = false;

    for (uint32_t i = 0; i < n_my; i++) {
        const uint32_t st = i % SM::stages;
        if (!__all_sync(0xffffffffu, mbar_wait(bars + st * 8, (i / SM::stages) & 1))) { failed = true; break; }
        const uint32_t kt = ring + st * SM::stage_bytes, vt = kt + SM::tile_bytes;
        const uint32_t tau = warp + SW * i;
        const uint32_t valid = min((uint32_t)TILE, tokens - tau * TILE);
        attend_tile<DT, D, (PRECISE ? 3 : 0)>(kt, vt, smem + (vt - sbase), valid, lane, qf, ql, a.scale_log2, o, m0, m1, l0, l1);
        __syncwarp();
        if (i + SM::stages < n_my) issue(i + SM::stages);
    }
#pragma unroll
    for (int sh = 4; sh <= 16; sh <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
        l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
    if (failed && lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
    if (__syncthreads_or(failed)) return;  // every ring is quiet here; a chunk that gave up writes nothing
    constexpr uint32_t RS = SM::ring_bytes / 4;  // floats between the warps' results
    float* res_all = reinterpret_cast<float*>(smem);
    float* res = res_all + warp * RS;
    if (g == 0) { res[2 * t] = m0; res[2 * t + 1] = m1; res[8 + 2 * t] = l0; res[8 + 2 * t + 1] = l1; }
#pragma unroll
    for (int mt = 0; mt < D / 16; mt++) {
        res[16 + (2 * t) * D + 16 * mt + g] = o[mt][0];
        res[16 + (2 * t + 1) * D + 16 * mt + g] = o[mt][1];
        res[16 + (2 * t) * D + 16 * mt + g + 8] = o[mt][2];
        res[16 + (2 * t + 1) * D + 16 * mt + g + 8] = o[mt][3];
    }
    __syncthreads();
    constexpr uint32_t PS = 8 * D + 16;
    const uint32_t pair = seq * a.ngroups + grp;
    float* part = a.partials + ((size_t)pair * a.max_chunks + chunk) * PS;
    for (uint32_t i = threadIdx.x; i < nheads * D; i += STHREADS) {
        const uint32_t h = i / D, x = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < SW; w++) M = fmaxf(M, res_all[w * RS + h]);
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < SW; w++) {
            const float* r = res_all + w * RS;
            const float wg = ex2(r[h] - M);
            acc = fmaf(r[16 + h * D + x], wg, acc);
            l = fmaf(r[8 + h], wg, l);
        }
        if (nch == 1) {
            a.out[((size_t)seq * a.heads + head0 + h) * D + x] = acc / l;
        } else {
            part[h * D + x] = acc;
            if (x == 0) { part[8 * D + h] = M; part[8 * D + 8 + h] = l; }
        }
    }
    if (nch == 1) return;
    __threadfence();  // the partial is visible device-wide before the arrival is counted
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(a.counters + pair, 1u) == nch - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The last chunk of this (sequence, group) to arrive: merge all of them, in chunk order.  The maxima, weights
    // and sums of nch <= max_chunks <= 1000 chunks ((16 nch + 8) floats) fit the rings, which are free by now.
    merge_chunks_in_order(a.partials + (size_t)pair * a.max_chunks * PS, nch, nheads, D,
                          a.out + ((size_t)seq * a.heads + head0) * D, reinterpret_cast<float*>(smem), STHREADS);
}

extern int* device_status_word(qvx_device* dev);

// The array's device address, looked up once per device (with that device current).
static std::mutex g_static_mu;
static void* g_static_ptr[64];

// `ordinal`: the device that is current.  The shared-memory opt-in belongs to the device's context, so it
// is made once per device and per kernel instantiation (under g_static_mu's caller-side lock: dev->mu).
template <int DT, int D, bool PRECISE>
static cudaError_t launch_static(int ordinal, const StaticArgs& a, dim3 grid, cudaStream_t s) {
    auto kernel = attn_static_kernel<DT, D, PRECISE>;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!configured[ordinal & 63]) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)StaticSmem<D>::total);
            if (e != cudaSuccess) return e;
            configured[ordinal & 63] = true;
        }
    }
    kernel<<<grid, STHREADS, StaticSmem<D>::total, s>>>(a);
    return cudaGetLastError();
}

}  // namespace qvx

using namespace qvx;

extern "C" int32_t qvx_attn_decode_static(qvx_device* dev, const qvx_geometry* geo, const void* pool, size_t heads,
                                          size_t s, const float* q, const uint32_t* pos, const uint32_t* blocks,
                                          const uint32_t* table_at, uint32_t max_pos, float* out, void* stream) {
    if (!dev) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    const Layout L = make_layout(geo);
    if (L.layout != QVX_LAYOUT_NATIVE || L.dtype == QVX_F32 || (L.d != 64 && L.d != 128) || L.B % TILE != 0 || L.B > 512)
        return fail(dev, QVX_ERR_UNSUPPORTED,
                    "qvx_attn_decode_static: native layout, bf16 or f16, head_dim 64 or 128, block_tokens a multiple of 16 up to 512");
    const uint32_t chunk_tokens = base_chunk_tokens(CHUNK_BASE_TOKENS, L.B);
    if (heads == 0 || heads % L.kvh != 0)
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: %zu tokens, %zu heads, %u KV heads of %u", s,
                    heads, L.kvh, L.d);
    if (s == 0) return QVX_OK;
    const uint32_t group = (uint32_t)(heads / L.kvh), gpk = (group + 7) / 8, ngroups = L.kvh * gpk;
    const uint64_t max_chunks = ((uint64_t)max_pos + chunk_tokens) / chunk_tokens;
    const uint64_t pairs = (uint64_t)s * ngroups;
    const uint64_t need = pairs * max_chunks * (8ull * L.d + 16) * 4;
    if (s > 65535 || ngroups > 65535 || max_chunks > 1000 || pairs > STATIC_MAX_COUNTERS || need > STATIC_PARTIAL_BYTES)
        return fail(dev, QVX_ERR_UNSUPPORTED,
                    "qvx_attn_decode_static: %zu sequences x %u head groups x %llu chunks need %llu bytes of scratch and %llu "
                    "counters; the fixed array holds %zu bytes and %u counters (use qvx_attn_decode)",
                    s, ngroups, (unsigned long long)max_chunks, (unsigned long long)need, (unsigned long long)pairs,
                    (size_t)STATIC_PARTIAL_BYTES, STATIC_MAX_COUNTERS);
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 15u) || ((uintptr_t)pool & 127u))
        return fail(dev, QVX_ERR_SHAPE,
                    "shape mismatch in routed moe attention: q and out must be 16-byte aligned, the pool 128-byte aligned");
    cudaError_t e = cudaSetDevice(dev->ordinal);
    if (e != cudaSuccess) return check_cuda(dev, e, "cudaSetDevice");
    void* base = nullptr;
    {
        // Set-up, once per device: the first call on a device does it, so make that call
        // outside any stream capture.
        std::lock_guard<std::mutex> lk2(g_static_mu);
        if (dev->ordinal < 0 || dev->ordinal >= 64) return fail(dev, QVX_ERR_DEVICE, "cuda device error: device ordinal %d", dev->ordinal);
        if (!g_static_ptr[dev->ordinal]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, qvx_static_scratch);
            if (e != cudaSuccess) return check_cuda(dev, e, "cudaGetSymbolAddress(static scratch)");
            g_static_ptr[dev->ordinal] = p;
        }
        base = g_static_ptr[dev->ordinal];
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* partials = reinterpret_cast<float*>(base);
    uint32_t* counters = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(base) + STATIC_PARTIAL_BYTES);
    // The array keeps whatever the last call (or a call that gave up) left: the arrival counters
    // must start from zero.  The partials are overwritten before they are read.
    e = cudaMemsetAsync(counters, 0, pairs * 4, st);
    if (e != cudaSuccess) return check_cuda(dev, e, "clearing the arrival counters");
    StaticArgs a;
    a.pool = (const uint8_t*)pool; a.q = q; a.out = out; a.partials = partials; a.counters = counters;
    a.pos = pos; a.blocks = blocks; a.table_at = table_at; a.status = device_status_word(dev);
    a.block_bytes = L.block_bytes; a.page_bytes = L.page_bytes; a.tiles_per_block = L.B / TILE;
    a.heads = (uint32_t)heads; a.group = group; a.groups_per_kv = gpk; a.ngroups = ngroups;
    a.max_chunks = (uint32_t)max_chunks; a.chunk_blocks = chunk_tokens / L.B; a.chunk_tokens = chunk_tokens;
    a.scale_log2 = (1.0f / sqrtf((float)L.d)) * 1.4426950408889634f;
    dim3 grid((unsigned)max_chunks, ngroups, (unsigned)s);
    e = cudaErrorInvalidValue;
    if (L.dtype == QVX_BF16 && L.d == 128) e = launch_static<QVX_BF16, 128, true>(dev->ordinal, a, grid, st);
    if (L.dtype == QVX_BF16 && L.d == 64) e = launch_static<QVX_BF16, 64, true>(dev->ordinal, a, grid, st);
    if (L.dtype == QVX_F16 && L.d == 128) e = launch_static<QVX_F16, 128, false>(dev->ordinal, a, grid, st);
    if (L.dtype == QVX_F16 && L.d == 64) e = launch_static<QVX_F16, 64, false>(dev->ordinal, a, grid, st);
    return check_cuda(dev, e, "qvx_attn_decode_static launch");
}
