// KV sync and KV append: one position's key row and value row (f32, kv_out each) written
// into its block of the pool, narrowed to the pool's element type.
//
// Replaces the `put` closure of the reference's CPU device
// (crates/qubivex-backend-cpu/src/sim.rs:377-399), `kv_sync.comp`
// (crates/qubivex-backend-vulkan/shaders/kv_sync.comp:36-50) and the store of
// `attn_prelude.comp` (shaders/attn_prelude.comp:92-104, :169-173).
//
// Native layout: one thread per 16-byte chunk of the pool — a row of d elements is d*e/16
// consecutive chunks, so a warp writes whole rows with 16-byte vector stores.
// Algorithmic bytes per row pair: 2 * kv_out * (4 + e).
// Reference layout: keys are dimension-major inside a block, a stride-B scatter of single
// elements; one thread per element (compatibility path, not the fast one).
//
// The block ids come from device memory the host of the device-pointer entry points has not seen:
// a row whose block lies at or past `pool_blocks` is skipped (nothing of it is written) and the
// device's status word gets STATUS_BLOCK_OUT_OF_POOL, which the host reports at its next wait.
#include <algorithm>

#include "qvx_common.cuh"

namespace qvx {

struct RowArgs {
    Layout L;
    uint8_t* pool;
    const float* k_rows;
    const float* v_rows;
    size_t row_stride;          // floats between consecutive rows of k_rows / v_rows
    const uint32_t* at_direct;  // sync: pool position per row (0xffffffff: skip); else null
    const uint32_t* pos;        // append: position, table start and tables
    const uint32_t* blocks;
    const uint32_t* table_at;
    uint32_t n;
    uint32_t pool_blocks;       // blocks the pool holds: a row for a block at or past it is skipped
    int* status;                // the device's status word
};

__device__ __forceinline__ bool row_target(const RowArgs& a, uint32_t r, uint32_t& block, uint32_t& slot) {
    if (a.at_direct) {
        uint32_t at = a.at_direct[r];
        if (at == 0xffffffffu) return false;
        block = at / a.L.B; slot = at % a.L.B;
    } else {
        uint32_t p = a.pos[r];
        block = a.blocks[a.table_at[r] + p / a.L.B];
        slot = p % a.L.B;
    }
    if (block >= a.pool_blocks) {
        atomicExch(a.status, STATUS_BLOCK_OUT_OF_POOL);
        return false;
    }
    return true;
}

// grid: (ceil(NATIVE_GROUP * kvh * 2 * chunks_per_row / 256), ceil(n / NATIVE_GROUP)) x 256 threads:
// blockIdx.y picks a group of NATIVE_GROUP rows, so a thread's index inside the group fits 32 bits
// and is split with 32-bit divisions.
constexpr uint32_t NATIVE_GROUP = 1024;
constexpr uint32_t OUT_OF_POOL = 0xfffffffeu;  // in place of a pool position: the row's block id is not the pool's
constexpr uint32_t NATIVE_PER_THREAD = 2;  // chunks per thread: all their loads are issued before anything waits
__global__ void __launch_bounds__(256) kv_rows_native_kernel(RowArgs a) {
    const uint32_t cpr = a.L.row_bytes >> 4;  // chunks per row
    const uint32_t per_row = a.L.kvh * 2u * cpr;
    const uint32_t row0 = blockIdx.y * NATIVE_GROUP, rows = min(NATIVE_GROUP, a.n - row0);
    const uint32_t total = rows * per_row;
    const bool pow2 = (cpr & (cpr - 1u)) == 0u && (per_row & (per_row - 1u)) == 0u;
    const uint32_t cpr_shift = 31u - (uint32_t)__clz((int)cpr), row_shift = 31u - (uint32_t)__clz((int)per_row);
    const uint32_t epc = 16u / a.L.e;  // elements per chunk
    const uint32_t dt = a.L.dtype;
    const uint32_t first = blockIdx.x * (256u * NATIVE_PER_THREAD) + threadIdx.x;
    float4 lo[NATIVE_PER_THREAD], hi[NATIVE_PER_THREAD];
    uint32_t at[NATIVE_PER_THREAD], rr[NATIVE_PER_THREAD], ww[NATIVE_PER_THREAD];
    // The source rows do not depend on where they go: their loads and the targets' loads go out together.
#pragma unroll
    for (uint32_t u = 0; u < NATIVE_PER_THREAD; u++) {
        const uint32_t idx = first + u * 256u;
        at[u] = 0xffffffffu;
        if (idx >= total) continue;
        // (powers of two in every configuration of interest: shifts instead of divisions)
        const uint32_t r = row0 + (pow2 ? idx >> row_shift : idx / per_row), w = pow2 ? idx & (per_row - 1u) : idx % per_row;
        rr[u] = r; ww[u] = w;
        const uint32_t g = pow2 ? w >> (cpr_shift + 1u) : w / (2u * cpr), kv = (pow2 ? w >> cpr_shift : w / cpr) & 1u,
                       c = pow2 ? w & (cpr - 1u) : w % cpr;
        const float* src = (kv ? a.v_rows : a.k_rows) + (size_t)r * a.row_stride + g * a.L.d + c * epc;
        lo[u] = *reinterpret_cast<const float4*>(src);
        if (dt != QVX_F32) hi[u] = *reinterpret_cast<const float4*>(src + 4);
        if (a.at_direct) {
            at[u] = a.at_direct[r];
        } else {
            const uint32_t p = a.pos[r], blk = a.blocks[a.table_at[r] + p / a.L.B];
            // (checked before the multiplication: a wild id must not wrap into the pool)
            at[u] = blk < a.pool_blocks ? blk * a.L.B + p % a.L.B : OUT_OF_POOL;
        }
    }
#pragma unroll
    for (uint32_t u = 0; u < NATIVE_PER_THREAD; u++) {
        if (at[u] == 0xffffffffu) continue;
        const uint32_t block = at[u] / a.L.B, slot = at[u] % a.L.B, w = ww[u];
        if (at[u] == OUT_OF_POOL || block >= a.pool_blocks) {  // not this pool's block: the row is skipped, the host told
            atomicExch(a.status, STATUS_BLOCK_OUT_OF_POOL);
            continue;
        }
        const uint32_t g = pow2 ? w >> (cpr_shift + 1u) : w / (2u * cpr), kv = (pow2 ? w >> cpr_shift : w / cpr) & 1u,
                       c = pow2 ? w & (cpr - 1u) : w % cpr;
        uint4 out;
        if (dt == QVX_F32) {
            out = make_uint4(__float_as_uint(lo[u].x), __float_as_uint(lo[u].y), __float_as_uint(lo[u].z), __float_as_uint(lo[u].w));
        } else {
            out.x = narrow16x2(lo[u].x, lo[u].y, dt);
            out.y = narrow16x2(lo[u].z, lo[u].w, dt);
            out.z = narrow16x2(hi[u].x, hi[u].y, dt);
            out.w = narrow16x2(hi[u].z, hi[u].w, dt);
        }
        uint8_t* dst = a.pool + (uint64_t)block * a.L.block_bytes + (uint64_t)g * 2u * a.L.page_bytes +
                       (uint64_t)kv * a.L.page_bytes + (uint64_t)slot * a.L.row_bytes + ((c ^ (slot & 7u)) << 4);
        *reinterpret_cast<uint4*>(dst) = out;
        (void)rr;
    }
}

// Any layout, one thread per element.
__global__ void __launch_bounds__(256) kv_rows_element_kernel(RowArgs a) {
    const uint32_t kv_out = a.L.kvh * a.L.d;
    uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)a.n * 2u * kv_out) return;
    uint32_t r = (uint32_t)(idx / (2u * kv_out)), w = (uint32_t)(idx % (2u * kv_out));
    uint32_t kv = w / kv_out, gi = w % kv_out, g = gi / a.L.d, i = gi % a.L.d;
    uint32_t block, slot;
    if (!row_target(a, r, block, slot)) return;
    float x = (kv ? a.v_rows : a.k_rows)[(size_t)r * a.row_stride + gi];
    uint8_t* dst = a.pool + (uint64_t)block * a.L.block_bytes + in_block_offset(a.L, slot, kv, g, i);
    if (a.L.dtype == QVX_F32) *reinterpret_cast<float*>(dst) = x;
    else *reinterpret_cast<uint16_t*>(dst) = narrow16(x, a.L.dtype);
}

extern int* device_status_word(qvx_device* dev);

int32_t launch_kv_rows(qvx_device* dev, const Layout& L, void* pool, const float* k_rows,
                       const float* v_rows, size_t row_stride_f32, const uint32_t* at_direct,
                       const uint32_t* pos, const uint32_t* blocks, const uint32_t* table_at, size_t n,
                       size_t pool_blocks, int kind, cudaStream_t s) {
    if (n == 0) return QVX_OK;
    if (n > 0x7fffffffu) return fail(dev, QVX_ERR_CORE, "kv rows: %zu rows do not fit 31 bits", n);
    RowArgs a{L, (uint8_t*)pool, k_rows, v_rows, row_stride_f32, at_direct, pos, blocks, table_at, (uint32_t)n,
              (uint32_t)std::min<size_t>(pool_blocks, 0xffffffffu), device_status_word(dev)};
    LaunchTimer timer(dev, kind, s);
    bool aligned = (((uintptr_t)k_rows | (uintptr_t)v_rows | (uintptr_t)pool) & 15u) == 0 &&
                   (row_stride_f32 * 4) % 16 == 0;
    if (L.layout == QVX_LAYOUT_NATIVE && aligned) {
        const uint32_t per_row = L.kvh * 2u * (L.row_bytes >> 4);
        const uint32_t rows_x = (uint32_t)std::min<size_t>(n, NATIVE_GROUP);
        const uint32_t span = 256u * NATIVE_PER_THREAD;
        dim3 grid((rows_x * per_row + span - 1u) / span, (unsigned)((n + NATIVE_GROUP - 1) / NATIVE_GROUP));
        kv_rows_native_kernel<<<grid, 256, 0, s>>>(a);
    } else {
        uint64_t total = (uint64_t)n * 2u * L.kvh * L.d;
        kv_rows_element_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(a);
    }
    return check_cuda(dev, cudaGetLastError(), "kv rows launch");
}

}  // namespace qvx
