// Whole-block copies inside the pool: src[i] -> dst[i].
//
// The reference has no counterpart: a prefix hit copies a whole cache on the host
// (KvCache::restore_from, crates/qubivex-arch/src/lib.rs:409-432) and its pool never moves
// a block (crates/qubivex-runtime/src/discrete.rs:227-243).  Here a shared block is copied
// before the first divergent append (copy-on-write), and a compaction pass gathers live
// blocks to the front of the pool; both are this kernel with a different list.
//
// HBM bound: 2 * block_bytes per move (one read, one write).  Each CTA moves one 16 KiB
// segment of one block: 256 threads x 4 independent 16-byte loads in flight, then 4 stores.
//
// A move that names a block at or past `pool_blocks` is skipped whole (nothing read, nothing
// written) and leaves STATUS_BLOCK_OUT_OF_POOL in the device's status word.
#include <algorithm>

#include "qvx_common.cuh"

namespace qvx {

constexpr uint32_t SEG_BYTES = 16384;

__global__ void __launch_bounds__(256) block_copy_kernel(uint8_t* pool, uint64_t block_bytes,
                                                         uint32_t segs_per_block,
                                                         const uint32_t* __restrict__ src,
                                                         const uint32_t* __restrict__ dst,
                                                         uint32_t pool_blocks, int* status) {
    uint32_t move = blockIdx.x / segs_per_block, seg = blockIdx.x % segs_per_block;
    uint32_t sb = src[move], db = dst[move];
    if (sb == db) return;
    if (sb >= pool_blocks || db >= pool_blocks) {
        if (threadIdx.x == 0 && seg == 0) atomicExch(status, STATUS_BLOCK_OUT_OF_POOL);
        return;
    }
    uint64_t off = (uint64_t)seg * SEG_BYTES;
    uint64_t len = block_bytes - off < SEG_BYTES ? block_bytes - off : SEG_BYTES;
    const uint4* s = reinterpret_cast<const uint4*>(pool + (uint64_t)sb * block_bytes + off);
    uint4* d = reinterpret_cast<uint4*>(pool + (uint64_t)db * block_bytes + off);
    uint32_t n16 = (uint32_t)(len >> 4);
    uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t i = threadIdx.x + k * 256u;
        if (i < n16) v[k] = __ldcs(s + i);  // streamed: a moved block is not read again soon
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        uint32_t i = threadIdx.x + k * 256u;
        if (i < n16) __stcs(d + i, v[k]);
    }
}

// Blocks whose size is not a multiple of 16 bytes (tiny reference-layout geometries).
__global__ void __launch_bounds__(256) block_copy_bytes_kernel(uint8_t* pool, uint64_t block_bytes,
                                                               const uint32_t* __restrict__ src,
                                                               const uint32_t* __restrict__ dst,
                                                               uint32_t pool_blocks, int* status) {
    uint32_t sb = src[blockIdx.x], db = dst[blockIdx.x];
    if (sb == db) return;
    if (sb >= pool_blocks || db >= pool_blocks) {
        if (threadIdx.x == 0) atomicExch(status, STATUS_BLOCK_OUT_OF_POOL);
        return;
    }
    for (uint64_t i = threadIdx.x; i < block_bytes; i += 256)
        pool[(uint64_t)db * block_bytes + i] = pool[(uint64_t)sb * block_bytes + i];
}

extern int* device_status_word(qvx_device* dev);

int32_t launch_block_copy(qvx_device* dev, const Layout& L, void* pool, const uint32_t* src,
                          const uint32_t* dst, size_t n, size_t pool_blocks, cudaStream_t s) {
    if (n == 0) return QVX_OK;
    const uint32_t held = (uint32_t)std::min<size_t>(pool_blocks, 0xffffffffu);
    int* status = device_status_word(dev);
    LaunchTimer timer(dev, QVX_K_COPY, s);
    if (L.block_bytes % 16 == 0 && ((uintptr_t)pool & 15u) == 0) {
        uint32_t segs = (uint32_t)((L.block_bytes + SEG_BYTES - 1) / SEG_BYTES);
        uint64_t grid = (uint64_t)n * segs;
        if (grid > 0x7fffffffull) return fail(dev, QVX_ERR_CORE, "block copy: %zu moves are too many for one launch", n);
        block_copy_kernel<<<(unsigned)grid, 256, 0, s>>>((uint8_t*)pool, L.block_bytes, segs, src, dst, held, status);
    } else {
        block_copy_bytes_kernel<<<(unsigned)n, 256, 0, s>>>((uint8_t*)pool, L.block_bytes, src, dst, held, status);
    }
    return check_cuda(dev, cudaGetLastError(), "block copy launch");
}

}  // namespace qvx
