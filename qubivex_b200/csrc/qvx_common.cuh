// Shared by every translation unit of libqvx_cuda: the pool's address function, element
// conversion, the device handle, and the launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <vector>

#include "../../include/qvx.h"

#if defined(__CUDACC__)
#define QVX_HD __host__ __device__ __forceinline__
#else
#define QVX_HD inline
#endif

namespace qvx {

// Values a kernel can leave in the device's status word (0 = fine).  The host reads the word at
// its next wait on the device; the word is sticky until then.
constexpr int STATUS_WAIT_TIMEOUT = 1;      // a bounded wait (mbarrier, published entries) ran out
constexpr int STATUS_POSITION_BOUND = 2;    // a position beyond the bound the caller gave (qvx_attn_decode_static)
constexpr int STATUS_BLOCK_OUT_OF_POOL = 3; // a block id >= pool_blocks: that row or move was skipped, nothing written

// ---- geometry ------------------------------------------------------------------------
QVX_HD uint32_t elem_size(uint32_t dtype) { return dtype == QVX_F32 ? 4u : 2u; }

// Everything a kernel needs to address the pool, precomputed once per launch.
struct Layout {
    uint32_t B, kvh, d, dtype, layout, e;
    uint32_t row_bytes;    // d * e
    uint32_t page_bytes;   // B * row_bytes: the keys (or the values) of one (block, kv head)
    uint64_t block_bytes;  // 2 * kvh * page_bytes
};

inline bool geometry_ok(const qvx_geometry* g) {
    if (!g || !g->block_tokens || !g->kv_heads || !g->head_dim) return false;
    if (g->dtype > QVX_F16 || g->layout > QVX_LAYOUT_NATIVE) return false;
    if (g->layout == QVX_LAYOUT_NATIVE && (g->head_dim * elem_size(g->dtype)) % 128 != 0) return false;
    // A block must stay addressable with 32-bit in-block offsets.
    uint64_t bb = 2ull * g->block_tokens * g->kv_heads * g->head_dim * elem_size(g->dtype);
    return bb < (1ull << 31);
}

inline Layout make_layout(const qvx_geometry* g) {
    Layout L;
    L.B = g->block_tokens; L.kvh = g->kv_heads; L.d = g->head_dim;
    L.dtype = g->dtype; L.layout = g->layout; L.e = elem_size(g->dtype);
    L.row_bytes = L.d * L.e;
    L.page_bytes = L.B * L.row_bytes;
    L.block_bytes = 2ull * L.kvh * L.page_bytes;
    return L;
}

// Byte offset inside one block of key (kv = 0) / value (kv = 1) element (g, i) of `slot`.
// REFERENCE: kv_key_word / kv_value_word (crates/qubivex-compute/src/discrete.rs:317-329)
// with KV_BLOCK generalised to B and the f32 word to one element.
// NATIVE: [kv_head][K|V][slot][d], 16-byte chunks of a row XORed with (slot & 7).
QVX_HD uint32_t in_block_offset(const Layout& L, uint32_t slot, uint32_t kv, uint32_t g, uint32_t i) {
    if (L.layout == QVX_LAYOUT_REFERENCE) {
        uint32_t kv_out = L.kvh * L.d;
        uint32_t w = kv ? L.B * kv_out + slot * kv_out + g * L.d + i : (g * L.d + i) * L.B + slot;
        return w * L.e;
    }
    uint32_t in_row = (i * L.e) ^ ((slot & 7u) << 4);
    return g * 2u * L.page_bytes + kv * L.page_bytes + slot * L.row_bytes + in_row;
}

// ---- element conversion ------------------------------------------------------------------
// Narrowing is round-to-nearest-even; a NaN keeps its sign and becomes quiet (the pool bytes
// are compared exactly with the CPU restatement, so the rule is spelled out rather than left
// to an intrinsic that canonicalises NaNs).  Widening bf16 is `bits << 16`
// (crates/qubivex-backend-cpu/src/formats.rs:76-80).
QVX_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
QVX_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
QVX_HD uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
QVX_HD float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
QVX_HD uint16_t f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x1ffu));
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);
    if (a >= 0x38800000u) {
        uint32_t m = a - 0x38000000u;
        return (uint16_t)(sign | ((m + 0xfffu + ((m >> 13) & 1u)) >> 13));
    }
    if (a < 0x33000000u) return (uint16_t)sign;
    uint32_t e = a >> 23, mant = (a & 0x7fffffu) | 0x800000u, shift = 126u - e;
    uint32_t q = mant >> shift, rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}
QVX_HD float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0x1fu) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e != 0) return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
    if (m == 0) return bits_f32(sign);
    float v = (float)m * 5.9604644775390625e-8f;
    return sign ? -v : v;
}
QVX_HD uint16_t narrow16(float f, uint32_t dtype) { return dtype == QVX_BF16 ? f32_to_bf16(f) : f32_to_f16(f); }
QVX_HD float widen16(uint16_t h, uint32_t dtype) { return dtype == QVX_BF16 ? bf16_to_f32(h) : f16_to_f32(h); }
#if defined(__CUDACC__)
// Two elements at once on the device (x0 in the low half): the hardware's round-to-nearest-even
// conversion gives the same bits as the integer code above for everything but NaNs, which it
// canonicalises; those take the integer code.
__device__ __forceinline__ uint32_t narrow16x2(float x0, float x1, uint32_t dtype) {
    uint32_t r;
    if (dtype == QVX_BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x1), "f"(x0));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(x1), "f"(x0));
    if (x0 != x0) r = (r & 0xffff0000u) | (uint32_t)narrow16(x0, dtype);
    if (x1 != x1) r = (r & 0x0000ffffu) | ((uint32_t)narrow16(x1, dtype) << 16);
    return r;
}
#endif

// ---- the device handle ---------------------------------------------------------------------
struct TimedLaunch {
    int kind;
    cudaEvent_t a, b;
};

}  // namespace qvx

struct qvx_buffer {
    qvx_device* dev;
    void* ptr;
    size_t len;
    bool arena;      // from qvx_alloc: writable
    int refs;
};

struct qvx_device {
    int ordinal = 0;
    qvx_config cfg{};
    cudaDeviceProp prop{};
    cudaStream_t stream = nullptr;  // the device's own stream: every _host call runs here
    std::mutex mu;                  // guards everything below
    std::string last_error;
    qvx_usage usage{};
    qvx_transfer_stats xfer{};
    qvx_kernel_times ktimes{};
    uint64_t timing_seen[QVX_K_COUNT] = {};
    std::vector<qvx::TimedLaunch> pending;  // events not read back yet
    std::vector<cudaEvent_t> event_pool;
    // Scratch the split kernel writes its partial results to, and the arrival counters of the
    // split sequences (zero between launches), both grown on demand.
    void* partials = nullptr;
    size_t partials_cap = 0;
    uint32_t* counters = nullptr;
    size_t counters_cap = 0;
    uint32_t* queue = nullptr;  // the streaming kernel's work queue: next item, CTAs done
    // The scratch comes twice: consecutive launches alternate halves, so that a launch allowed to
    // overlap the tail of the one before never shares partials, counters or queue with it.
    uint32_t scratch_half = 0;
    void* plan_cache = nullptr;  // the last host op's work list (PlanCache, qvx_api.cu)
    // Pinned staging ring for the _host calls and its device twin; the ops in flight hold slices.
    char* staging = nullptr;
    size_t staging_cap = 0, staging_used = 0;
    char* dstaging = nullptr;
    size_t dstaging_cap = 0;
    struct PendingOut { float* dst; const float* src; size_t bytes; };
    std::vector<PendingOut> pending_out;
};

namespace qvx {

int32_t fail(qvx_device* dev, int32_t code, const char* fmt, ...);
int32_t check_cuda(qvx_device* dev, cudaError_t e, const char* what);

// Brackets a kernel launch with events when the device was opened with timing on.
struct LaunchTimer {
    qvx_device* dev; int kind; cudaStream_t s; cudaEvent_t a = nullptr, b = nullptr;
    LaunchTimer(qvx_device* dev, int kind, cudaStream_t s);
    ~LaunchTimer();
};

// Kernel entry points of the other translation units.
int32_t launch_kv_rows(qvx_device* dev, const Layout& L, void* pool, const float* k_rows,
                       const float* v_rows, size_t row_stride_f32, const uint32_t* at_direct,
                       const uint32_t* pos, const uint32_t* blocks, const uint32_t* table_at, size_t n,
                       size_t pool_blocks, int kind, cudaStream_t s);
int32_t launch_attn_prelude(qvx_device* dev, const Layout& L, size_t heads, size_t s, float* q, float* k_new, float* v_new,
                            const qvx_prelude* p, cudaStream_t stream);
// The positions of one chunk -- the unit of the online softmax -- before long sequences double it: 576 rounded down to
// whole blocks (at least one block).  One rule for the streaming kernel and the fixed-scratch one: same chunks, same bits
// per chunk.
constexpr uint32_t CHUNK_BASE_TOKENS = 576;
inline uint32_t base_chunk_tokens(uint32_t base, uint32_t B) { return (base > B ? base : B) / B * B; }

int32_t launch_block_copy(qvx_device* dev, const Layout& L, void* pool, const uint32_t* src,
                          const uint32_t* dst, size_t n, size_t pool_blocks, cudaStream_t s);

}  // namespace qvx

// One work item of the split kernel: up to `chunk` blocks of one sequence's table for one
// (kv head, group of <= 8 query heads).  In device memory an item is ITEM_HEADER_WORDS
// 32-bit words followed by the ids of its blocks, so that one round trip brings a CTA
// everything it needs to start its copies.
// A work item: a run of consecutive chunks of one (sequence, group of query heads).  A chunk's
// result is the same whatever run it is part of; runs only say how the chunks are dealt out.
#define QVX_ITEM_HEADER_WORDS 12
struct qvx_item_header {
    uint32_t seq;
    uint32_t tokens;      // valid positions in this item (the last block may be partly filled)
    uint32_t head0;       // first query head of the group
    uint32_t nheads_kv;   // query heads in the group (<= 8) | kv head << 16
    uint32_t part;        // index of the partial result of the item's first chunk; 0xffffffff: write `out` directly
    uint32_t part0;       // the partial of the first chunk of this (sequence, group)
    uint32_t nch;         // chunks of this (sequence, group)
    uint32_t counter;     // which arrival counters the chunks of this (sequence, group) share
    uint32_t chunk_tokens;  // positions per chunk of this sequence (its last chunk may hold fewer)
    uint32_t run;           // chunks in this item
    uint32_t reserved[2];
};

struct qvx_tables {
    qvx_device* dev;
    qvx::Layout L;
    size_t pool_blocks, heads, s, n_blocks, n_items, n_parts, n_counters;
    uint32_t max_pos;
    uint32_t chunk_blocks;
    uint32_t item_words;  // header + block ids, padded to a multiple of 4 words
    // One device allocation: pos | table_at | blocks | items
    void* dmem = nullptr;
    size_t dmem_bytes = 0;
    bool owns_dmem = true;
    uint32_t *d_pos, *d_table_at, *d_blocks, *d_items;
};

namespace qvx {
int32_t launch_attn_split(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          float* partials, uint32_t* counters, uint32_t* queue, const float* k_new, const float* v_new,
                          bool overlap, cudaStream_t s);
bool attn_split_fuses_append(const Layout& L, size_t heads);
int32_t launch_attn_exact(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          cudaStream_t s);
size_t attn_partial_floats(const qvx_tables* t);  // floats of scratch the split kernel needs
bool attn_split_supported(const Layout& L, size_t heads);
uint32_t attn_parts_per_group(const Layout& L, uint32_t nch);
uint32_t attn_counters_per_group(const Layout& L, uint32_t nch);
}  // namespace qvx
