// The C ABI of libqvx_cuda: the device handle (the DiscreteDevice subset of
// crates/qubivex-compute/src/discrete.rs:433-570 that the decode-attention stage uses),
// buffers, block tables, and the op with host memory in and out.  Validation follows the
// reference's CPU device (crates/qubivex-backend-cpu/src/sim.rs:313-324, :359-376).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <deque>
#include <unordered_set>

#include "qvx_common.cuh"

namespace qvx {

static thread_local std::string g_last_error;  // errors with no device to hang them on

int32_t fail(qvx_device* dev, int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (dev) dev->last_error = buf;
    g_last_error = buf;
    return code;
}

int32_t check_cuda(qvx_device* dev, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return QVX_OK;
    return fail(dev, QVX_ERR_DEVICE, "cuda device error: %s: %s", what, cudaGetErrorString(e));
}

static uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

// ---- launch timing ---------------------------------------------------------------------------
LaunchTimer::LaunchTimer(qvx_device* dev, int kind, cudaStream_t s) : dev(dev), kind(kind), s(s) {
    if (!dev || !dev->cfg.timing) return;
    if (dev->timing_seen[kind]++ % dev->cfg.timing != 0) return;  // timing = n: every n-th launch of a kind
    auto get = [&]() {
        cudaEvent_t e = nullptr;
        if (!dev->event_pool.empty()) { e = dev->event_pool.back(); dev->event_pool.pop_back(); }
        else cudaEventCreate(&e);
        return e;
    };
    a = get(); b = get();
    cudaEventRecord(a, s);
}
LaunchTimer::~LaunchTimer() {
    if (!a) return;
    cudaEventRecord(b, s);
    dev->pending.push_back(TimedLaunch{kind, a, b});
}

static void drain_timers(qvx_device* dev) {
    for (auto& p : dev->pending) {
        cudaEventSynchronize(p.b);
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) {
            dev->ktimes.launches[p.kind]++;
            uint64_t ns = (uint64_t)((double)ms * 1e6);
            dev->ktimes.gpu_ns[p.kind] += ns;
            dev->xfer.timed++;
            dev->xfer.gpu_ns += ns;
            dev->xfer.gpu_busy_ns += ns;  // one stream: the launches do not overlap
        }
        dev->event_pool.push_back(p.a);
        dev->event_pool.push_back(p.b);
    }
    dev->pending.clear();
}

// The status word lives in mapped pinned memory: kernels write it, the host reads it with no copy.
// A host op in flight: its slice of the staging ring, its tables, and the three events that order
// its copies in, its kernels and its copy out.  `out_done` says the slice may be reused.
struct HostOp {
    size_t begin = 0, end = 0;
    qvx_tables* tables = nullptr;
    cudaEvent_t in_done = nullptr, kernels_done = nullptr, out_done = nullptr;
};

struct DeviceExtras {
    int* status_host = nullptr;
    int* status_dev = nullptr;
    cudaStream_t h2d = nullptr, d2h = nullptr;
    cudaStream_t kernels2 = nullptr;       // the second kernel stream of independent host ops (see paged_attention_submit)
    cudaEvent_t last_kernels[2] = {nullptr, nullptr};  // kernels_done of the last op on each kernel stream
    std::vector<cudaEvent_t> sync_events;  // spare events, handed to ops and taken back
    std::deque<HostOp> ops;                // oldest first
    size_t ring_head = 0;                  // where the next op's slice starts
    bool ring_was_short = false;           // an op had to wait for a slice: grow at the next drain
};
static std::mutex g_extras_mu;
static std::vector<std::pair<qvx_device*, DeviceExtras*>> g_extras;
static DeviceExtras* extras(qvx_device* dev) {
    std::lock_guard<std::mutex> lk(g_extras_mu);
    for (auto& p : g_extras)
        if (p.first == dev) return p.second;
    return nullptr;
}
int* device_status_word(qvx_device* dev) { return extras(dev)->status_dev; }

static int32_t check_status(qvx_device* dev) {
    DeviceExtras* x = extras(dev);
    int st = *(volatile int*)x->status_host;
    if (st == 0) return QVX_OK;
    *(volatile int*)x->status_host = 0;
    if (dev->counters) {  // an item that gave up never arrived: start the counters from zero again
        cudaDeviceSynchronize();
        cudaMemset(dev->counters, 0, 2 * dev->counters_cap * 4);
        if (dev->queue) cudaMemset(dev->queue, 0, 16);
    }
    const char* what = st == STATUS_POSITION_BOUND      ? "a position beyond the bound the caller gave"
                       : st == STATUS_BLOCK_OUT_OF_POOL ? "a block id at or past pool_blocks (that row or move was skipped)"
                                                        : "a kernel gave up a bounded wait";
    return fail(dev, QVX_ERR_DEVICE, "cuda device error: %s (status %d); the op's outputs are not valid", what, st);
}

// ---- capacity accounting, as SimDevice::reserve (sim.rs:176-203) -----------------------------
static int32_t reserve(qvx_device* dev, uint64_t bytes) {
    uint64_t next = dev->usage.used + bytes;
    if (next < dev->usage.used || next > dev->usage.capacity) {
        dev->usage.refused++;
        return fail(dev, QVX_ERR_OUT_OF_MEMORY, "cuda device is out of memory: %llu bytes requested, %llu of %llu in use",
                    (unsigned long long)bytes, (unsigned long long)dev->usage.used,
                    (unsigned long long)dev->usage.capacity);
    }
    dev->usage.used = next;
    dev->usage.peak = std::max(dev->usage.peak, next);
    return QVX_OK;
}

static int32_t new_buffer(qvx_device* dev, size_t len, bool arena, qvx_buffer** out) {
    int32_t rc = reserve(dev, len);
    if (rc) return rc;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, len ? len : 1);
    if (e != cudaSuccess) {
        dev->usage.used -= len;
        cudaGetLastError();
        return fail(dev, QVX_ERR_DEVICE, "cuda device error: cannot allocate %zu bytes: %s", len, cudaGetErrorString(e));
    }
    *out = new qvx_buffer{dev, p, len, arena, 1};
    return QVX_OK;
}

static int32_t buffer_of(qvx_device* dev, qvx_buffer* b) {
    if (!b || b->dev != dev) return fail(dev, QVX_ERR_DEVICE, "cuda device error: the buffer belongs to another device");
    return QVX_OK;
}

// ---- staging for the host ops ---------------------------------------------------------------
// One pinned ring on the host and its twin on the device.  Each op takes a contiguous slice and
// gives it back when its copy out has finished, so submitting runs ahead of the device by as many
// ops as the ring holds and never has to drain it; an op that finds no room waits for the oldest
// op only.  The ring starts small and grows fourfold (to RING_AUTO_MAX, or to one op's own need) at a
// drain after an op had to wait.
static const size_t RING_MIN = 32u << 20, RING_AUTO_MAX = 128u << 20;

static cudaEvent_t take_event(DeviceExtras* x) {
    if (x->sync_events.empty()) {
        cudaEvent_t e = nullptr;
        cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        return e;
    }
    cudaEvent_t e = x->sync_events.back();
    x->sync_events.pop_back();
    return e;
}

static void retire(qvx_device* dev, DeviceExtras* x, HostOp& op) {
    (void)dev;
    delete op.tables;
    for (cudaEvent_t e : {op.in_done, op.kernels_done, op.out_done})
        if (e) x->sync_events.push_back(e);
}

static int32_t resize_staging(qvx_device* dev, size_t cap) {
    // Only called with nothing in flight.
    if (dev->staging) cudaFreeHost(dev->staging);
    if (dev->dstaging) cudaFree(dev->dstaging);
    dev->staging = nullptr; dev->dstaging = nullptr; dev->staging_cap = dev->dstaging_cap = 0;
    cudaError_t e = cudaHostAlloc((void**)&dev->staging, cap, cudaHostAllocDefault);
    if (e != cudaSuccess) return check_cuda(dev, e, "pinned staging");
    e = cudaMalloc((void**)&dev->dstaging, cap);
    if (e != cudaSuccess) return check_cuda(dev, e, "device staging");
    dev->staging_cap = dev->dstaging_cap = cap;
    return QVX_OK;
}

// `own_stream_only`: everything in flight was queued on the device's own stream (a serial op).
static int32_t wait_locked(qvx_device* dev, bool own_stream_only = false) {
    uint64_t t0 = now_ns();
    DeviceExtras* x = extras(dev);
    cudaError_t e = own_stream_only ? cudaSuccess : cudaStreamSynchronize(x->h2d);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
    if (e == cudaSuccess && !own_stream_only) e = cudaStreamSynchronize(x->kernels2);
    if (e == cudaSuccess && !own_stream_only) e = cudaStreamSynchronize(x->d2h);
    x->last_kernels[0] = x->last_kernels[1] = nullptr;
    dev->xfer.wait_ns += now_ns() - t0;
    dev->xfer.fence_waits++;
    for (HostOp& op : x->ops) retire(dev, x, op);
    x->ops.clear();
    x->ring_head = 0;
    dev->staging_used = 0;
    if (e != cudaSuccess) return check_cuda(dev, e, "wait");
    if (x->ring_was_short && dev->staging_cap && dev->staging_cap < RING_AUTO_MAX) {
        x->ring_was_short = false;
        int32_t rc = resize_staging(dev, std::min(dev->staging_cap * 4, RING_AUTO_MAX));
        if (rc) return rc;
    }
    return check_status(dev);
}

// A slice of `need` bytes (a multiple of 256) for a new op; *begin is its offset in both rings.
static int32_t take_slice(qvx_device* dev, DeviceExtras* x, size_t need, size_t* begin) {
    if (need > dev->staging_cap) {
        int32_t rc = wait_locked(dev);
        if (rc) return rc;
        if (need > dev->staging_cap) {  // the drain itself may have grown the ring
            rc = resize_staging(dev, std::max(need, std::max(dev->staging_cap * 2, RING_MIN)));
            if (rc) return rc;
        }
    }
    const size_t cap = dev->staging_cap;
    for (;;) {
        if (x->ops.empty()) { x->ring_head = 0; *begin = 0; break; }
        const size_t head = x->ring_head, tail = x->ops.front().begin;
        // Never fill the ring to the last byte: head == tail then always means "empty".
        if (head >= tail) {
            if (cap - head >= need) { *begin = head; break; }
            if (tail > need) { *begin = 0; break; }
        } else if (tail - head > need) { *begin = head; break; }
        // No room: the oldest op's slice comes back when its copy out is done.
        uint64_t t0 = now_ns();
        cudaError_t e = cudaEventSynchronize(x->ops.front().out_done);
        dev->xfer.wait_ns += now_ns() - t0;
        x->ring_was_short = true;
        if (e != cudaSuccess) return check_cuda(dev, e, "wait for a staging slice");
        retire(dev, x, x->ops.front());
        x->ops.pop_front();
    }
    x->ring_head = *begin + need;
    dev->staging_used = x->ring_head;
    return QVX_OK;
}

// ---- tables ----------------------------------------------------------------------------------
// The chunk a sequence of `len` positions is split into: a function of its own length and of
// constants only (never of the batch or the device), so its result is the same whatever shares
// the op.  576 positions (36 tiles: nine per consumer warp), doubled once (1152) when the sequence would
// make more than 32 chunks: long contexts get fewer, larger items and a shallower merge tree; a chunk never
// exceeds 2048 positions (its block ids ride in the work item's record).  576 rather than 512: a tenth fewer
// hand-overs and merge entries (over five batches of the MoE-decoder shape 0.5 us per launch on average, never
// more than 0.1 us worse; the head-sharded shape 3 %, the churn shape 0.3 %; 16 x 32768 loses 1.2 %); 640 and
// more leave the CTAs too few items to even out.
// These constants fix the bits of every result (a chunk is the unit of the online softmax), so the
// shipped library reads them from nowhere; an experiment build (-DQVX_EXPERIMENTS) takes them from the
// environment: QVX_CHUNK_TOKENS (a fixed size), QVX_CHUNK_BASE, QVX_CHUNK_MOST.
#ifdef QVX_EXPERIMENTS
static uint32_t env_u32(const char* name, uint32_t otherwise) {
    const char* v = getenv(name);
    const long n = v ? atol(v) : 0;
    return n > 0 ? (uint32_t)n : otherwise;
}
#endif
static uint32_t chunk_tokens_for(const Layout& L, uint32_t len) {
#ifdef QVX_EXPERIMENTS
    static const uint32_t configured = env_u32("QVX_CHUNK_TOKENS", 0), base = env_u32("QVX_CHUNK_BASE", CHUNK_BASE_TOKENS),
                          most = env_u32("QVX_CHUNK_MOST", 32);
#else
    constexpr uint32_t configured = 0, base = CHUNK_BASE_TOKENS, most = 32;
#endif
    uint32_t c = base_chunk_tokens(configured ? configured : base, L.B);
    while (c > 2048 && c > L.B) c -= L.B;
    if (!configured)
        while ((len + c - 1) / c > most && c * 2 <= 2048) c *= 2;
    return c;
}

// How many consecutive chunks of a (sequence, group) make one work item.  A chunk's result does
// not depend on it (the kernel keeps one state per chunk whatever run it streams it in), so
// unlike the chunk size this may look at the whole op: with many chunks per resident CTA the
// items grow, and what a CTA pays per item (the next record, the query rows, the queue) is paid
// less often; with few, items stay single chunks and the queue evens the CTAs out.  A run never
// exceeds RUN_TOKENS positions (its block ids ride in the item's record).
static const uint32_t RUN_TOKENS = 2048;
#ifndef QVX_SMALL_TOKENS_DEFAULT
#define QVX_SMALL_TOKENS_DEFAULT 256
#endif
#ifndef QVX_SPREAD_DEFAULT
#define QVX_SPREAD_DEFAULT 1
#endif
// An experiment build reads a fixed run length from QVX_RUN_CHUNKS at every op (the tests that show
// that the run length moves no bit use it); the shipped library always chooses by the rule below.
static uint32_t run_chunks_override() {
#ifdef QVX_EXPERIMENTS
    const char* v = getenv("QVX_RUN_CHUNKS");
    const long n = v ? atol(v) : 0;
    return n > 0 ? (uint32_t)n : 0u;
#else
    return 0u;
#endif
}
static uint32_t run_chunks_for(size_t total_chunks, uint32_t resident_ctas) {
    if (const uint32_t configured = run_chunks_override()) return configured;
    const size_t per_cta = total_chunks / std::max(1u, resident_ctas);
    return (uint32_t)std::min<size_t>(4, std::max<size_t>(1, per_cta / 6));
}

// The CTA that merges a sequence's splits keeps every split's maximum and row sum in shared
// memory: 64 bytes per split of the 64 KiB a CTA always has.
constexpr size_t MAX_CHUNKS = 1000;
static int32_t too_many_chunks(qvx_device* dev, size_t nch) {
    return fail(dev, QVX_ERR_UNSUPPORTED,
                "cuda backend splits a context into at most %zu chunks, this one needs %zu",
                MAX_CHUNKS, nch);
}

struct TableImage {
    size_t off_pos, off_table_at, off_blocks, off_items, bytes;
    size_t n_items, n_parts, n_counters, max_nch;
    uint32_t max_pos, chunk_blocks, item_words, run;
};

static int32_t validate_tables(qvx_device* dev, const Layout& L, size_t pool_blocks, size_t heads, size_t s,
                               const uint32_t* pos, const uint32_t* blocks, size_t n_blocks,
                               const uint32_t* table_at) {
    if (heads == 0 || heads % L.kvh != 0)
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: %zu tokens, %zu heads, %u KV heads of %u",
                    s, heads, L.kvh, L.d);
    if (s > 65535) return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: %zu tokens in one op (at most 65535)", s);
    if (n_blocks > 0x7fffffffu) return fail(dev, QVX_ERR_CORE, "block tables of %zu entries", n_blocks);
    uint32_t top = 0;  // (a running maximum, no branch per id: this loop is on every op's way to its first copy)
    for (size_t i = 0; i < n_blocks; i++) top = blocks[i] > top ? blocks[i] : top;
    if (n_blocks && top >= pool_blocks)
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: a block past the pool's %zu", pool_blocks);
    for (size_t t = 0; t < s; t++)
        if ((size_t)table_at[t] + pos[t] / L.B >= n_blocks)
            return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: token %zu has no block for position %u",
                        t, pos[t]);
    return QVX_OK;
}

// The last op's work list, kept per device: the layers of one decode step come one after the
// other with the same positions, so everything but the block ids is the same 48 times over.
struct PlanCache {
    bool valid = false;
    uint32_t B = 0, kvh = 0, d = 0, dtype = 0, layout = 0;
    size_t heads = 0, s = 0;
    bool split = false;
    uint32_t ctas = 0, knobs = 0;
    std::vector<uint32_t> pos;
    TableImage im{};                       // counts and sizes; the offsets depend on n_blocks and are redone
    std::vector<qvx_item_header> headers;  // in launch order
    std::vector<uint32_t> seq_off, count;  // per item: first block's offset in its sequence's table, blocks
};

static uint32_t run_tail_chunks();
// What the environment says about runs right now: a kept work list made under other settings is not reused.
static uint32_t run_knobs() { return run_chunks_override() * 65536u + run_tail_chunks(); }

static bool plan_hit(const PlanCache* c, const Layout& L, size_t heads, size_t s, const uint32_t* pos, bool split, uint32_t ctas) {
    return c && c->valid && c->knobs == run_knobs() && c->B == L.B && c->kvh == L.kvh && c->d == L.d && c->dtype == L.dtype && c->layout == L.layout &&
           c->heads == heads && c->s == s && c->split == split && c->ctas == ctas && memcmp(c->pos.data(), pos, 4 * s) == 0;
}

static void image_offsets(TableImage& im, size_t s, size_t n_blocks) {
    size_t off = 0;
    im.off_pos = off; off += 4 * s;
    im.off_table_at = off; off += 4 * s;
    im.off_blocks = off; off += 4 * n_blocks;
    off = (off + 15) & ~(size_t)15;
    im.off_items = off; off += 4ull * im.item_words * im.n_items;
    im.bytes = (off + 255) & ~(size_t)255;
}

// The runs a (sequence, group) of `nch` chunks is cut into, given the op's run length: runs of
// `run` chunks from the front; the last `tail` chunks stay single, so that the end of the launch
// has small items to even the CTAs out with.  Calls f(first chunk, chunks).
static uint32_t run_tail_chunks() {
#ifdef QVX_EXPERIMENTS
    const char* v = getenv("QVX_RUN_TAIL");
    return v ? (uint32_t)atol(v) : 0u;
#else
    return 0u;
#endif
}
template <typename F>
static void for_each_run(uint32_t nch, uint32_t run, uint32_t tail, F f) {
    const uint32_t singles = run > 1 ? std::min(nch, tail) : 0u, front = nch - singles;
    for (uint32_t c = 0; c < front; c += run) f(c, std::min(run, front - c));
    for (uint32_t c = front; c < nch; c++) f(c, 1u);
}

// Where the short work items go in the queue: items of fewer than `small_tokens` positions are taken
// out of the longest-first order and dealt out after the first `small_after` x (resident CTAs) items.
// The order changes no bit of any result (a chunk's arithmetic does not depend on when it runs).
struct QueueOrder { uint32_t small_tokens, small_after, spread; };
static QueueOrder queue_order() {
    QueueOrder qo{QVX_SMALL_TOKENS_DEFAULT, 0, QVX_SPREAD_DEFAULT};
#ifdef QVX_EXPERIMENTS
    if (const char* v = getenv("QVX_SMALL_TOKENS")) qo.small_tokens = (uint32_t)atol(v);
    if (const char* v = getenv("QVX_SMALL_AFTER")) qo.small_after = (uint32_t)atol(v);
    if (const char* v = getenv("QVX_SPREAD")) qo.spread = (uint32_t)atol(v);
#endif
    return qo;
}

// CTAs of the streaming attention kernel the device keeps resident for this geometry; 0 when another
// kernel serves it (one CTA per item there: items stay single chunks).
static uint32_t stream_ctas(const qvx_device* dev, const Layout& L, size_t heads) {
    if (!attn_split_supported(L, heads)) return 0;
    return (uint32_t)dev->prop.multiProcessorCount * (L.d <= 128 ? 2u : 1u);
}

// `ctas`: stream_ctas() of the device.
static TableImage plan_image(const Layout& L, size_t heads, size_t s, const uint32_t* pos, size_t n_blocks,
                             bool split, uint32_t ctas, PlanCache* cache = nullptr) {
    if (plan_hit(cache, L, heads, s, pos, split, ctas)) {
        TableImage im = cache->im;
        image_offsets(im, s, n_blocks);
        return im;
    }
    if (cache) cache->valid = false;
    TableImage im{};
    size_t group = heads / L.kvh, groups = L.kvh * ((group + 7) / 8);
    im.chunk_blocks = 1;
    size_t total_chunks = 0;
    for (size_t t = 0; t < s; t++) {
        im.max_pos = std::max(im.max_pos, pos[t]);
        if (!split) continue;
        const uint32_t chunk = chunk_tokens_for(L, pos[t] + 1u);
        size_t nch = ((size_t)pos[t] + chunk) / chunk;
        im.max_nch = std::max<size_t>(im.max_nch, nch);
        total_chunks += nch * groups;
        if (nch > 1) {
            im.n_parts += (size_t)attn_parts_per_group(L, (uint32_t)nch) * groups;
            im.n_counters += (size_t)attn_counters_per_group(L, (uint32_t)nch) * groups;
        }
    }
    im.run = split && ctas ? run_chunks_for(total_chunks, ctas) : 1u;
    for (size_t t = 0; split && t < s; t++) {
        const uint32_t chunk = chunk_tokens_for(L, pos[t] + 1u);
        const uint32_t nch = (uint32_t)(((size_t)pos[t] + chunk) / chunk);
        const uint32_t run = std::min(nch, std::max(1u, std::min(im.run, RUN_TOKENS / chunk)));
        im.chunk_blocks = std::max(im.chunk_blocks, run * (chunk / L.B));
        size_t runs = 0;
        for_each_run(nch, run, run_tail_chunks(), [&](uint32_t, uint32_t) { runs++; });
        im.n_items += runs * groups;
    }
    im.item_words = (QVX_ITEM_HEADER_WORDS + im.chunk_blocks + 3u) & ~3u;
    image_offsets(im, s, n_blocks);
    return im;
}

static void fill_image(const TableImage& im, uint8_t* img, const Layout& L, size_t heads, size_t s,
                       const uint32_t* pos, const uint32_t* blocks, size_t n_blocks, const uint32_t* table_at,
                       uint32_t ctas, PlanCache* cache = nullptr, bool split = true) {
    memcpy(img + im.off_pos, pos, 4 * s);
    memcpy(img + im.off_table_at, table_at, 4 * s);
    memcpy(img + im.off_blocks, blocks, 4 * n_blocks);
    if (im.n_items == 0) return;
    const uint32_t id_words = im.item_words - QVX_ITEM_HEADER_WORDS;
    if (plan_hit(cache, L, heads, s, pos, split, ctas)) {
        uint32_t* items = (uint32_t*)(img + im.off_items);
        for (size_t n = 0; n < cache->headers.size(); n++) {
            uint32_t* w = items + n * im.item_words;
            memcpy(w, &cache->headers[n], sizeof(qvx_item_header));
            const uint32_t* src = blocks + table_at[cache->headers[n].seq] + cache->seq_off[n];
            const uint32_t count = cache->count[n];
            memcpy(w + QVX_ITEM_HEADER_WORDS, src, 4 * count);
            if (count < id_words) memset(w + QVX_ITEM_HEADER_WORDS + count, 0, 4 * (id_words - count));
        }
        return;
    }
    if (cache) {
        cache->B = L.B; cache->kvh = L.kvh; cache->d = L.d; cache->dtype = L.dtype; cache->layout = L.layout;
        cache->heads = heads; cache->s = s; cache->split = split; cache->ctas = ctas; cache->knobs = run_knobs();
        cache->pos.assign(pos, pos + s);
        cache->im = im;
        cache->headers.resize(im.n_items); cache->seq_off.resize(im.n_items); cache->count.resize(im.n_items);
    }
    const uint32_t max_chunk = im.chunk_blocks * L.B;
    const uint32_t group = (uint32_t)(heads / L.kvh), gpk = (group + 7) / 8, groups = L.kvh * gpk;
    // Longest first, so the short tails fill the end of the launch.  The order is a function
    // of the lengths alone: a counting sort by tokens, ties in (sequence, group, chunk) order.
    struct Key { uint32_t tokens, seq, grp, c, run, nch; };
    std::vector<Key> keys;
    keys.reserve(im.n_items);
    std::vector<uint32_t> part_base(s), counter_base(s);
    uint32_t part = 0, counter = 0;
    for (size_t t = 0; t < s; t++) {
        const uint32_t len = pos[t] + 1u, chunk = chunk_tokens_for(L, len), nch = (len + chunk - 1) / chunk;
        const uint32_t run = std::min(nch, std::max(1u, std::min(im.run, RUN_TOKENS / chunk)));
        part_base[t] = part; counter_base[t] = counter;
        if (nch > 1) { part += attn_parts_per_group(L, nch) * groups; counter += attn_counters_per_group(L, nch) * groups; }
        for (uint32_t grp = 0; grp < groups; grp++)
            for_each_run(nch, run, run_tail_chunks(), [&](uint32_t c, uint32_t r) {
                keys.push_back(Key{std::min(len, (c + r) * chunk) - c * chunk, (uint32_t)t, grp, c, r, nch});
            });
    }
    // Among items of equal size a sequence's chunks sit at even distances over the whole queue (chunk c of n at the
    // fraction c / n of it): the chunks of one merge node then arrive rounds apart, not together, and the queue's
    // last round holds at most one full chunk of a node -- so a node's last arrival finds the others long published
    // and folds them while it streams, instead of eight CTAs finishing a node's chunks at once and one of them
    // waiting for seven publications.  (`spread` 0: chunk 0 of every sequence, then chunk 1 of every sequence, ...,
    // which bunches a long sequence's last chunks in the last round; 2: by place alone, sizes not looked at.)
    if (queue_order().spread)
        std::stable_sort(keys.begin(), keys.end(), [](const Key& a, const Key& b) { return (uint64_t)a.c * b.nch < (uint64_t)b.c * a.nch; });
    else
        std::stable_sort(keys.begin(), keys.end(), [](const Key& a, const Key& b) { return a.c < b.c; });
    // (a counting sort: tokens <= max_chunk, and this runs once per op on the host's critical path)
    std::vector<uint32_t> start(max_chunk + 2, 0);
    for (const Key& k : keys) start[max_chunk - k.tokens + 1]++;
    for (uint32_t v = 0; v <= max_chunk; v++) start[v + 1] += start[v];
    std::vector<uint32_t> order(keys.size());
    if (queue_order().spread == 2)
        for (uint32_t i = 0; i < keys.size(); i++) order[i] = i;  // by place in the sequence alone: sizes are not looked at (the short ones still go first, below)
    else
        for (uint32_t i = 0; i < keys.size(); i++) order[start[max_chunk - keys[i].tokens]++] = i;
    // The short items do not go last.  Nearly every short item is a sequence's last, partly filled chunk,
    // and whichever chunk of a sequence finishes last merges the others' results: at the very end of
    // the queue that merge (a few rounds of loads) lasts longer than the item itself and every CTA's exit
    // waits for one.  Dealt out first instead (or after the first `small_after` x CTAs items), the short ones
    // are finished while every CTA still streams, the queue ends with long items -- which fold the others'
    // results while they stream -- and the CTAs run dry within a fraction of a long item of one another.
    const QueueOrder qo = queue_order();
    if (ctas && qo.small_tokens) {
        const size_t front = std::min<size_t>((size_t)qo.small_after * ctas, order.size());
        std::vector<uint32_t> small, rest;
        for (size_t n = front; n < order.size(); n++)
            (keys[order[n]].tokens < qo.small_tokens ? small : rest).push_back(order[n]);
        if (rest.size() >= ctas) {  // (with fewer long items than CTAs there is no long tail to end on)
            std::copy(small.begin(), small.end(), order.begin() + front);
            std::copy(rest.begin(), rest.end(), order.begin() + front + small.size());
        }
    }
    uint32_t* items = (uint32_t*)(img + im.off_items);
    for (size_t n = 0; n < keys.size(); n++) {
        const Key& k = keys[order[n]];
        const uint32_t t = k.seq, len = pos[t] + 1u, chunk = chunk_tokens_for(L, len), nch = (len + chunk - 1) / chunk;
        uint32_t kvh = k.grp / gpk, sub = k.grp % gpk;
        uint32_t* w = items + n * im.item_words;
        qvx_item_header h{};
        h.seq = t;
        h.tokens = k.tokens;
        h.head0 = kvh * group + sub * 8;
        h.nheads_kv = std::min(8u, group - sub * 8) | (kvh << 16);
        h.part0 = nch > 1 ? part_base[t] + k.grp * attn_parts_per_group(L, nch) : 0xffffffffu;
        h.part = nch > 1 ? h.part0 + k.c : 0xffffffffu;
        h.nch = nch;
        h.counter = nch > 1 ? counter_base[t] + k.grp * attn_counters_per_group(L, nch) : 0;  // the group's first arrival counter
        h.chunk_tokens = chunk;
        h.run = k.run;
        memcpy(w, &h, sizeof h);
        uint32_t count = (k.tokens + L.B - 1) / L.B;
        const uint32_t* src = blocks + table_at[t] + (size_t)k.c * (chunk / L.B);
        for (uint32_t b = 0; b < id_words; b++) w[QVX_ITEM_HEADER_WORDS + b] = b < count ? src[b] : 0;
        if (cache) { cache->headers[n] = h; cache->seq_off[n] = k.c * (chunk / L.B); cache->count[n] = count; }
    }
    if (cache) cache->valid = true;
}

static void bind_image(qvx_tables* t, const TableImage& im, void* dmem) {
    uint8_t* d = (uint8_t*)dmem;
    t->dmem = dmem; t->dmem_bytes = im.bytes;
    t->d_pos = (uint32_t*)(d + im.off_pos);
    t->d_table_at = (uint32_t*)(d + im.off_table_at);
    t->d_blocks = (uint32_t*)(d + im.off_blocks);
    t->d_items = (uint32_t*)(d + im.off_items);
    t->n_items = im.n_items; t->n_parts = im.n_parts; t->n_counters = im.n_counters;
    t->max_pos = im.max_pos; t->chunk_blocks = im.chunk_blocks; t->item_words = im.item_words;
}

static int32_t ensure_partials(qvx_device* dev, size_t floats, size_t counters) {
    if (floats * 4 <= dev->partials_cap && counters <= dev->counters_cap && dev->queue) return QVX_OK;
    // Work queued earlier may still use the old scratch.
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return check_cuda(dev, e, "partials");
    if (floats * 4 > dev->partials_cap) {
        if (dev->partials) cudaFree(dev->partials);
        dev->partials = nullptr; dev->partials_cap = 0;
        size_t cap = (std::max<size_t>(floats * 4 * 5 / 4, 1u << 20) + 255) & ~(size_t)255;
        e = cudaMalloc(&dev->partials, 2 * cap);  // two halves, used by alternate launches
        if (e != cudaSuccess) return check_cuda(dev, e, "partials");
        dev->partials_cap = cap;
    }
    if (!dev->queue) {
        e = cudaMalloc((void**)&dev->queue, 16);
        if (e == cudaSuccess) e = cudaMemset(dev->queue, 0, 16);
        if (e != cudaSuccess) return check_cuda(dev, e, "work queue");
    }
    if (counters > dev->counters_cap) {
        if (dev->counters) cudaFree(dev->counters);
        dev->counters = nullptr; dev->counters_cap = 0;
        size_t cap = std::max<size_t>(counters * 2, 4096);
        e = cudaMalloc((void**)&dev->counters, 2 * cap * 4);
        if (e == cudaSuccess) e = cudaMemset(dev->counters, 0, 2 * cap * 4);  // every launch leaves them at zero again
        if (e != cudaSuccess) return check_cuda(dev, e, "arrival counters");
        dev->counters_cap = cap;
    }
    return QVX_OK;
}

// Attention, with the step's KV append in front of it when k_new / v_new are given: inside the
// same launch where the kernel can (native-layout pools), as its own launch otherwise.
static int32_t run_attention(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                             uint32_t variant_flags, cudaStream_t s, const float* k_new = nullptr, const float* v_new = nullptr) {
    const uint32_t variant = variant_flags & 0xffu;
    bool split_ok = attn_split_supported(t->L, t->heads) && t->n_items > 0;
    if (variant == QVX_ATTN_SPLIT && !attn_split_supported(t->L, t->heads))
        return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no split attention kernel for this geometry");
    const bool split = variant != QVX_ATTN_EXACT && split_ok;
    const bool fused = split && k_new && attn_split_fuses_append(t->L, t->heads);
    if (k_new && !fused) {
        int32_t rc = launch_kv_rows(dev, t->L, const_cast<void*>(pool), k_new, v_new, (size_t)t->L.kvh * t->L.d, nullptr, t->d_pos,
                                    t->d_blocks, t->d_table_at, t->s, t->pool_blocks, QVX_K_APPEND, s);
        if (rc) return rc;
    }
    if (!split) return launch_attn_exact(dev, t, pool, q, out, s);
    int32_t rc = ensure_partials(dev, attn_partial_floats(t), t->n_counters);
    if (rc) return rc;
    const uint32_t half = dev->scratch_half;
    dev->scratch_half ^= 1u;
    const bool overlap = (variant_flags & QVX_ATTN_POOL_SETTLED) != 0;
    return launch_attn_split(dev, t, pool, q, out, (float*)((char*)dev->partials + half * dev->partials_cap),
                             dev->counters + half * dev->counters_cap, dev->queue + 2 * half, fused ? k_new : nullptr,
                             fused ? v_new : nullptr, overlap, s);
}

}  // namespace qvx

using namespace qvx;

// =================================================================================================
extern "C" {

size_t qvx_block_bytes(const qvx_geometry* geo) { return geometry_ok(geo) ? (size_t)make_layout(geo).block_bytes : 0; }

size_t qvx_elem_offset(const qvx_geometry* geo, size_t at, int kv, size_t g, size_t i) {
    Layout L = make_layout(geo);
    return (at / L.B) * (size_t)L.block_bytes + in_block_offset(L, (uint32_t)(at % L.B), kv ? 1u : 0u, (uint32_t)g, (uint32_t)i);
}

const char* qvx_name(void) { return "cuda"; }

int32_t qvx_open(const qvx_config* cfg, qvx_device** out) {
    if (!out) return QVX_ERR_SHAPE;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(nullptr, QVX_ERR_DEVICE, "cuda device error: no CUDA device (%s); this backend has no CPU path",
                    e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
    }
    int ord = cfg ? cfg->device : 0;
    if (ord < 0 || ord >= n) return fail(nullptr, QVX_ERR_DEVICE, "cuda device error: no device %d (%d present)", ord, n);
    if ((e = cudaSetDevice(ord)) != cudaSuccess) return check_cuda(nullptr, e, "cudaSetDevice");
    qvx_device* dev = new qvx_device;
    dev->ordinal = ord;
    if (cfg) dev->cfg = *cfg;
    cudaGetDeviceProperties(&dev->prop, ord);
    if (dev->prop.major < 9) {
        int major = dev->prop.major, minor = dev->prop.minor;
        delete dev;
        return fail(nullptr, QVX_ERR_UNSUPPORTED, "cuda backend is built for sm_100a; device %d is sm_%d%d", ord, major, minor);
    }
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    dev->usage.capacity = dev->cfg.capacity ? dev->cfg.capacity : free_b;
    DeviceExtras* x = new DeviceExtras;
    e = cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&x->h2d, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&x->d2h, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&x->kernels2, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&x->status_host, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *x->status_host = 0;
        e = cudaHostGetDevicePointer((void**)&x->status_dev, x->status_host, 0);
    }
    if (e != cudaSuccess) {
        delete x; delete dev;
        return check_cuda(nullptr, e, "open");
    }
    {
        std::lock_guard<std::mutex> lk(g_extras_mu);
        g_extras.emplace_back(dev, x);
    }
    *out = dev;
    return QVX_OK;
}

void qvx_close(qvx_device* dev) {
    if (!dev) return;
    cudaSetDevice(dev->ordinal);
    cudaDeviceSynchronize();
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        drain_timers(dev);
        if (DeviceExtras* x = extras(dev)) {
            for (HostOp& op : x->ops) retire(dev, x, op);
            x->ops.clear();
        }
    }
    for (cudaEvent_t ev : dev->event_pool) cudaEventDestroy(ev);
    delete static_cast<PlanCache*>(dev->plan_cache);
    if (dev->partials) cudaFree(dev->partials);
    if (dev->counters) cudaFree(dev->counters);
    if (dev->queue) cudaFree(dev->queue);
    if (dev->staging) cudaFreeHost(dev->staging);
    if (dev->dstaging) cudaFree(dev->dstaging);
    DeviceExtras* x = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_extras_mu);
        for (size_t i = 0; i < g_extras.size(); i++)
            if (g_extras[i].first == dev) { x = g_extras[i].second; g_extras.erase(g_extras.begin() + i); break; }
    }
    if (x) {
        for (cudaEvent_t ev : x->sync_events) cudaEventDestroy(ev);
        cudaStreamDestroy(x->h2d); cudaStreamDestroy(x->d2h); cudaStreamDestroy(x->kernels2);
        cudaFreeHost(x->status_host);
        delete x;
    }
    cudaStreamDestroy(dev->stream);
    delete dev;
}

int32_t qvx_describe(qvx_device* dev, char* out, size_t cap) {
    if (!dev || !out || !cap) return QVX_ERR_SHAPE;
    snprintf(out, cap, "%s (sm_%d%d, %d SMs, %.1f GB, device %d)", dev->prop.name, dev->prop.major, dev->prop.minor,
             dev->prop.multiProcessorCount, (double)dev->prop.totalGlobalMem / 1e9, dev->ordinal);
    return QVX_OK;
}

int32_t qvx_supports(qvx_device*, uint32_t dtype) { return dtype <= QVX_F16 ? 1 : 0; }

const char* qvx_last_error(qvx_device* dev) { return dev ? dev->last_error.c_str() : g_last_error.c_str(); }

uint64_t qvx_kv_pool(qvx_device* dev) { return dev ? dev->cfg.kv_pool : 0; }

uint64_t qvx_max_arena(qvx_device* dev) { return dev ? (uint64_t)dev->prop.totalGlobalMem : 0; }

int32_t qvx_routes_moe_attention(qvx_device* dev, size_t, size_t, size_t s) { return dev && s > 0 && s <= 65535; }

int32_t qvx_alloc(qvx_device* dev, size_t len, qvx_buffer** out) {
    if (!dev || !out) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return new_buffer(dev, len, true, out);
}

int32_t qvx_upload(qvx_device* dev, const void* data, size_t len, qvx_buffer** out) {
    if (!dev || !out || (!data && len)) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    int32_t rc = new_buffer(dev, len, false, out);
    if (rc) return rc;
    uint64_t t0 = now_ns();
    cudaError_t e = cudaMemcpy((*out)->ptr, data, len, cudaMemcpyHostToDevice);
    dev->xfer.transfer_ns += now_ns() - t0;
    dev->xfer.uploads++; dev->xfer.upload_bytes += len;
    return check_cuda(dev, e, "upload");
}

int32_t qvx_write(qvx_device* dev, qvx_buffer* buf, size_t offset, const void* data, size_t len) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    int32_t rc = buffer_of(dev, buf);
    if (rc) return rc;
    if (!buf->arena) return fail(dev, QVX_ERR_DEVICE, "cuda device error: only an arena (alloc) can be written");
    if (offset > buf->len || len > buf->len - offset)
        return fail(dev, QVX_ERR_DEVICE, "cuda device error: %zu bytes at %zu are outside a %zu-byte buffer", len, offset, buf->len);
    cudaSetDevice(dev->ordinal);
    uint64_t t0 = now_ns();
    cudaError_t e = cudaMemcpy((char*)buf->ptr + offset, data, len, cudaMemcpyHostToDevice);
    dev->xfer.transfer_ns += now_ns() - t0;
    dev->xfer.uploads++; dev->xfer.upload_bytes += len;
    return check_cuda(dev, e, "write");
}

int32_t qvx_read(qvx_device* dev, qvx_buffer* buf, size_t offset, void* data, size_t len) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    int32_t rc = buffer_of(dev, buf);
    if (rc) return rc;
    if (offset > buf->len || len > buf->len - offset)
        return fail(dev, QVX_ERR_DEVICE, "cuda device error: %zu bytes at %zu are outside a %zu-byte buffer", len, offset, buf->len);
    cudaSetDevice(dev->ordinal);
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(data, (char*)buf->ptr + offset, len, cudaMemcpyDeviceToHost);
    return check_cuda(dev, e, "read");
}

void qvx_retain(qvx_buffer* buf) {
    if (!buf) return;
    std::lock_guard<std::mutex> lk(buf->dev->mu);
    buf->refs++;
}

void qvx_free(qvx_buffer* buf) {
    if (!buf) return;
    qvx_device* dev = buf->dev;
    {
        std::lock_guard<std::mutex> lk(dev->mu);
        if (--buf->refs > 0) return;
        cudaSetDevice(dev->ordinal);
        cudaDeviceSynchronize();
        cudaFree(buf->ptr);
        dev->usage.used -= buf->len;
    }
    delete buf;
}

void* qvx_buffer_ptr(qvx_buffer* buf) { return buf ? buf->ptr : nullptr; }
size_t qvx_buffer_len(qvx_buffer* buf) { return buf ? buf->len : 0; }

int32_t qvx_get_usage(qvx_device* dev, qvx_usage* out) {
    if (!dev || !out) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    *out = dev->usage;
    return QVX_OK;
}

int32_t qvx_get_transfers(qvx_device* dev, qvx_transfer_stats* out) {
    if (!dev || !out) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    drain_timers(dev);
    *out = dev->xfer;
    return QVX_OK;
}

int32_t qvx_get_kernel_times(qvx_device* dev, qvx_kernel_times* out) {
    if (!dev || !out) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    drain_timers(dev);
    *out = dev->ktimes;
    return check_status(dev);
}

int32_t qvx_reset_kernel_times(qvx_device* dev) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    drain_timers(dev);
    memset(&dev->ktimes, 0, sizeof dev->ktimes);
    return QVX_OK;
}

// ---- kernels on device memory ---------------------------------------------------------------------
int32_t qvx_kv_sync(qvx_device* dev, const qvx_geometry* geo, void* pool, size_t pool_blocks, const float* rows,
                    const uint32_t* sync_to, size_t n, void* stream) {
    if (!dev) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    Layout L = make_layout(geo);
    size_t kv_out = (size_t)L.kvh * L.d;
    return launch_kv_rows(dev, L, pool, rows, rows + kv_out, 2 * kv_out, sync_to, nullptr, nullptr, nullptr, n,
                          pool_blocks, QVX_K_SYNC, (cudaStream_t)stream);
}

int32_t qvx_kv_append(qvx_device* dev, const qvx_geometry* geo, void* pool, size_t pool_blocks, const float* k_new,
                      const float* v_new, const uint32_t* pos, const uint32_t* blocks, const uint32_t* table_at,
                      size_t s, void* stream) {
    if (!dev) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    Layout L = make_layout(geo);
    size_t kv_out = (size_t)L.kvh * L.d;
    return launch_kv_rows(dev, L, pool, k_new, v_new, kv_out, nullptr, pos, blocks, table_at, s, pool_blocks,
                          QVX_K_APPEND, (cudaStream_t)stream);
}

int32_t qvx_tables_create(qvx_device* dev, const qvx_geometry* geo, size_t pool_blocks, size_t heads, size_t s,
                          const uint32_t* pos, const uint32_t* blocks, size_t n_blocks, const uint32_t* table_at,
                          qvx_tables** out) {
    if (!dev || !out) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    Layout L = make_layout(geo);
    int32_t rc = validate_tables(dev, L, pool_blocks, heads, s, pos, blocks, n_blocks, table_at);
    if (rc) return rc;
    const uint32_t ctas = stream_ctas(dev, L, heads);
    TableImage im = plan_image(L, heads, s, pos, n_blocks, attn_split_supported(L, heads), ctas);
    if (im.max_nch > MAX_CHUNKS) return too_many_chunks(dev, im.max_nch);
    std::vector<uint8_t> img(im.bytes);
    fill_image(im, img.data(), L, heads, s, pos, blocks, n_blocks, table_at, ctas);
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, im.bytes);
    if (e != cudaSuccess) return check_cuda(dev, e, "tables");
    e = cudaMemcpy(d, img.data(), im.bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(d); return check_cuda(dev, e, "tables"); }
    qvx_tables* t = new qvx_tables;
    t->dev = dev; t->L = L; t->pool_blocks = pool_blocks; t->heads = heads; t->s = s; t->n_blocks = n_blocks;
    bind_image(t, im, d);
    t->owns_dmem = true;
    // Grow the scratch now, so a later launch never has to.
    rc = ensure_partials(dev, attn_partial_floats(t), t->n_counters);
    if (rc) { cudaFree(d); delete t; return rc; }
    *out = t;
    return QVX_OK;
}

void qvx_tables_free(qvx_tables* t) {
    if (!t) return;
    if (t->owns_dmem && t->dmem) {
        std::lock_guard<std::mutex> lk(t->dev->mu);
        cudaSetDevice(t->dev->ordinal);
        cudaFree(t->dmem);
    }
    delete t;
}
const uint32_t* qvx_tables_pos(qvx_tables* t) { return t ? t->d_pos : nullptr; }
const uint32_t* qvx_tables_blocks(qvx_tables* t) { return t ? t->d_blocks : nullptr; }
const uint32_t* qvx_tables_table_at(qvx_tables* t) { return t ? t->d_table_at : nullptr; }

int32_t qvx_attn_decode(qvx_device* dev, qvx_tables* tables, const void* pool, const float* q, float* out,
                        uint32_t variant, void* stream) {
    if (!dev || !tables || tables->dev != dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return run_attention(dev, tables, pool, q, out, variant, (cudaStream_t)stream);
}

int32_t qvx_kv_append_attn_decode(qvx_device* dev, qvx_tables* tables, void* pool, const float* k_new, const float* v_new,
                                  const float* q, float* out, uint32_t variant, void* stream) {
    if (!dev || !tables || tables->dev != dev || !k_new || !v_new) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return run_attention(dev, tables, pool, q, out, variant, (cudaStream_t)stream, k_new, v_new);
}

int32_t qvx_block_copy(qvx_device* dev, const qvx_geometry* geo, void* pool, size_t pool_blocks, const uint32_t* src,
                       const uint32_t* dst, size_t n, void* stream) {
    if (!dev) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return launch_block_copy(dev, make_layout(geo), pool, src, dst, n, pool_blocks, (cudaStream_t)stream);
}

// ---- the op with host memory ----------------------------------------------------------------------
static bool prelude_ok(const qvx_prelude* p) {
    if (!p || !p->rope) return false;
    if (p->has_clip && !(p->clip >= 0.0f)) return false;  // Rust's clamp(-c, c) panics on c < 0 or NaN
    return (p->q_norm == nullptr) == (p->k_norm == nullptr);
}

// `pre` (host pointers), when given, runs the prelude on the staged q, k_new and v_new and copies
// the new rows back into k_back / v_back.
// The device's address for `bytes` of the caller's host array, or null when the device cannot reach it with plain
// 16-byte stores: memory that is not page-locked, not mapped, or not 16-byte aligned.
static float* mapped_host_pointer(const qvx_device* dev, const void* host, size_t bytes) {
    if (!host || ((uintptr_t)host & 15u)) return nullptr;
    cudaPointerAttributes at{}, end{};
    if (cudaPointerGetAttributes(&at, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (at.type != cudaMemoryTypeHost || !at.devicePointer) return nullptr;
    // (memory page-locked under another device's context may not be mapped for this one: it takes the copy)
    if (at.device != dev->ordinal) return nullptr;
    // (the whole range must be page-locked: look at its last byte as well)
    if (cudaPointerGetAttributes(&end, (const char*)host + bytes - 1) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (end.type != cudaMemoryTypeHost || !end.devicePointer || end.device != dev->ordinal) return nullptr;
    if ((const char*)end.devicePointer - (const char*)at.devicePointer != (ptrdiff_t)(bytes - 1)) return nullptr;
    return (float*)at.devicePointer;
}

static int32_t paged_attention_submit(qvx_device* dev, qvx_buffer* pool, const qvx_geometry* geo, size_t heads,
                                      size_t s, const float* q, const float* k_new, const float* v_new,
                                      const uint32_t* pos, const uint32_t* blocks, size_t n_blocks,
                                      const uint32_t* table_at, const float* sync, const uint32_t* sync_to,
                                      size_t n_sync, float* out, uint32_t variant, const qvx_prelude* pre = nullptr,
                                      float* k_back = nullptr, float* v_back = nullptr, bool serial = false) {
    // `serial`: the caller waits for this op right away and nothing else is in flight, so copies in, kernels and
    // copies out all go on the device's own stream in order: no event hand-over between streams (each costs
    // microseconds of latency that nothing would hide).
    uint64_t t0 = now_ns();
    if (pre && !prelude_ok(pre))
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: a prelude needs a RoPE table, a clip >= 0 and both norms or neither");
    int32_t rc = buffer_of(dev, pool);
    if (rc) return rc;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    if (!pool->arena) return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: the KV pool is not an arena");
    Layout L = make_layout(geo);
    const size_t held = pool->len / L.block_bytes;
    rc = validate_tables(dev, L, held, heads, s, pos, blocks, n_blocks, table_at);
    if (rc) return rc;
    for (size_t i = 0; i < n_sync; i++)
        if (sync_to[i] / L.B >= held)
            return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: a block past the pool's %zu", held);
    if ((variant & 0xffu) == QVX_ATTN_SPLIT && !attn_split_supported(L, heads))
        return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no split attention kernel for this geometry");
    if (s == 0 && n_sync == 0) return QVX_OK;

    const size_t kv_out = (size_t)L.kvh * L.d, q_out = heads * L.d;
    const bool split = attn_split_supported(L, heads) && (variant & 0xffu) != QVX_ATTN_EXACT;
    // QVX_ATTN_POOL_SETTLED on a host op: the caller's word that no op still in flight writes the blocks
    // this op reads or writes (the ops of one decode step serve different layers).  Such ops alternate
    // between two kernel streams, each tied to one half of the scratch, so that an op's kernel fills
    // the SMs the previous op's kernel leaves at its end; an op without the flag waits for both.
    const bool independent = (variant & QVX_ATTN_POOL_SETTLED) != 0 && split && n_sync == 0 && s > 0;
    variant &= 0xffu;  // (the streams give the overlap: no programmatic dependent launch here)
    if (!dev->plan_cache) dev->plan_cache = new PlanCache;
    PlanCache* cache = static_cast<PlanCache*>(dev->plan_cache);
    const uint32_t ctas = stream_ctas(dev, L, heads);
    TableImage im = plan_image(L, heads, s, pos, n_blocks, split, ctas, cache);
    if (im.max_nch > MAX_CHUNKS) return too_many_chunks(dev, im.max_nch);
    // Staged on the device for this op: the tables image, sync_to, q, k_new, v_new, sync rows, out.
    auto up = [](size_t b) { return (b + 255) & ~(size_t)255; };
    const bool norms = pre && pre->q_norm;
    const size_t o_img = 0, o_syncto = o_img + im.bytes, o_q = o_syncto + up(4 * n_sync),
                 o_k = o_q + up(4 * s * q_out), o_v = o_k + up(4 * s * kv_out), o_sync = o_v + up(4 * s * kv_out),
                 o_out = o_sync + up(8 * n_sync * kv_out), o_rope = o_out + up(4 * s * q_out),
                 o_qn = o_rope + (pre ? up(4 * s * L.d) : 0), o_kn = o_qn + (norms ? up(4 * q_out) : 0),
                 total = o_kn + (norms ? up(4 * kv_out) : 0);
    DeviceExtras* x = extras(dev);
    size_t base = 0;
    rc = take_slice(dev, x, total, &base);
    if (rc) return rc;
    uint8_t* hs = (uint8_t*)dev->staging + base;
    uint8_t* ds = (uint8_t*)dev->dstaging + base;
    // From here on the op is in the list: whatever happens, its slice and tables go back at a drain.
    x->ops.emplace_back();
    HostOp& op = x->ops.back();
    op.begin = base; op.end = base + total;
    op.in_done = take_event(x); op.kernels_done = take_event(x); op.out_done = take_event(x);

    serial = serial && x->ops.size() == 1;  // (this op is the only one in the list)
    // The scratch half the attention launch will take decides the stream: every user of a half is on
    // the same stream, so two launches never share a half at the same time.
    const uint32_t lane = split && !serial ? (dev->scratch_half & 1u) : 0u;
    cudaStream_t h2d = serial ? dev->stream : x->h2d, cs = lane ? x->kernels2 : dev->stream, d2h = serial ? dev->stream : x->d2h;
    if (!serial) cudaEventRecord(op.out_done, x->d2h);  // re-recorded after the copy out; a failed op's slice is free at once
    // The caller's arrays go first, straight from where they are (pinned memory makes these true asynchronous
    // copies; from pageable memory the runtime stages them and the call blocks for as long): they are on their
    // way while the work list is built below.
    cudaError_t e = cudaSuccess;
    size_t in_bytes = im.bytes + 4 * n_sync;
    auto copy_in = [&](size_t off, const void* src, size_t bytes) {
        if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(ds + off, src, bytes, cudaMemcpyHostToDevice, h2d);
        in_bytes += bytes;
    };
    copy_in(o_q, q, 4 * s * q_out);
    copy_in(o_k, k_new, 4 * s * kv_out);
    copy_in(o_v, v_new, 4 * s * kv_out);
    copy_in(o_sync, sync, 8 * n_sync * kv_out);
    if (pre) {
        copy_in(o_rope, pre->rope, 4 * s * L.d);
        if (norms) { copy_in(o_qn, pre->q_norm, 4 * q_out); copy_in(o_kn, pre->k_norm, 4 * kv_out); }
    }

    fill_image(im, hs + o_img, L, heads, s, pos, blocks, n_blocks, table_at, ctas, cache, split);
    // A position listed twice: the later row wins (the reference writes them in list order).
    uint32_t* st = (uint32_t*)(hs + o_syncto);
    {
        std::unordered_set<uint32_t> seen;
        seen.reserve(n_sync * 2);
        for (size_t i = n_sync; i-- > 0;) st[i] = seen.insert(sync_to[i]).second ? sync_to[i] : 0xffffffffu;
    }
    qvx_tables* t = new qvx_tables;
    t->dev = dev; t->L = L; t->pool_blocks = held; t->heads = heads; t->s = s; t->n_blocks = n_blocks;
    bind_image(t, im, ds + o_img);
    t->owns_dmem = false;
    op.tables = t;
    if (split) {
        rc = ensure_partials(dev, attn_partial_floats(t), t->n_counters);
        if (rc) return rc;
    }
    if (!serial && !independent && x->last_kernels[lane ^ 1u]) cudaStreamWaitEvent(cs, x->last_kernels[lane ^ 1u], 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ds + o_img, hs + o_img, im.bytes + up(4 * n_sync), cudaMemcpyHostToDevice, h2d);
    if (e != cudaSuccess) return check_cuda(dev, e, "copy in");
    if (!serial) {
        cudaEventRecord(op.in_done, h2d);
        cudaStreamWaitEvent(cs, op.in_done, 0);
    }

    if (pre && s) {  // clip, norms, RoPE on the staged projections: sim.rs:333-357
        qvx_prelude dp = *pre;
        dp.rope = (const float*)(ds + o_rope);
        dp.q_norm = norms ? (const float*)(ds + o_qn) : nullptr;
        dp.k_norm = norms ? (const float*)(ds + o_kn) : nullptr;
        rc = launch_attn_prelude(dev, L, heads, s, (float*)(ds + o_q), (float*)(ds + o_k), (float*)(ds + o_v), &dp, cs);
        if (rc) return rc;
    }
    // sync rows, then the new rows, then attention: sim.rs:385-429.
    const float* d_sync = (const float*)(ds + o_sync);
    rc = launch_kv_rows(dev, L, pool->ptr, d_sync, d_sync + kv_out, 2 * kv_out, (const uint32_t*)(ds + o_syncto), nullptr,
                        nullptr, nullptr, n_sync, held, QVX_K_SYNC, cs);
    // The outputs go straight into the caller's array when the device can address it (pinned memory, which
    // unified addressing maps into the device's address space): the kernel's stores cross the bus while it runs,
    // and the op needs no copy out.  Pageable (or misaligned) memory takes the staged copy.
    float* d_out = s ? mapped_host_pointer(dev, out, 4 * s * q_out) : nullptr;
    const bool out_direct = d_out != nullptr;
    if (!out_direct) d_out = (float*)(ds + o_out);
    if (rc == QVX_OK && s)
        rc = run_attention(dev, t, pool->ptr, (const float*)(ds + o_q), d_out, variant, cs,
                           (const float*)(ds + o_k), (const float*)(ds + o_v));
    if (rc) return rc;
    if (!serial) {
        cudaEventRecord(op.kernels_done, cs);
        x->last_kernels[lane] = op.kernels_done;
        cudaStreamWaitEvent(d2h, op.kernels_done, 0);
    }
    if (s) {
        if (!out_direct) e = cudaMemcpyAsync(out, ds + o_out, 4 * s * q_out, cudaMemcpyDeviceToHost, d2h);
        if (e == cudaSuccess && k_back) e = cudaMemcpyAsync(k_back, ds + o_k, 4 * s * kv_out, cudaMemcpyDeviceToHost, d2h);
        if (e == cudaSuccess && v_back) e = cudaMemcpyAsync(v_back, ds + o_v, 4 * s * kv_out, cudaMemcpyDeviceToHost, d2h);
        if (e != cudaSuccess) return check_cuda(dev, e, "copy out");
    }
    cudaEventRecord(op.out_done, d2h);
    // A later op's copies overwrite nothing this op reads: its slice is its own until out_done.
    dev->xfer.submissions++;
    dev->xfer.activations_in += in_bytes;
    dev->xfer.activations_out += 4 * s * q_out;
    dev->xfer.submit_ns += now_ns() - t0;
    return QVX_OK;
}

int32_t qvx_paged_attention_host_async(qvx_device* dev, qvx_buffer* pool, const qvx_geometry* geo, size_t heads,
                                       size_t s, const float* q, const float* k_new, const float* v_new,
                                       const uint32_t* pos, const uint32_t* blocks, size_t n_blocks,
                                       const uint32_t* table_at, const float* sync, const uint32_t* sync_to,
                                       size_t n_sync, float* out, uint32_t variant) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return paged_attention_submit(dev, pool, geo, heads, s, q, k_new, v_new, pos, blocks, n_blocks, table_at, sync,
                                  sync_to, n_sync, out, variant);
}

int32_t qvx_wait(qvx_device* dev) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    return wait_locked(dev);
}

int32_t qvx_paged_attention_host(qvx_device* dev, qvx_buffer* pool, const qvx_geometry* geo, size_t heads, size_t s,
                                 const float* q, const float* k_new, const float* v_new, const uint32_t* pos,
                                 const uint32_t* blocks, size_t n_blocks, const uint32_t* table_at, const float* sync,
                                 const uint32_t* sync_to, size_t n_sync, float* out, uint32_t variant) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    const bool alone = extras(dev)->ops.empty();
    int32_t rc = paged_attention_submit(dev, pool, geo, heads, s, q, k_new, v_new, pos, blocks, n_blocks, table_at,
                                        sync, sync_to, n_sync, out, variant, nullptr, nullptr, nullptr, alone);
    int32_t rc2 = wait_locked(dev, alone);
    return rc ? rc : rc2;
}

int32_t qvx_attention_stage_host(qvx_device* dev, qvx_buffer* pool, const qvx_geometry* geo, size_t heads, size_t s,
                                 const float* q, float* k_new, float* v_new, const qvx_prelude* prelude, const uint32_t* pos,
                                 const uint32_t* blocks, size_t n_blocks, const uint32_t* table_at, const float* sync,
                                 const uint32_t* sync_to, size_t n_sync, float* out, uint32_t variant) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    if (!prelude) return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: no prelude given");
    const bool alone = extras(dev)->ops.empty();
    int32_t rc = paged_attention_submit(dev, pool, geo, heads, s, q, k_new, v_new, pos, blocks, n_blocks, table_at, sync,
                                        sync_to, n_sync, out, variant, prelude, k_new, v_new, alone);
    int32_t rc2 = wait_locked(dev, alone);
    return rc ? rc : rc2;
}

int32_t qvx_attn_prelude(qvx_device* dev, const qvx_geometry* geo, size_t heads, size_t s, float* q, float* k_new,
                         float* v_new, const qvx_prelude* prelude, void* stream) {
    if (!dev) return QVX_ERR_SHAPE;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    Layout L = make_layout(geo);
    if (!prelude_ok(prelude) || heads == 0 || heads % L.kvh != 0 || (L.d & 1u))
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: %zu tokens, %zu heads, %u KV heads of %u", s, heads,
                    L.kvh, L.d);
    return launch_attn_prelude(dev, L, heads, s, q, k_new, v_new, prelude, (cudaStream_t)stream);
}

int32_t qvx_block_copy_host(qvx_device* dev, qvx_buffer* pool, const qvx_geometry* geo, const uint32_t* src,
                            const uint32_t* dst, size_t n) {
    if (!dev) return QVX_ERR_SHAPE;
    std::lock_guard<std::mutex> lk(dev->mu);
    cudaSetDevice(dev->ordinal);
    int32_t rc = buffer_of(dev, pool);
    if (rc) return rc;
    if (!geometry_ok(geo)) return fail(dev, QVX_ERR_UNSUPPORTED, "cuda backend has no KV pool of this geometry");
    if (!pool->arena) return fail(dev, QVX_ERR_SHAPE, "shape mismatch in block copy: the KV pool is not an arena");
    Layout L = make_layout(geo);
    const size_t held = pool->len / L.block_bytes;
    std::unordered_set<uint32_t> dsts, srcs;
    for (size_t i = 0; i < n; i++) {
        if (src[i] >= held || dst[i] >= held)
            return fail(dev, QVX_ERR_SHAPE, "shape mismatch in block copy: a block past the pool's %zu", held);
        if (src[i] != dst[i]) { srcs.insert(src[i]); }
    }
    for (size_t i = 0; i < n; i++) {
        if (src[i] == dst[i]) continue;
        if (!dsts.insert(dst[i]).second || srcs.count(dst[i]))
            return fail(dev, QVX_ERR_SHAPE, "shape mismatch in block copy: block %u is written twice or also read", dst[i]);
    }
    if (n == 0) return QVX_OK;
    rc = wait_locked(dev);
    if (rc) return rc;
    uint32_t* d = nullptr;
    cudaError_t e = cudaMalloc((void**)&d, 8 * n);
    if (e != cudaSuccess) return check_cuda(dev, e, "block copy lists");
    e = cudaMemcpyAsync(d, src, 4 * n, cudaMemcpyHostToDevice, dev->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d + n, dst, 4 * n, cudaMemcpyHostToDevice, dev->stream);
    rc = e == cudaSuccess ? launch_block_copy(dev, L, pool->ptr, d, d + n, n, held, dev->stream) : check_cuda(dev, e, "block copy lists");
    cudaStreamSynchronize(dev->stream);
    cudaFree(d);
    dev->xfer.submissions++;
    dev->xfer.activations_in += 8 * n;
    return rc;
}

}  // extern "C"
