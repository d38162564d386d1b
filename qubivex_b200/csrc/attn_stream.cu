// Paged decode attention over native-layout pools (bf16, f16 on the tensor cores; f32 on the CUDA cores): a
// persistent, warp-specialised streaming kernel.
//
// Computes what `attn_decode.comp` (crates/qubivex-backend-vulkan/shaders/attn_decode.comp:60-175)
// and the gather + `attend` of the CPU device (crates/qubivex-backend-cpu/src/sim.rs:400-429,
// crates/qubivex-compute/src/math.rs:142-155) compute, with an online softmax and the context
// split into chunks: results agree within a tolerance, not bit for bit.
//
// The kernel is HBM bound (per position per kv head: 2*d*e bytes, 4*d*G flops), so it is
// organised around keeping bulk copies in flight, not around the arithmetic:
//
//   - CTAs are persistent.  Each takes work items (a chunk of one sequence for one kv head
//     and its group of <= 8 query heads) from a device-wide queue, longest first, until
//     the queue is empty; a CTA never waits for another CTA.
//   - The step's KV append can ride in the same launch: the producer warp of the CTA that takes
//     a sequence's last chunk stores the new key and value rows of its KV head first.
//   - One producer warp per CTA walks the queue one item ahead of its own copies: the next
//     item's index (an atomic) and record (header + block ids, one bulk copy) are in flight
//     while it issues the current item's tiles.  For every tile of 16 positions it issues bulk
//     async copies (cp.async.bulk global -> shared, completion counted on an mbarrier) of the
//     key rows and the value rows, contiguous in the native pool layout, into a ring of
//     stages shared by the CTA.  It runs ahead across item boundaries, so neither the
//     start-up nor the wind-down of an item drains the memory pipe.
//   - The consumer warps take the tiles in turn (tile n of the stream -> warp n mod CW), each
//     with its own online-softmax state: S^T = K Q^T for the tile (16 positions x 8 heads,
//     m16n8k16 with K as the A operand straight from the swizzled page), then
//     O^T += V^T P^T (V through ldmatrix.trans, P transposed in registers by movmatrix).
//     Every key and value byte is read from shared memory exactly once.  (f32 pools: the same warps, the same
//     tiles and states, the products on the CUDA cores, two per instruction; see WarpState32.)
//   - The consumer warps never wait for one another.  At the end of a chunk each leaves its state
//     (maxima, row sums, unnormalised outputs over the tiles it took) in one of two buffers in
//     shared memory, arrives on the buffer's mbarrier and goes on with the next chunk's tiles.
//   - An epilogue warp per CTA puts a chunk together: it merges the consumers' states in the order
//     of the tiles' places in the chunk and writes the output (a sequence in one chunk) or climbs
//     the merge tree of the sequence's chunks: an arrival takes a number from its node's
//     `claimed` word; every arrival but the node's last stores its entry and adds to `published`
//     (nothing waits for that); the last folds the node's entries in entry order -- the ones
//     before its own already while its chunk is still streaming, when they are all there -- and
//     writes the output or the next level's entry.  The only wait on another CTA is the bounded
//     one of a node's last arrival for entries already claimed.
//
// bf16 carries 8 mantissa bits: queries and probabilities go through the tensor cores as a
// 16-bit value plus a 16-bit remainder (two passes), which keeps the result within 1e-5 of the
// f32 arithmetic instead of 5e-3.  f16's 11 bits need one pass.
#include <stdio.h>

#include <vector>

#include "attn_ptx.cuh"

namespace qvx {

#ifndef QVX_CW
#define QVX_CW 4                               // consumer warps per CTA
#endif
constexpr int CW = QVX_CW;
constexpr int CT = CW * 32;                    // consumer threads
constexpr int STREAM_THREADS = CT + 64;        // + the producer warp and the epilogue warp
constexpr int MAIL_SLOTS = 2;                  // buffers of consumer states: one being merged, one being filled
constexpr int NOTE_SLOTS = 4;                  // items the epilogue warp is told about ahead of their states
constexpr int Q_SLOTS = 2;
constexpr int REC_SLOTS = 4;
#ifndef QVX_CLAIM_AHEAD
#define QVX_CLAIM_AHEAD 8
#endif
#ifndef QVX_FETCH_AHEAD
#define QVX_FETCH_AHEAD (QVX_CLAIM_AHEAD / 2)
#endif
#ifndef QVX_ISSUE_LANES
#define QVX_ISSUE_LANES 4
#endif
#ifndef QVX_BF16_PASSES
#define QVX_BF16_PASSES 3   // bf16 pools: 3 = queries and probabilities as value + remainder, 1 = the queries only
#endif
#ifndef QVX_PF_DIST
#define QVX_PF_DIST 0    // tiles the producer asks into the L2 ahead of the tile it copies into the ring (0: none)
#endif
constexpr uint32_t PF_DIST = QVX_PF_DIST;
#ifndef QVX_PREFETCH_TILES
#define QVX_PREFETCH_TILES 128   // tiles of a CTA's first item asked into the L2 while it waits for the launch before it (0: none)
#endif
constexpr uint32_t ISSUE_LANES = QVX_ISSUE_LANES;  // lanes of the producer warp that issue tiles side by side
constexpr uint32_t CLAIM_AHEAD = QVX_CLAIM_AHEAD;  // tiles before an item's end at which the producer claims the next item
constexpr uint32_t FETCH_AHEAD = QVX_FETCH_AHEAD;  // ... and at which it asks for the item's record
constexpr int REC_WORDS = 144;                 // header + up to 136 block ids

struct StreamArgs {
    const uint8_t* pool;
    const float* q;
    float* out;
    float* partials;        // per partial: acc[8][d], then CW copies of { m[8], l[8] }
    uint32_t* counters;     // per split (sequence, group): CW arrival counters, zero between launches
    uint32_t* queue;        // [0] next item, [1] CTAs done; both zero between launches
    const uint32_t* items;
    int* status;
    const float* k_new;     // the step's new rows, s x kv_out f32 each, stored by this launch; or null
    const float* v_new;
    uint64_t block_bytes;
    uint32_t page_bytes, tiles_per_block, heads, item_words, n_items, kv_out;
    uint32_t overlap;       // the pool and the tables do not depend on the work before this launch in the stream
    uint32_t trace_id;      // the launch's number (experiment builds that trace; otherwise unused)
    uint32_t test_hooks;    // test builds (-DQVX_TEST_HOOKS): 1 = lose one publication; otherwise unused
    float scale_log2;
};

// Programmatic dependent launch: `grid_dep_wait` returns once everything earlier in the stream
// has completed and is visible (at once when the launch did not ask for the overlap);
// `grid_dep_launch` lets the next launch in the stream start filling SMs this grid has left.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Per-CTA timestamps of the kernel's phases, for experiment builds (-DQVX_EXPERIMENTS -DQVX_TRACE): the host
// dumps the marks of the QVX_TRACE_AT-th launch (every launch without it) to the file QVX_TRACE_FILE names.
// Launches alternate between two buffers and tag their marks with their number, so a launch that overlaps
// its neighbours can be told from them.  In every other build a Tracer is empty and its marks cost nothing.
#if defined(QVX_EXPERIMENTS) && defined(QVX_TRACE)
#define QVX_TRACING 1
constexpr int TRACE_PER_CTA = 256;
__device__ unsigned long long g_trace[2][512 * TRACE_PER_CTA];
struct Tracer {
    uint32_t base, n = 0, id;
    bool on;
    __device__ __forceinline__ Tracer(uint32_t id, uint32_t quarter, bool on) : base(quarter * (TRACE_PER_CTA / 4)), id(id), on(on) {}
    __device__ __forceinline__ void mark(uint32_t tag) {
        if (!on || n >= TRACE_PER_CTA / 4) return;
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_trace[id & 1][blockIdx.x * TRACE_PER_CTA + base + n++] = (t << 12) | ((id & 15u) << 8) | tag;
    }
};
#else
#define QVX_TRACING 0
struct Tracer {
    __device__ __forceinline__ Tracer(uint32_t, uint32_t, bool) {}
    __device__ __forceinline__ void mark(uint32_t) {}
};
#endif

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// E: bytes per pool element (2: bf16 / f16, 4: f32).
template <int D, int E = 2>
struct StreamSmem {
    static constexpr int ctas_per_sm = (D <= 128 && CW <= 4) ? 2 : 1;
    static constexpr uint32_t budget = (227u * 1024u) / ctas_per_sm - 1024u;
    static constexpr uint32_t tile_bytes = TILE * D * E;
    static constexpr uint32_t stage_bytes = 2 * tile_bytes;
    static constexpr uint32_t q_stride = D * 4 + 16;  // padded rows: fragment reads hit 32 distinct banks
    // One warp's state: m[8], l[8], acc[8][D] with rows of D + 4 floats: the lanes that hold heads 2t
    // and positions g then store to 32 distinct banks.
    static constexpr uint32_t res_row = D + 4;
    static constexpr uint32_t res_floats = 16 + 8 * res_row;
    static constexpr uint32_t res_bytes = MAIL_SLOTS * CW * res_floats * 4;  // two items' worth: one being merged, one being filled
    static constexpr uint32_t q_bytes = Q_SLOTS * 8 * q_stride;
    static constexpr uint32_t rec_bytes = REC_SLOTS * REC_WORDS * 4;
    // f32 pools: the consumers' probabilities of a tile, [position][8 heads] of (p, p) pairs per warp
    static constexpr uint32_t ps_bytes = E == 4 ? CW * TILE * 8 * 8 : 0;
    // (+ the barriers, the notes and the last word; an f32 ring has at most 8 stages, and d = 128 only fits its four
    // 16 KB stages beside a second CTA with the smaller allowance)
    static constexpr uint32_t fixed = res_bytes + q_bytes + rec_bytes + ps_bytes + (E == 4 ? 512 : 1024);
    static constexpr uint32_t stages_fit = (budget - fixed) / stage_bytes;
    // A multiple of CW: tile n goes to stage n % stages and to warp n % CW, so a stage is
    // always read by the same warp and a warp waits for its stages' phases strictly in order
    // (waiting two phases ahead on an mbarrier parity would return at once).
    static constexpr uint32_t stages_most = (stages_fit > 4 * CW ? 4 * CW : stages_fit) / CW * CW;
#ifdef QVX_MAX_STAGES  // experiments: a shallower ring
    static constexpr uint32_t stages = stages_most < QVX_MAX_STAGES ? stages_most : QVX_MAX_STAGES;
#else
    static constexpr uint32_t stages = stages_most;
#endif
    static constexpr uint32_t ring_off = 0;
    static constexpr uint32_t res_off = stages * stage_bytes;
    static constexpr uint32_t q_off = res_off + res_bytes;
    static constexpr uint32_t rec_off = q_off + q_bytes;
    static constexpr uint32_t ps_off = rec_off + rec_bytes;
    static constexpr uint32_t bar_off = ps_off + ps_bytes;
    // full[stages], empty[stages], qfull[Q_SLOTS], qempty[Q_SLOTS], rec[REC_SLOTS],
    // res_full[MAIL_SLOTS], res_free[MAIL_SLOTS], note[NOTE_SLOTS], then the notes
    static constexpr uint32_t n_bars = 2 * stages + 2 * Q_SLOTS + REC_SLOTS + 2 * MAIL_SLOTS + NOTE_SLOTS;
    static constexpr uint32_t mail_off = (bar_off + n_bars * 8 + 15u) & ~15u;
    static constexpr uint32_t final_off = mail_off + NOTE_SLOTS * 32;  // chunks this CTA hands over in all, once its producer knows
    static constexpr uint32_t total = final_off + 16;
    static_assert(total <= budget, "the CTA's shared memory fits beside its neighbour's");
#if QVX_CW <= 4  // (experiment builds with more consumer warps only run the head sizes that fit)
    static_assert(stages >= CW, "the ring needs a stage per consumer warp");
#endif
};

// What the consumers tell the epilogue warp about an item when they start it, long before its
// states are ready.  `chunk` is the item's place among its sequence's chunks, NO_PART for a
// sequence in one piece; `stop` marks the end of the queue.
struct Mail {
    uint32_t seq, head0, nheads, part0, nch, counter, stop, chunk;
};

// The partial results of a split sequence are merged as a tree of fan-in MERGE_FAN: entry i of
// level k belongs to node i / MERGE_FAN (full nodes first, the remainder last: a sequence's last
// chunk, which usually arrives last, then finds little left to merge -- dealing the entries to nodes
// of equal size, QVX_MERGE_BALANCED, measured 1 % slower); the warp that delivers the last entry of a node merges
// the node's entries (in entry order) into one entry of level k + 1, or into the output when the
// level has at most MERGE_FAN entries.  The tree is a function of the chunk count alone, so the
// sum order is fixed; no merge reads more than MERGE_FAN entries, so the work left after a
// sequence's last chunk does not grow with its length.
#ifndef QVX_MERGE_FAN
#define QVX_MERGE_FAN 8
#endif
constexpr uint32_t MERGE_FAN = QVX_MERGE_FAN;

// Where entry `idx` of a level of `n` entries sits: its node, the node's first entry and size.
struct MergeNode {
    uint32_t node, first, size;
};
__host__ __device__ inline MergeNode merge_node_of(uint32_t idx, uint32_t n) {
#ifndef QVX_MERGE_BALANCED
    MergeNode p;
    p.node = idx / MERGE_FAN; p.first = p.node * MERGE_FAN; p.size = n - p.first < MERGE_FAN ? n - p.first : MERGE_FAN;
    return p;
#endif
    // (experiments) nodes of as equal a size as possible: 9 entries make nodes of 5 and 4, not of 8 and 1
    const uint32_t nodes = (n + MERGE_FAN - 1) / MERGE_FAN, base = n / nodes, extra = n % nodes;
    const uint32_t split = extra * (base + 1);  // the first `extra` nodes hold one entry more
    MergeNode m;
    if (idx < split) {
        m.node = idx / (base + 1); m.first = m.node * (base + 1); m.size = base + 1;
    } else {
        m.node = extra + (idx - split) / base; m.first = split + (m.node - extra) * base; m.size = base;
    }
    return m;
}

// Entries and counters one (sequence, group) of `nch` chunks needs, over all levels.
__host__ __device__ inline uint32_t merge_entries_total(uint32_t nch) {
    uint32_t total = nch, n = nch;
    while (n > MERGE_FAN) { n = (n + MERGE_FAN - 1) / MERGE_FAN; total += n; }
    return total;
}
// Two words per node: arrivals claimed, entries published.
__host__ __device__ inline uint32_t merge_counters_total(uint32_t nch) {
    uint32_t total = 0, n = nch;
    for (;;) {
        total += 2 * ((n + MERGE_FAN - 1) / MERGE_FAN);
        if (n <= MERGE_FAN) break;
        n = (n + MERGE_FAN - 1) / MERGE_FAN;
    }
    return total;
}

// Run by the epilogue warp with a chunk's merged result in registers (output i = lane + 32 j of
// the chunk's 8 x D/4 float4 values in E[j], the maximum and row sum of that output's head in
// Em[j], El[j]).  It counts the arrival at the chunk's node and climbs the tree as far as this
// arrival completes nodes.
//
// A node has two words.  An arrival first takes a number from `claimed`.  Every arrival but the
// last stores its entry, fences, and adds one to `published`: nothing waits for that.  The last
// arrival keeps its entry in registers, waits (bounded) until `published` shows the others, and
// merges the node: the others' entries from memory, its own from registers, in entry order.  So
// the chunk that finishes a sequence pays one atomic round trip and the loads, not a store, a
// fence, an atomic and the loads.  The merge keeps a running maximum, so an entry's maximum is
// needed only together with its values: no round of loads for the maxima first.
// A running merge over entries of a node: unnormalised outputs, running maxima and row sums
// (output i = lane + 32 j of the 8 x D/4 float4 values; the maximum and sum of that output's head).
template <int D>
struct Running {
    static constexpr int NJ = 8 * D / 4 / 32;
    float4 acc[NJ];
    float M[NJ], L[NJ];
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int j = 0; j < NJ; j++) { acc[j] = make_float4(0.f, 0.f, 0.f, 0.f); M[j] = -INFINITY; L[j] = 0.f; }
    }
};

// Folds entries c0 .. c1-1 of the node whose first entry is at p0 into `r`, in entry order.  Entry
// `mine` is not read from memory: it is E (values) and Eml (lane h < 8: maximum of head h, lane
// 8 + h: its row sum).  PAIR entries' loads are in flight at a time.
template <int D, int PAIR>
__device__ __forceinline__ void fold_range(Running<D>& r, const float* p0, uint32_t c0, uint32_t c1, uint32_t mine,
                                           const float4 (&E)[8 * D / 4 / 32], float Eml, uint32_t lane) {
    constexpr uint32_t PART_STRIDE = 8 * D + 16;
    constexpr int NJ = 8 * D / 4 / 32;
    for (uint32_t c = c0; c < c1; c += PAIR) {
        float4 v[PAIR][NJ];
        float ml[PAIR];
#pragma unroll
        for (int u = 0; u < PAIR; u++) {
            const float* pe = p0 + (size_t)(c + u) * PART_STRIDE;
            const bool load = c + u < c1 && c + u != mine;
            ml[u] = Eml;
            if (load && lane < 16) ml[u] = __ldcg(pe + 8 * D + lane);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const uint32_t i = lane + j * 32, h = i / (D / 4);
                v[u][j] = load ? __ldcg(reinterpret_cast<const float4*>(pe + h * D + (i % (D / 4)) * 4)) : E[j];
            }
        }
#pragma unroll
        for (int u = 0; u < PAIR; u++) {
            if (c + u >= c1) break;
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const uint32_t h = (lane + j * 32) / (D / 4);
                const float m = __shfl_sync(0xffffffffu, ml[u], h), l = __shfl_sync(0xffffffffu, ml[u], 8 + h);
                const float mn = fmaxf(r.M[j], m);
                const float so = ex2(r.M[j] - mn), w = ex2(m - mn);
                r.acc[j].x = fmaf(v[u][j].x, w, r.acc[j].x * so); r.acc[j].y = fmaf(v[u][j].y, w, r.acc[j].y * so);
                r.acc[j].z = fmaf(v[u][j].z, w, r.acc[j].z * so); r.acc[j].w = fmaf(v[u][j].w, w, r.acc[j].w * so);
                r.L[j] = fmaf(l, w, r.L[j] * so);
                r.M[j] = mn;
            }
        }
    }
}

// The same fold with every entry's loads in flight at once: the entries are first copied into shared memory
// at `stage` (cp.async: no register holds them meanwhile), then folded from there, in entry order.  One round
// trip to the L2 instead of one per PAIR entries.  `stage` must hold (c1 - c0) entries of 8 * D + 16 floats
// and be nobody else's: the epilogue warp uses the CTA's ring for it once the CTA has streamed its last tile.
template <int D>
__device__ __forceinline__ void fold_range_staged(Running<D>& r, const float* p0, uint32_t c0, uint32_t c1, uint32_t mine,
                                                  const float4 (&E)[8 * D / 4 / 32], float Eml, uint32_t lane,
                                                  uint8_t* stage_ptr, uint32_t stage) {
    constexpr uint32_t PART_STRIDE = 8 * D + 16;
    constexpr uint32_t PIECES = PART_STRIDE / 4;  // 16-byte pieces of an entry
    constexpr int NJ = 8 * D / 4 / 32;
    for (uint32_t c = c0; c < c1; c++) {
        if (c == mine) continue;
        const float* pe = p0 + (size_t)c * PART_STRIDE;
        const uint32_t dst = stage + (c - c0) * PART_STRIDE * 4;
        for (uint32_t i = lane; i < PIECES; i += 32) cp_async_16(dst + i * 16, pe + i * 4);
    }
    cp_async_wait_all();
    __syncwarp();
    for (uint32_t c = c0; c < c1; c++) {
        const float* se = reinterpret_cast<const float*>(stage_ptr) + (size_t)(c - c0) * PART_STRIDE;
        float ml = Eml;
        if (c != mine && lane < 16) ml = se[8 * D + lane];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const uint32_t i = lane + j * 32, h = i / (D / 4);
            const float4 v = c != mine ? *reinterpret_cast<const float4*>(se + h * D + (i % (D / 4)) * 4) : E[j];
            const float m = __shfl_sync(0xffffffffu, ml, h), l = __shfl_sync(0xffffffffu, ml, 8 + h);
            const float mn = fmaxf(r.M[j], m);
            const float so = ex2(r.M[j] - mn), w = ex2(m - mn);
            r.acc[j].x = fmaf(v.x, w, r.acc[j].x * so); r.acc[j].y = fmaf(v.y, w, r.acc[j].y * so);
            r.acc[j].z = fmaf(v.z, w, r.acc[j].z * so); r.acc[j].w = fmaf(v.w, w, r.acc[j].w * so);
            r.L[j] = fmaf(l, w, r.L[j] * so);
            r.M[j] = mn;
        }
    }
}

// Release / acquire fences at device scope (__threadfence() is the sequentially consistent one).
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// Waits (bounded) until a node's `published` word shows `want` entries.
__device__ __forceinline__ bool wait_published(const uint32_t* published, uint32_t want) {
    bool seen = false;
    for (uint32_t i = 0; i < WAIT_LIMIT && !seen; i++) {
        seen = *reinterpret_cast<const volatile uint32_t*>(published) == want;
        if (!seen && i > 64) __nanosleep(32);
    }
    return __all_sync(0xffffffffu, seen);
}

// Run by the epilogue warp when it learns of a split item, while the consumers are still
// streaming it.  If every other chunk of the item's node has already arrived, this item is the
// node's last arrival for certain, and the entries before it can be folded now: when the item's
// own result is ready only that (and the entries after it, if any) remain.  Returns whether
// `r` holds that prefix.
enum : uint32_t { FOLD_NOT_YET = 0, FOLD_DONE = 1, FOLD_GAVE_UP = 2 };
template <int D>
__device__ __forceinline__ uint32_t fold_ahead(const StreamArgs& a, const Mail& it, uint32_t lane, Running<D>& r) {
    constexpr uint32_t PART_STRIDE = 8 * D + 16;
    const MergeNode mn = merge_node_of(it.chunk, it.nch);
    const uint32_t node = mn.node, first = mn.first, size = mn.size, mine = it.chunk - first;
    if (size < 2) return FOLD_GAVE_UP;  // nothing to fold, now or later
    const uint32_t* claimed = a.counters + it.counter + 2 * node;
    // Both words in one round trip: lane 0 reads `claimed`, lane 1 `published`.
    uint32_t word = 0;
    if (lane < 2) word = *reinterpret_cast<const volatile uint32_t*>(claimed + lane);
    if (__shfl_sync(0xffffffffu, word, 0) != size - 1) return FOLD_NOT_YET;
    if (__shfl_sync(0xffffffffu, word, 1) != size - 1 && !wait_published(claimed + 1, size - 1))
        return FOLD_GAVE_UP;  // a bounded wait ran out: no second try; the arrival's own wait reports it
    fence_acq_rel_gpu();
    r.clear();
    float4 none[8 * D / 4 / 32];
#pragma unroll
    for (int j = 0; j < 8 * D / 4 / 32; j++) none[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    fold_range<D, (8 * D / 4 / 32 <= 8 ? 3 : 1)>(r, a.partials + (size_t)(it.part0 + first) * PART_STRIDE, 0, mine, NO_PART, none, 0.f, lane);
    return FOLD_DONE;
}

// Run by the epilogue warp with a chunk's merged result in registers (E, Eml as in fold_range).
// It counts the arrival at the chunk's node and climbs the tree as far as this arrival completes
// nodes.
//
// A node has two words.  An arrival first takes a number from `claimed`.  Every arrival but the
// last stores its entry, fences, and adds one to `published`: nothing waits for that.  The last
// arrival keeps its entry in registers, waits (bounded) until `published` shows the others, and
// merges the node: the others' entries from memory, its own from registers, in entry order.  So
// the chunk that finishes a sequence pays one atomic round trip and the loads, not a store, a
// fence, an atomic and the loads -- and with `ahead` (fold_ahead succeeded) not even those.  The
// merge keeps a running maximum, so an entry's maximum is needed only together with its values.
template <int D>
__device__ __forceinline__ void climb(const StreamArgs& a, const Mail& it, uint32_t lane, float4 (&E)[8 * D / 4 / 32], float Eml,
                                      bool ahead, Running<D>& r, Tracer& tr, bool ring_free, uint8_t* stage_ptr, uint32_t stage) {
    constexpr uint32_t PART_STRIDE = 8 * D + 16;
    constexpr int NJ = 8 * D / 4 / 32;
    uint32_t hh[NJ], off[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const uint32_t i = lane + j * 32;
        hh[j] = i / (D / 4);
        off[j] = hh[j] * D + (i % (D / 4)) * 4;
    }
    uint32_t n = it.nch, idx = it.chunk, part_base = it.part0, cnt_base = it.counter;
    for (;;) {
        const MergeNode mn = merge_node_of(idx, n);
        const uint32_t node = mn.node, first = mn.first, size = mn.size, mine = idx - first;
        uint32_t* claimed = a.counters + cnt_base + 2 * node;
        uint32_t* published = claimed + 1;
        float* p0 = a.partials + (size_t)(part_base + first) * PART_STRIDE;
        if (!ahead) {
            uint32_t ticket = 0;
            if (lane == 0) ticket = atomicAdd(claimed, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            const bool last = ticket == size - 1;
            tr.mark(last ? 14 : 17);  // claim answered
            if (!last) {
                float* pe = p0 + (size_t)mine * PART_STRIDE;
                const uint64_t keep = l2_policy_evict_last();  // read again by the node's last arrival: stay in the L2
#pragma unroll
                for (int j = 0; j < NJ; j++) st_global_hint(reinterpret_cast<float4*>(pe + off[j]), E[j], keep);
                if (lane < 16) pe[8 * D + lane] = Eml;
                fence_acq_rel_gpu();
                __syncwarp();
#ifdef QVX_TEST_HOOKS
                // A test build can lose one publication (sequence 0's first group, the first arrival at its node): the node's last
                // arrival must then give up its bounded wait, report it, and leave the device usable.
                if (a.test_hooks == 1u && it.seq == 0 && it.head0 == 0 && ticket == 0 && n == it.nch) return;
#endif
                if (lane == 0) atomicAdd(published, 1u);
                return;
            }
            // The last arrival: the others have claimed before it, and publish within a store and a fence.
            if (!wait_published(published, size - 1)) {
                if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
                return;
            }
            tr.mark(15);  // the others' entries are published
            fence_acq_rel_gpu();
            r.clear();
        }
        if (lane == 0) { *claimed = 0; *published = 0; }  // ready for the next launch
        // `ring_free`: the CTA has streamed its last tile and its ring (at `stage`) is free to stage the entries in.
        if (ring_free && !ahead && size * PART_STRIDE * 4 <= StreamSmem<D>::stages * StreamSmem<D>::stage_bytes) {
            tr.mark(26);  // staged fold begins
            fold_range_staged<D>(r, p0, 0u, size, mine, E, Eml, lane, stage_ptr, stage);
        } else {
            tr.mark(27);  // fold from registers begins
            fold_range<D, (NJ <= 8 ? 2 : 1)>(r, p0, ahead ? mine : 0u, size, mine, E, Eml, lane);
        }
        ahead = false;
        tr.mark(16);  // node merged
        if (n <= MERGE_FAN) {
            // The root: the sequence's output.
#pragma unroll
            for (int j = 0; j < NJ; j++)
                if (hh[j] < it.nheads) {
                    const float inv = 1.0f / r.L[j];
                    *reinterpret_cast<float4*>(a.out + ((size_t)it.seq * a.heads + it.head0) * D + off[j]) =
                        make_float4(r.acc[j].x * inv, r.acc[j].y * inv, r.acc[j].z * inv, r.acc[j].w * inv);
                }
            return;
        }
        // The node's result is this warp's entry of the next level.
#pragma unroll
        for (int j = 0; j < NJ; j++) E[j] = r.acc[j];
#pragma unroll
        for (int h = 0; h < 8; h++) {
            // Head h's first output, h * D/4, is held by lane (h * D/4) % 32 at j = (h * D/4) / 32.
            constexpr int Q = D / 4;
            const float mv = __shfl_sync(0xffffffffu, r.M[(h * Q) / 32], (h * Q) % 32);
            const float lv = __shfl_sync(0xffffffffu, r.L[(h * Q) / 32], (h * Q) % 32);
            if (lane == (uint32_t)h) Eml = mv;
            if (lane == (uint32_t)(8 + h)) Eml = lv;
        }
        cnt_base += 2 * ((n + MERGE_FAN - 1) / MERGE_FAN);
        part_base += n;
        n = (n + MERGE_FAN - 1) / MERGE_FAN;
        idx = node;
    }
}

// ---- what a consumer warp carries through a chunk ---------------------------------------------------------
// Two forms with one interface: begin_item (the group's queries), begin_chunk, tile, store (the warp's state into
// the hand-over buffer: m[8], l[8], then acc[8][res_row]).  `queries_in_registers`: the query slot is free as soon
// as begin_item returns; otherwise the warp reads it until the item's last tile.
template <int DT, int D, int PASSES>
struct WarpState16 {   // bf16 / f16 pools: tensor cores (attend_tile)
    static constexpr bool queries_in_registers = true;
    uint32_t qf[D / 16][2], ql[D / 16][2];
    float o[D / 16][4];
    float m0, m1, l0, l1;  // heads 2t and 2t+1
    __device__ __forceinline__ void begin_item(const uint8_t* qslot, uint32_t q_stride, uint32_t nheads, uint32_t lane, uint8_t*) {
        // Q^T fragments (the B operand), once per item: this lane holds head g, dims 16*ks + 2t + {0,1,8,9}.
        const uint32_t g = lane >> 2, t = lane & 3;
        const bool live = g < nheads;
        const float* qrow = reinterpret_cast<const float*>(qslot + g * q_stride);
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            float2 x0 = make_float2(0.f, 0.f), x1 = x0;
            if (live) {
                x0 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 2 * t);
                x1 = *reinterpret_cast<const float2*>(qrow + 16 * ks + 2 * t + 8);
            }
            split16<DT>(x0.x, x0.y, qf[ks][0], ql[ks][0]);
            split16<DT>(x1.x, x1.y, qf[ks][1], ql[ks][1]);
        }
    }
    __device__ __forceinline__ void begin_chunk() {
#pragma unroll
        for (int m = 0; m < D / 16; m++) { o[m][0] = o[m][1] = o[m][2] = o[m][3] = 0.f; }
        m0 = m1 = -INFINITY; l0 = l1 = 0.f;
    }
    __device__ __forceinline__ void tile(uint32_t kt, uint32_t vt, uint8_t*, uint8_t* vt_rows, uint32_t valid, uint32_t lane, float scale_log2) {
        attend_tile<DT, D, PASSES>(kt, vt, vt_rows, valid, lane, qf, ql, scale_log2, o, m0, m1, l0, l1);
    }
    __device__ __forceinline__ void store(float* res, uint32_t res_row, uint32_t lane) {
        const uint32_t g = lane >> 2, t = lane & 3;
        // Row sums over the positions held by the other lanes of the same t.
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
            l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
        }
        if (g == 0) {
            res[2 * t] = m0; res[2 * t + 1] = m1;
            res[8 + 2 * t] = l0; res[8 + 2 * t + 1] = l1;
        }
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            res[16 + (2 * t) * res_row + 16 * mt + g] = o[mt][0];
            res[16 + (2 * t + 1) * res_row + 16 * mt + g] = o[mt][1];
            res[16 + (2 * t) * res_row + 16 * mt + g + 8] = o[mt][2];
            res[16 + (2 * t + 1) * res_row + 16 * mt + g + 8] = o[mt][3];
        }
    }
};

// f32 pools: CUDA cores.  Scores: lane = (position = lane & 15, half = lane >> 4) computes heads half, half + 2, ...
// of the group's NH; values: lane owns output dims 2 lane, 2 lane + 1 (+ 64) of all NH heads.  The multiply-adds go
// out two at a time (fma.rn.f32x2): a score is summed as an even and an odd half.  The queries stay in their shared-
// memory slot for the whole item; `ps` holds the tile's probabilities as (p, p) pairs between the two phases.
// Every pair lives in one 64-bit register from its load to its last use (P2): taken apart and put together again
// around each instruction, a pair costs two moves per multiply-add.
using P2 = unsigned long long;
__device__ __forceinline__ P2 fma2(P2 a, P2 b, P2 c) {
    P2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ P2 mul2(P2 a, P2 b) {
    P2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ P2 pair_of(float x, float y) {
    P2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(x), "f"(y));
    return d;
}
__device__ __forceinline__ float2 floats_of(P2 p) {
    float2 v;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ void lds_pairs(uint32_t addr, P2& a, P2& b) {   // 16 bytes: two pairs
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(addr));
}
__device__ __forceinline__ P2 lds_pair(uint32_t addr) {
    P2 a;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(a) : "r"(addr));
    return a;
}
__device__ __forceinline__ void sts_pair(uint32_t addr, P2 v) { asm volatile("st.shared.b64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }

template <int D, int NH>
struct WarpState32 {
    static constexpr bool queries_in_registers = false;
    static constexpr int NJ = NH / 2, DK = D / 64;
    uint32_t q;         // shared address of [8] rows of q_stride bytes; rows past the group's heads hold anything
    uint32_t q_stride, nheads;
    uint32_t ps;        // shared address of this warp's [16 positions][8 heads] (p, p) pairs
    float m[NH], lpart[NJ];
    P2 o[NH][DK];
    __device__ __forceinline__ void begin_item(const uint8_t* qslot, uint32_t stride, uint32_t nh, uint32_t, uint8_t* ps_warp) {
        q = smem_u32(qslot); q_stride = stride; nheads = nh;
        ps = smem_u32(ps_warp);
    }
    __device__ __forceinline__ void begin_chunk() {
#pragma unroll
        for (int h = 0; h < NH; h++) {
            m[h] = -INFINITY;
#pragma unroll
            for (int k = 0; k < DK; k++) o[h][k] = 0ull;   // (0.f, 0.f)
        }
#pragma unroll
        for (int j = 0; j < NJ; j++) lpart[j] = 0.f;
    }
    __device__ __forceinline__ void tile(uint32_t kt, uint32_t vt, uint8_t*, uint8_t*, uint32_t valid, uint32_t lane, float scale_log2) {
        const uint32_t tok = lane & 15, half = lane >> 4;
        P2 s2[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) s2[j] = 0ull;
        const uint32_t krow = kt + tok * (D * 4), qrow = q + half * q_stride, sw = (tok & 7) << 4;
#pragma unroll 8
        for (int c = 0; c < D / 4; c++) {
            P2 k01, k23;
            lds_pairs(krow + ((c << 4) ^ sw), k01, k23);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                P2 q01, q23;
                lds_pairs(qrow + 2 * j * q_stride + 16 * c, q01, q23);
                s2[j] = fma2(q01, k01, s2[j]);
                s2[j] = fma2(q23, k23, s2[j]);
            }
        }
        float s[NJ];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            // (a head past the group's: its query row is whatever the slot held; its scores are made harmless)
            const float2 two = floats_of(s2[j]);
            s[j] = (half + 2 * j < nheads && tok < valid) ? (two.x + two.y) * scale_log2 : -INFINITY;
        }
        // Tile maximum per head over the 16 positions, then across the two halves.
        float mx[NH];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            float v = s[j];
#pragma unroll
            for (int sh = 1; sh <= 8; sh <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, sh));
            const float other = __shfl_xor_sync(0xffffffffu, v, 16);
            mx[2 * j] = half == 0 ? v : other;       // head half + 2j is mine, head (1 - half) + 2j the other half's
            mx[2 * j + 1] = half == 0 ? other : v;
        }
        float al[NH];
        bool moved = false;
#pragma unroll
        for (int h = 0; h < NH; h++) {
            const float mn = fmaxf(m[h], mx[h]);
            // (a head with no valid score yet keeps -inf; exp2(-inf - -inf) would be NaN)
            al[h] = mn == -INFINITY ? 1.0f : ex2(m[h] - mn);
            moved = moved || al[h] != 1.0f;
            m[h] = mn;
        }
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const float mine = half == 0 ? m[2 * j] : m[2 * j + 1];
            const float al_mine = half == 0 ? al[2 * j] : al[2 * j + 1];
            const float pr = s[j] == -INFINITY ? 0.0f : ex2(s[j] - mine);
            lpart[j] = fmaf(lpart[j], al_mine, pr);
            sts_pair(ps + (tok * 8 + half + 2 * j) * 8, pair_of(pr, pr));
        }
        __syncwarp();
        if (moved) {   // (the maxima settle after a chunk's first tiles: x * 1.0f is x, so skipping changes no bit)
#pragma unroll
            for (int h = 0; h < NH; h++) {
                const P2 a2 = pair_of(al[h], al[h]);
#pragma unroll
                for (int k = 0; k < DK; k++) o[h][k] = mul2(o[h][k], a2);
            }
        }
        // This lane's dims 2 lane, 2 lane + 1 (+ 64 k) of a value row: one 8-byte load in the row's swizzled chunk.
        const uint32_t vlane = lane << 3;   // byte offset of the pair in an unswizzled row: chunk lane >> 1, half lane & 1
        auto accumulate = [&](uint32_t p) {
            P2 pv[NH];
#pragma unroll
            for (int h = 0; h < NH; h += 2) lds_pairs(ps + (p * 8 + h) * 8, pv[h], pv[h + 1]);
#pragma unroll
            for (int k = 0; k < DK; k++) {
                // (chunk (lane >> 1) + 16 k of the row, swizzled by the row's place; the lane's half of the chunk)
                const P2 v = lds_pair(vt + p * (D * 4) + 256u * k + (vlane ^ ((p & 7) << 4)));
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
        __syncwarp();  // the probabilities are read: the next tile may overwrite them
    }
    __device__ __forceinline__ void store(float* res, uint32_t res_row, uint32_t lane) {
        const uint32_t half = lane >> 4;
        // Row sums: over the 16 positions, then hand each half's heads to the other.
        float l[NH];
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            float v = lpart[j];
#pragma unroll
            for (int sh = 1; sh <= 8; sh <<= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
            const float other = __shfl_xor_sync(0xffffffffu, v, 16);
            l[2 * j] = half == 0 ? v : other;
            l[2 * j + 1] = half == 0 ? other : v;
        }
        if (lane < 8) {   // heads past NH: no weight in any merge
            float mv = -INFINITY, lv = 0.f;
#pragma unroll
            for (int h = 0; h < NH; h++)
                if (lane == (uint32_t)h) { mv = m[h]; lv = l[h]; }
            res[lane] = mv; res[8 + lane] = lv;
        }
#pragma unroll
        for (int h = 0; h < NH; h++) {
#pragma unroll
            for (int k = 0; k < DK; k++) *reinterpret_cast<float2*>(res + 16 + h * res_row + 2 * lane + 64 * k) = floats_of(o[h][k]);
        }
    }
};
template <int DT, int D, int VAR> struct WarpStateOf { using type = WarpState16<DT, D, VAR>; };
template <int D, int VAR> struct WarpStateOf<QVX_F32, D, VAR> { using type = WarpState32<D, VAR>; };

// VAR: for bf16 / f16 pools, which operands go through the tensor cores as value + remainder (bit 0: the queries,
// bit 1: the probabilities); for f32 pools, the query heads of a group the arithmetic is unrolled for (2, 4 or 8).
template <int DT, int D, int VAR>
__global__ void __launch_bounds__(STREAM_THREADS, StreamSmem<D, (DT == QVX_F32 ? 4 : 2)>::ctas_per_sm) attn_stream_kernel(StreamArgs a) {
    constexpr int E = DT == QVX_F32 ? 4 : 2;
    using SM = StreamSmem<D, E>;
    using WS = typename WarpStateOf<DT, D, VAR>::type;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t full0 = sbase + SM::bar_off, empty0 = full0 + SM::stages * 8;
    const uint32_t qfull0 = empty0 + SM::stages * 8, qempty0 = qfull0 + Q_SLOTS * 8, recbar0 = qempty0 + Q_SLOTS * 8;
    const uint32_t rfull0 = recbar0 + REC_SLOTS * 8, rfree0 = rfull0 + MAIL_SLOTS * 8, note0 = rfree0 + MAIL_SLOTS * 8;
    volatile Mail* mailbox = reinterpret_cast<volatile Mail*>(smem + SM::mail_off);
    volatile uint32_t* final_chunks = reinterpret_cast<volatile uint32_t*>(smem + SM::final_off);

    if (threadIdx.x == 0) grid_dep_launch();
    // Without the caller's word that the pool is settled, nothing is touched before the stream's
    // earlier work is done.  With it, only what that work produces (q, k_new, v_new) and what
    // this grid writes wait for it; the old positions' tiles start streaming right away.
    if (!a.overlap) grid_dep_wait();
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < SM::stages; s++) { mbar_init(full0 + s * 8, 1); mbar_init(empty0 + s * 8, 1); }
        for (uint32_t s = 0; s < Q_SLOTS; s++) { mbar_init(qfull0 + s * 8, 1); mbar_init(qempty0 + s * 8, CW); }
        for (uint32_t s = 0; s < REC_SLOTS; s++) mbar_init(recbar0 + s * 8, 1);
        for (uint32_t s = 0; s < MAIL_SLOTS; s++) { mbar_init(rfull0 + s * 8, CW); mbar_init(rfree0 + s * 8, 1); }
        for (uint32_t s = 0; s < NOTE_SLOTS; s++) mbar_init(note0 + s * 8, 1);
        *final_chunks = NO_PART;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (warp == CW) {
        // ================================ producer ================================
        // Lane 0 walks the queue and issues every copy; the whole warp meets once per item, to
        // store the sequence's new key and value rows when the item holds its last position.
        uint32_t* rec_base = reinterpret_cast<uint32_t*>(smem + SM::rec_off);
        const uint32_t rec_bytes_one = a.item_words * 4;
        // Fetches item `idx` into record slot j % REC_SLOTS (or writes the end-of-queue record).
        auto fetch = [&](uint32_t j, uint32_t idx) {
            const uint32_t slot = j % REC_SLOTS;
            if (idx < a.n_items) {
                mbar_expect_tx(recbar0 + slot * 8, rec_bytes_one);
                bulk_g2s(sbase + SM::rec_off + slot * REC_WORDS * 4, a.items + (size_t)idx * a.item_words, rec_bytes_one,
                         recbar0 + slot * 8);
            } else {
                rec_base[slot * REC_WORDS + 1] = 0;  // an item of no positions: the end of the queue
                mbar_arrive(recbar0 + slot * 8);
            }
        };
        // What one lane pays per tile -- an mbarrier wait, an expect-tx, the bulk copy, each a round
        // through the shared-memory pipe -- is about 0.3 us, close to the 0.34 us a tile takes at the
        // memory's rate: one lane alone can barely keep the ring full and never catches up after a
        // pause.  So ISSUE_LANES lanes issue consecutive tiles in step (one instruction stream, a tile
        // each); everything per tile is derived with shifts and constants, nothing with a division.
        uint32_t nprod = 0;  // tiles issued before the current item, over all items
        uint32_t nchunks = 0;  // chunks of the items up to the current one, over all items
        const bool one_copy = a.page_bytes == SM::tile_bytes;  // one tile per block: its values follow its keys
        const uint32_t tpb = a.tiles_per_block;
        const bool tpb_pow2 = (tpb & (tpb - 1u)) == 0u;
        const uint32_t tpb_shift = 31u - (uint32_t)__clz((int)tpb);
        // Every KV byte is read once per launch: its lines leave the L2 first, so that what the launch
        // keeps coming back to (partial results, records, queries) stays there.
        const uint64_t stream_policy = l2_policy_evict_first();
        bool failed = false, queue_dry = false;
        Tracer tr(a.trace_id, 0, lane == 0);
        tr.mark(1);  // producer start
        // The first item needs no atomic: CTA b starts with item b, the queue hands out the rest.
        if (lane == 0) fetch(0, blockIdx.x);
        for (uint32_t k = 0;; k++) {
            const uint32_t rslot = k % REC_SLOTS, qslot = k % Q_SLOTS;
            // The consumers are done with the queries of item k - Q_SLOTS (and so with every
            // record before it).
            bool ok = mbar_wait(recbar0 + rslot * 8, (k / REC_SLOTS) & 1);
            ok = ok && mbar_wait(qempty0 + qslot * 8, ((k / Q_SLOTS) & 1) ^ 1);
            if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
            tr.mark(5);  // record and query slot ready
            const uint32_t* rec = rec_base + rslot * REC_WORDS;
            const uint32_t seq = rec[0], tokens = rec[1], head0 = rec[2], nheads = rec[3] & 0xffffu, kvh = rec[3] >> 16;
            if (tokens == 0) {
                if (lane == 0) mbar_arrive(qfull0 + qslot * 8);  // hand the end-of-queue record to the consumers
                break;
            }
            const uint8_t* base = a.pool + (uint64_t)kvh * 2u * a.page_bytes;
            const uint32_t ntiles = (tokens + TILE - 1) / TILE;
            nchunks += rec[9];
            const uint32_t* ids = rec + QVX_ITEM_HEADER_WORDS;
            auto issue_tile = [&](uint32_t tau) -> bool {  // any lane: tile `tau` of this item
                const uint32_t n = nprod + tau;
                const uint32_t st = n % SM::stages, parity = ((n / SM::stages) & 1u) ^ 1u;
                const uint32_t eb = empty0 + st * 8, fb = full0 + st * 8;
                if (!mbar_try_wait(eb, parity) && !mbar_wait(eb, parity)) return false;
                const uint32_t bi = tpb_pow2 ? tau >> tpb_shift : tau / tpb, bj = tau - bi * tpb;
                const uint8_t* src = base + (uint64_t)ids[bi] * a.block_bytes + bj * SM::tile_bytes;
                const uint32_t dst = sbase + SM::ring_off + st * SM::stage_bytes;
                mbar_expect_tx(fb, SM::stage_bytes);
                if (one_copy) {
                    bulk_g2s_hint(dst, src, SM::stage_bytes, fb, stream_policy);
                } else {
                    bulk_g2s_hint(dst, src, SM::tile_bytes, fb, stream_policy);
                    bulk_g2s_hint(dst + SM::tile_bytes, src + a.page_bytes, SM::tile_bytes, fb, stream_policy);
                }
                return true;
            };
            // Asks the L2 for tile `tau` of this item; nothing waits for it.  The ring holds only what fits the shared
            // memory, and half of it is being multiplied at any time: run ahead of it in the L2, where there is room,
            // so that the device memory sees requests PF_DIST tiles deep and the ring only has to cover the L2's latency.
            auto prefetch_tile = [&](uint32_t tau) {
                const uint32_t bi = tpb_pow2 ? tau >> tpb_shift : tau / tpb, bj = tau - bi * tpb;
                const uint8_t* src = base + (uint64_t)ids[bi] * a.block_bytes + bj * SM::tile_bytes;
                if (one_copy) {
                    bulk_prefetch_l2(src, SM::stage_bytes);
                } else {
                    bulk_prefetch_l2(src, SM::tile_bytes);
                    bulk_prefetch_l2(src + a.page_bytes, SM::tile_bytes);
                }
            };
            const bool last_chunk = rec[4] == NO_PART || rec[4] - rec[5] + rec[9] == rec[6];  // the run ends the sequence
            uint32_t tau0 = 0;
            if (PF_DIST > 0 && !(k == 0 && a.overlap)) {  // the item's head, a tile per lane (the first item of an overlapped launch: below)
                const uint32_t upto = ntiles < PF_DIST ? ntiles : PF_DIST;
                for (uint32_t tau = lane; tau < upto; tau += 32) prefetch_tile(tau);
            }
            if (k == 0 && a.overlap) {
                // The first item's old positions stream while the stream's earlier work finishes;
                // a chunk that holds the step's new row waits, since its rows come from that work.
                if (!(last_chunk && a.k_new != nullptr)) {
                    tau0 = ntiles < SM::stages ? ntiles : SM::stages;
                    if (lane < ISSUE_LANES)
                        for (uint32_t tau = lane; tau < tau0; tau += ISSUE_LANES)
                            if (!issue_tile(tau)) { failed = true; break; }
                }
#if QVX_PREFETCH_TILES > 0
                // The ring is full and nothing more can be asked for until the queries exist; the memory the
                // draining launch before this one no longer uses is idle meanwhile.  The rest of this first
                // item is asked into the L2 now (one request per tile and lane; nothing waits for them), so
                // that its copies find it there once the launch proper begins.
                {
                    const uint32_t upto = ntiles < tau0 + QVX_PREFETCH_TILES ? ntiles : tau0 + QVX_PREFETCH_TILES;
                    for (uint32_t tau = tau0 + lane; tau < upto; tau += 32) prefetch_tile(tau);
                }
#endif
                grid_dep_wait();
            }
            if (a.k_new != nullptr) {
                // KV append fused in: the chunk that ends the sequence holds the position the step
                // adds.  Its rows go into the pool now, long before the tile that reads them is
                // asked for (sim.rs:394-398: the new row is stored, then attention reads 0..=pos).
                if (last_chunk) {
                    const uint32_t p = tokens - 1, B = a.tiles_per_block * TILE, slot = p % B;
                    const uint32_t blk = rec[QVX_ITEM_HEADER_WORDS + p / B];
                    uint8_t* row = const_cast<uint8_t*>(base) + (uint64_t)blk * a.block_bytes + (uint64_t)slot * (D * E);
                    constexpr uint32_t CPR = D * E / 16;  // 16-byte chunks per row
                    for (uint32_t i = lane; i < 2 * CPR; i += 32) {
                        const uint32_t kv = i / CPR, c = i % CPR;
                        const float* src = (kv ? a.v_new : a.k_new) + (size_t)seq * a.kv_out + kvh * D + c * (16 / E);
                        uint4 w;
                        if constexpr (E == 4) {
                            w = *reinterpret_cast<const uint4*>(src);
                        } else {
                            const float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
                            w.x = narrow16x2(lo.x, lo.y, DT);
                            w.y = narrow16x2(lo.z, lo.w, DT);
                            w.z = narrow16x2(hi.x, hi.y, DT);
                            w.w = narrow16x2(hi.z, hi.w, DT);
                        }
                        *reinterpret_cast<uint4*>(row + (uint64_t)kv * a.page_bytes + ((c ^ (slot & 7u)) << 4)) = w;
                    }
                    __threadfence();  // the rows are in device memory ...
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // ... before any bulk copy reads them
                }
                __syncwarp();
            }
            // The group's query rows, one copy each, issued side by side by the first lanes.
            if (lane == 0) mbar_expect_tx(qfull0 + qslot * 8, nheads * D * 4);
            __syncwarp();
            if (lane < nheads) {
                asm volatile("fence.proxy.async.global;" ::: "memory");
                bulk_g2s(sbase + SM::q_off + (qslot * 8 + lane) * SM::q_stride, a.q + ((size_t)seq * a.heads + head0 + lane) * D, D * 4,
                         qfull0 + qslot * 8);
            }
            if (lane < ISSUE_LANES) {
                tr.mark(2);  // item issue begins
                // Item k + 1 is claimed late: CLAIM_AHEAD tiles before this item's last tile is
                // asked for, which is about the time its index and then its record take to come
                // back.  A CTA so never sits on work that an idle CTA could take: the launch ends
                // within a few tiles' time of the queue running dry.
                uint32_t claim_at = ntiles > CLAIM_AHEAD ? ntiles - CLAIM_AHEAD : 0u;
                uint32_t fetch_at = ntiles > FETCH_AHEAD ? ntiles - FETCH_AHEAD : 0u;
                claim_at = claim_at < tau0 ? tau0 : claim_at;
                fetch_at = fetch_at < claim_at ? claim_at : fetch_at;
                // The queue's answer is not touched before `fetch_at`: an instruction that needs it
                // would hold up the tiles issued in between for the atomic's round trip.
                uint32_t claimed = 0;
                bool asked = false, fetched = false;
                auto fetch_next = [&]() {
                    asm volatile("" : "+r"(claimed));  // nothing computed from the answer moves above this point
                    const uint32_t idx_next = asked ? gridDim.x + claimed : a.n_items;
                    fetch(k + 1, idx_next);
                    queue_dry = idx_next >= a.n_items;
                    // The item being issued is this CTA's last: once its last chunk's states are handed over, nothing
                    // is copied into the ring any more and the epilogue warp may use it.
                    if (queue_dry) *final_chunks = nchunks;
                    fetched = true;
                };
                for (uint32_t t0 = tau0; t0 < ntiles && !failed; t0 += ISSUE_LANES) {
                    if (lane == 0) {  // the queue is lane 0's business
                        if (!asked && !queue_dry && t0 + ISSUE_LANES > claim_at) { claimed = atomicAdd(a.queue, 1u); asked = true; }
                        if (!fetched && t0 + ISSUE_LANES > fetch_at) fetch_next();
                    }
                    const uint32_t tau = t0 + lane;
                    if (tau < ntiles && !issue_tile(tau)) failed = true;
                    if (PF_DIST > 0 && tau + PF_DIST < ntiles) prefetch_tile(tau + PF_DIST);
                }
                if (lane == 0 && !fetched && !failed) {  // every tile went out before the dependency wait
                    if (!queue_dry) { claimed = atomicAdd(a.queue, 1u); asked = true; }
                    fetch_next();
                }
                tr.mark(3);  // item issue ends
            }
            nprod += ntiles;
            if (__any_sync(0xffffffffu, failed)) { failed = true; break; }
        }
        if (lane == 0) {
            if (failed) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
            tr.mark(4);  // producer exit
            // The last CTA to run out of work leaves the queue ready for the next launch.
            const uint32_t done = atomicAdd(a.queue + 1, 1u);
            if (done == gridDim.x - 1) { a.queue[0] = 0; a.queue[1] = 0; }
        }
        return;
    }

    if (warp == CW + 1) {
        // ================================ epilogue ================================
        // The consumer warps never wait for one another: each leaves its state of an item (its
        // maxima, row sums and unnormalised outputs over the tiles it took) in a buffer and goes
        // on with the next item.  This warp puts the item together: it merges the CW states in
        // the order of the tiles' places in the item, stores the chunk's partial result (or the
        // output, for a sequence in one piece), gives the buffer back, and then does what has
        // device-wide latency: the fence, the arrival count and, for the last chunk of a
        // sequence to arrive, the merge over chunks.
        if (a.overlap) grid_dep_wait();  // before this grid's first write to `out` or the scratch
        constexpr int NJ = 8 * D / 4 / 32;
        const float* res_all = reinterpret_cast<const float*>(smem + SM::res_off);
        Tracer tr(a.trace_id, 1, lane == 0);
        Running<D> run;
        for (uint32_t kp = 0;; kp++) {
            const uint32_t ms = kp % MAIL_SLOTS, ns = kp % NOTE_SLOTS;
            // What the item is: the consumers say so when they start it.
            if (!__all_sync(0xffffffffu, mbar_wait(note0 + ns * 8, (kp / NOTE_SLOTS) & 1))) return;  // the abort path
            Mail m;
            m.seq = mailbox[ns].seq; m.head0 = mailbox[ns].head0; m.nheads = mailbox[ns].nheads; m.part0 = mailbox[ns].part0;
            m.nch = mailbox[ns].nch; m.counter = mailbox[ns].counter; m.stop = mailbox[ns].stop; m.chunk = mailbox[ns].chunk;
            if (m.stop) return;
            // While they stream it: if the item is its node's last arrival, fold what precedes it.
            uint32_t folded = m.chunk != NO_PART ? fold_ahead<D>(a, m, lane, run) : (uint32_t)FOLD_GAVE_UP;
            // Not yet: some other chunk of the node has not arrived.  This warp has nothing else to do until the
            // item's states are ready, so it looks again (a round trip to the L2 each time) in between.
            for (uint32_t i = 0; folded == FOLD_NOT_YET && i < WAIT_LIMIT; i++) {
                const uint32_t ready = mbar_try_wait(rfull0 + ms * 8, (kp / MAIL_SLOTS) & 1) ? 1u : 0u;
                if (__shfl_sync(0xffffffffu, ready, 0)) break;
                folded = fold_ahead<D>(a, m, lane, run);
            }
            const bool ahead = folded == FOLD_DONE;
            tr.mark(ahead ? 18 : 19);  // note read (and the node's other entries folded)
            if (!__all_sync(0xffffffffu, mbar_wait(rfull0 + ms * 8, (kp / MAIL_SLOTS) & 1))) return;
            tr.mark(10);  // states ready
            const bool direct = m.chunk == NO_PART;
            const float* rb = res_all + ms * CW * SM::res_floats;
            // Output i = lane + 32 j of the item's 8 x D/4 float4 values, over the CW states in
            // the order of the tiles' places in the item.
            float4 E[NJ];
            float El[NJ];
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const uint32_t i = lane + j * 32, h = i / (D / 4), x = (i % (D / 4)) * 4;
                float mc[CW];
                float M = -INFINITY;
#pragma unroll
                for (int c = 0; c < CW; c++) { mc[c] = rb[c * SM::res_floats + h]; M = fmaxf(M, mc[c]); }
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float l = 0.f;
#pragma unroll
                for (int c = 0; c < CW; c++) {
                    const float* r = rb + c * SM::res_floats;
                    const float wg = ex2(mc[c] - M);
                    const float4 v = *reinterpret_cast<const float4*>(r + 16 + h * SM::res_row + x);
                    acc.x = fmaf(v.x, wg, acc.x); acc.y = fmaf(v.y, wg, acc.y);
                    acc.z = fmaf(v.z, wg, acc.z); acc.w = fmaf(v.w, wg, acc.w);
                    l = fmaf(r[8 + h], wg, l);
                }
                E[j] = acc; El[j] = l;
            }
            // The chunk's maxima (lanes 0..7) and row sums (lanes 8..15), by the same sums.
            float Eml = 0.f;
            if (!direct) {
                const uint32_t h = lane & 7;
                float M = -INFINITY, l = 0.f;
#pragma unroll
                for (int c = 0; c < CW; c++) M = fmaxf(M, rb[c * SM::res_floats + h]);
#pragma unroll
                for (int c = 0; c < CW; c++) {
                    const float* r = rb + c * SM::res_floats;
                    l = fmaf(r[8 + h], ex2(r[h] - M), l);
                }
                Eml = lane < 8 ? M : l;
            }
            __syncwarp();  // every lane has read what it needs of the buffer
            if (lane == 0) mbar_arrive(rfree0 + ms * 8);
            tr.mark(13);  // states merged, buffer given back
            if (direct) {
#pragma unroll
                for (int j = 0; j < NJ; j++) {
                    const uint32_t i = lane + j * 32, h = i / (D / 4), x = (i % (D / 4)) * 4;
                    if (h < m.nheads) {
                        const float inv = 1.0f / El[j];
                        *reinterpret_cast<float4*>(a.out + ((size_t)m.seq * a.heads + m.head0 + h) * D + x) =
                            make_float4(E[j].x * inv, E[j].y * inv, E[j].z * inv, E[j].w * inv);
                    }
                }
            } else {
                // The CTA's last chunk: its states are in, so every copy into the ring has landed and been read.
                const bool ring_free = kp + 1 == *final_chunks;
                climb<D>(a, m, lane, E, Eml, ahead, run, tr, ring_free, smem + SM::ring_off, sbase + SM::ring_off);
            }
            tr.mark(11);  // deliver done
        }
    }

    // ================================ consumers ================================
    float* res_all = reinterpret_cast<float*>(smem + SM::res_off);
    WS ws;
    uint32_t nbase = 0;   // tiles of the items before this one
    Tracer tr(a.trace_id, warp == 0 ? 2 : 3, lane == 0 && (warp == 0 || warp == CW - 1));
    bool dead = false;    // this warp gave up a wait
    uint32_t kc = 0;      // chunks handed over so far, over all items
    // The queries come from the stream's earlier work, which the producer waits for before it asks for
    // them: wait for it here too (it returns when that work is done, however long it takes), so that the
    // bounded wait below only ever measures this CTA's own copies.
    if (a.overlap) grid_dep_wait();
    for (uint32_t k = 0;; k++) {
        const uint32_t rslot = k % REC_SLOTS, qslot = k % Q_SLOTS;
        Item it{};
        uint32_t chunk_tokens = 0, run = 1;
        if (!dead && !__all_sync(0xffffffffu, mbar_wait(qfull0 + qslot * 8, (k / Q_SLOTS) & 1))) dead = true;
        // The record came by bulk copy: observe its own barrier too before reading it.
        if (!dead && !__all_sync(0xffffffffu, mbar_wait(recbar0 + rslot * 8, (k / REC_SLOTS) & 1))) dead = true;
        if (!dead) {
            const uint32_t* rec = reinterpret_cast<const uint32_t*>(smem + SM::rec_off) + rslot * REC_WORDS;
            it.seq = rec[0]; it.tokens = rec[1]; it.head0 = rec[2]; it.nheads = rec[3] & 0xffffu; it.kv_head = rec[3] >> 16;
            it.part = rec[4]; it.part0 = rec[5]; it.nch = rec[6]; it.counter = rec[7];
            chunk_tokens = rec[8]; run = rec[9];
        }
        if (dead) {
            // Every other wait in the CTA is bounded too: the others give up in their turn.
            if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
            return;
        }
        // The epilogue warp learns of every chunk when the consumers start it (below), and of the
        // end of the queue here.  It has finished chunk kc - 3 at least -- the state buffers are
        // handed over two at a time -- so note slot kc % NOTE_SLOTS is free.
        if (it.tokens == 0) {  // the end of the queue: every consumer warp reads the same record
            if (warp == 0 && lane == 0) {
                const uint32_t ns = kc % NOTE_SLOTS;
                mailbox[ns].stop = 1u;
                mbar_arrive(note0 + ns * 8);
            }
            return;
        }
        tr.mark(20);  // item header read
        ws.begin_item(smem + SM::q_off + qslot * 8 * SM::q_stride, SM::q_stride, it.nheads, lane, smem + SM::ps_off + warp * (TILE * 8 * 8));
        if (WS::queries_in_registers) {
            __syncwarp();
            if (lane == 0) mbar_arrive(qempty0 + qslot * 8);  // the producer may reuse this query slot
        }
        // The item's chunks, one after the other: each has its own state and its own hand-over, so
        // its result is what it would be as an item of its own; the queries, the record and the
        // producer's set-up are shared by the run.
        for (uint32_t j = 0; j < run; j++, kc++) {
        const uint32_t ms = kc % MAIL_SLOTS;
        const uint32_t ctokens = min(chunk_tokens, it.tokens - j * chunk_tokens);
        if (warp == 0 && lane == 0) {
            const uint32_t ns = kc % NOTE_SLOTS;
            mailbox[ns].seq = it.seq; mailbox[ns].head0 = it.head0; mailbox[ns].nheads = it.nheads;
            mailbox[ns].part0 = it.part0; mailbox[ns].nch = it.nch; mailbox[ns].counter = it.counter;
            mailbox[ns].stop = 0u;
            mailbox[ns].chunk = it.part == NO_PART ? NO_PART : it.part - it.part0 + j;
            mbar_arrive(note0 + ns * 8);
        }
        // Tiles are dealt to the warps by their number in the whole stream; this warp takes the
        // chunk's tiles first, first + CW, ...  Its state goes to place `first` of the buffer, so
        // the merge runs in the order of the tiles' places in the chunk and the sum order does not
        // depend on how many tiles this CTA happened to stream before it.
        const uint32_t first = (warp + CW - nbase % CW) % CW;
        ws.begin_chunk();
        {
            const uint32_t ntiles = (ctokens + TILE - 1) / TILE;
            for (uint32_t tau = first; tau < ntiles; tau += CW) {
                const uint32_t n = nbase + tau;
                const uint32_t st = n % SM::stages, ph = (n / SM::stages) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(full0 + st * 8, ph))) { dead = true; break; }
                const uint32_t kt = sbase + SM::ring_off + st * SM::stage_bytes, vt = kt + SM::tile_bytes;
                const uint32_t valid = min((uint32_t)TILE, ctokens - tau * TILE);
#if !(defined(QVX_EXPERIMENTS) && defined(QVX_EXPERIMENT_NOCOMPUTE))
                ws.tile(kt, vt, smem + SM::ring_off + st * SM::stage_bytes, smem + SM::ring_off + st * SM::stage_bytes + SM::tile_bytes, valid,
                        lane, a.scale_log2);
#else
                (void)kt; (void)vt; (void)valid;
#endif
                __syncwarp();  // every lane is done with this stage
                if (lane == 0) mbar_arrive(empty0 + st * 8);
            }
            nbase += ntiles;
        }
        tr.mark(21);  // tiles done
        if (dead) {
            if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
            return;
        }
        // ---- this warp's state goes to the epilogue warp, and the warp goes on -------------------
        // The buffer is free once the epilogue warp has merged the item two before this one.
        if (!__all_sync(0xffffffffu, mbar_wait(rfree0 + ms * 8, ((kc / MAIL_SLOTS) & 1) ^ 1))) {
            if (lane == 0) atomicExch(a.status, STATUS_WAIT_TIMEOUT);
            return;
        }
        ws.store(res_all + (ms * CW + first) * SM::res_floats, SM::res_row, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(rfull0 + ms * 8);
        tr.mark(23);  // state handed over
        }  // chunks of the item
        if (!WS::queries_in_registers && lane == 0) mbar_arrive(qempty0 + qslot * 8);  // (the __syncwarp above: every lane is done with the queries)
    }
}

// ---- host side -----------------------------------------------------------------------------------
extern int* device_status_word(qvx_device* dev);

// The geometries this kernel serves: native-layout pools of any dtype, blocks of whole tiles, GQA groups.
// Everything else runs in the reference's operation order (attn_exact.cu).
bool attn_split_supported(const Layout& L, size_t heads) {
    if (L.layout != QVX_LAYOUT_NATIVE) return false;
    if (L.B % TILE != 0 || heads == 0 || heads % L.kvh != 0) return false;
    if (L.dtype == QVX_F32) return L.d == 64 || L.d == 128;
    return L.d == 64 || L.d == 128 || L.d == 256;
}
// The new position's rows are stored by the attention launch itself.
bool attn_split_fuses_append(const Layout& L, size_t heads) { return attn_split_supported(L, heads); }

// Floats of scratch the partial results take; partial slots and arrival counters a split (sequence, group) of
// `nch` chunks takes (the merge tree's entries and nodes).
size_t attn_partial_floats(const qvx_tables* t) { return t->n_parts * (8 * (size_t)t->L.d + 16); }
uint32_t attn_parts_per_group(const Layout&, uint32_t nch) { return merge_entries_total(nch); }
uint32_t attn_counters_per_group(const Layout&, uint32_t nch) { return merge_counters_total(nch); }

template <int DT, int D, int VAR>
static int32_t launch_stream(qvx_device* dev, const StreamArgs& a, cudaStream_t s) {
    using SM = StreamSmem<D, (DT == QVX_F32 ? 4 : 2)>;
    // (the cross-chunk merge stages a node's entries in the ring, sized by the 16-bit layout's)
#ifndef QVX_MAX_STAGES
    static_assert(SM::stages * SM::stage_bytes >= MERGE_FAN * (8 * D + 16) * 4 || D > 128, "the ring holds a merge node's entries");
#endif
    auto kernel = attn_stream_kernel<DT, D, VAR>;
    static int per_device[64] = {};  // set up once per device (the attribute belongs to the device's context)
    int& ctas_per_sm = per_device[dev->ordinal & 63];
    if (!ctas_per_sm) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::total);
        if (e == cudaSuccess)
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kernel, STREAM_THREADS, SM::total);
        if (e != cudaSuccess) { ctas_per_sm = 0; return check_cuda(dev, e, "streaming attention set-up"); }
        if (ctas_per_sm < 1) ctas_per_sm = 1;
    }
    const unsigned grid = (unsigned)std::min<size_t>(a.n_items, (size_t)ctas_per_sm * dev->prop.multiProcessorCount);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(STREAM_THREADS); cfg.dynamicSmemBytes = SM::total; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = a.overlap ? 1 : 0;
#if QVX_TRACING
    {
        static uint32_t launches = 0;
        StreamArgs at = a;
        at.trace_id = launches++;
        const char* path = getenv("QVX_TRACE_FILE");
        const char* only = getenv("QVX_TRACE_AT");
        cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, at);
        if (e == cudaSuccess && path && (!only || (uint32_t)atol(only) == launches)) {
            cudaDeviceSynchronize();
            std::vector<unsigned long long> h(2 * 512 * TRACE_PER_CTA);  // this launch's buffer first, then the one before it
            cudaMemcpyFromSymbol(h.data(), g_trace, h.size() * 4, (at.trace_id & 1) * h.size() * 4);
            cudaMemcpyFromSymbol(h.data() + h.size() / 2, g_trace, h.size() * 4, ((at.trace_id & 1) ^ 1) * h.size() * 4);
            FILE* f = fopen(path, "wb");
            if (f) { unsigned hdr[2] = {grid, at.trace_id & 15u}; fwrite(hdr, 4, 2, f); fwrite(h.data(), 8, h.size(), f); fclose(f); }
        }
        return check_cuda(dev, e, "streaming attention launch");
    }
#endif
    return check_cuda(dev, cudaLaunchKernelEx(&cfg, kernel, a), "streaming attention launch");
}

int32_t launch_attn_split(qvx_device* dev, qvx_tables* t, const void* pool, const float* q, float* out,
                          float* partials, uint32_t* counters, uint32_t* queue, const float* k_new, const float* v_new,
                          bool overlap, cudaStream_t s) {
    if (t->n_items == 0) return QVX_OK;
    const Layout& L = t->L;
    if (t->item_words > REC_WORDS)
        return fail(dev, QVX_ERR_UNSUPPORTED, "streaming attention: %u blocks per chunk are too many", t->chunk_blocks);
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 15u) || ((uintptr_t)pool & 127u))
        return fail(dev, QVX_ERR_SHAPE,
                    "shape mismatch in routed moe attention: q and out must be 16-byte aligned, the pool 128-byte aligned");
    StreamArgs a;
    a.pool = (const uint8_t*)pool; a.q = q; a.out = out; a.partials = partials; a.counters = counters; a.queue = queue;
    a.items = t->d_items; a.status = device_status_word(dev);
    a.k_new = k_new; a.v_new = v_new; a.kv_out = L.kvh * L.d; a.overlap = overlap ? 1u : 0u;
    if (k_new && (((uintptr_t)k_new | (uintptr_t)v_new) & 15u))
        return fail(dev, QVX_ERR_SHAPE, "shape mismatch in routed moe attention: k_new and v_new must be 16-byte aligned");
    a.block_bytes = L.block_bytes; a.page_bytes = L.page_bytes; a.tiles_per_block = L.B / TILE;
    a.heads = (uint32_t)t->heads; a.item_words = t->item_words; a.n_items = (uint32_t)t->n_items;
    a.scale_log2 = (1.0f / sqrtf((float)L.d)) * 1.4426950408889634f;
    a.trace_id = 0;
    a.test_hooks = 0;
#ifdef QVX_TEST_HOOKS
    if (const char* v = getenv("QVX_TEST_LOSE_A_PUBLICATION")) a.test_hooks = atol(v) ? 1u : 0u;
#endif
    // bf16 carries 8 mantissa bits: the queries and the probabilities go through the tensor cores as a value and
    // a remainder (bit 0: queries, bit 1: probabilities).  An experiment build can leave passes out
    // (QVX_ATTN_ONE_PASS = 1: both, 2: the probabilities', 3: the queries').
    int passes = L.dtype == QVX_BF16 ? QVX_BF16_PASSES : 0;
#ifdef QVX_EXPERIMENTS
    if (const char* v = getenv("QVX_ATTN_ONE_PASS")) {
        const long n = atol(v);
        if (L.dtype == QVX_BF16) passes = n == 1 ? 0 : n == 2 ? 1 : n == 3 ? 2 : 3;
    }
#endif
    LaunchTimer timer(dev, QVX_K_ATTN, s);
    int32_t rc = QVX_ERR_UNSUPPORTED;
#define QVX_STREAM_CASE(TT, DD, PP) \
    if (L.dtype == TT && L.d == DD && passes == PP) rc = launch_stream<TT, DD, PP>(dev, a, s);
    QVX_STREAM_CASE(QVX_BF16, 64, QVX_BF16_PASSES) QVX_STREAM_CASE(QVX_BF16, 128, QVX_BF16_PASSES)
    QVX_STREAM_CASE(QVX_BF16, 256, QVX_BF16_PASSES)
#ifdef QVX_EXPERIMENTS
    if (L.d == 128 && passes != QVX_BF16_PASSES) {
        QVX_STREAM_CASE(QVX_BF16, 128, 0) QVX_STREAM_CASE(QVX_BF16, 128, 1) QVX_STREAM_CASE(QVX_BF16, 128, 2)
        QVX_STREAM_CASE(QVX_BF16, 128, 3)
    }
#endif
    QVX_STREAM_CASE(QVX_F16, 64, 0) QVX_STREAM_CASE(QVX_F16, 128, 0) QVX_STREAM_CASE(QVX_F16, 256, 0)
    if (L.dtype == QVX_F32) {
        // The arithmetic is unrolled over the query heads of a group (items hold up to 8 of them).
        const size_t group = t->heads / L.kvh;
        passes = group <= 2 ? 2 : group <= 4 ? 4 : 8;
        QVX_STREAM_CASE(QVX_F32, 64, 2) QVX_STREAM_CASE(QVX_F32, 64, 4) QVX_STREAM_CASE(QVX_F32, 64, 8)
        QVX_STREAM_CASE(QVX_F32, 128, 2) QVX_STREAM_CASE(QVX_F32, 128, 4) QVX_STREAM_CASE(QVX_F32, 128, 8)
    }
#undef QVX_STREAM_CASE
    if (rc == QVX_ERR_UNSUPPORTED) return fail(dev, rc, "streaming attention: no kernel for this geometry");
    return rc;
}

}  // namespace qvx
