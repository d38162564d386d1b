// Host-side block bookkeeping: integers only, no CUDA.
//
// Mirrors, for the paged decode path, what the reference keeps in its runtime and in its
// prefix index:
//   KvPool / KvFree / Mirror / LayerMirror / AttnPlan / attention_plan
//       crates/qubivex-runtime/src/discrete.rs:215-290, :429-455, :929-1009
//   PrefixCache<V>
//       crates/qubivex-kv-cache/src/lib.rs:22-209
// and adds what the reference lists as not built (docs/decisions/ADR-016-KV-SUBSYSTEM.md:82-89,
// :148-150): blocks shared between sequences by reference count, copy-on-write before the
// first divergent append, and a compaction pass that gathers live blocks to the front.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/qvx.h"

namespace {

uint32_t elem_size(uint32_t dtype) { return dtype == QVX_F32 ? 4u : 2u; }

struct PoolCore {
    std::mutex mu;
    qvx_geometry geo{};
    uint64_t block_bytes = 0;
    uint32_t blocks = 0;
    std::vector<uint32_t> free;      // LIFO: back() is handed out next
    std::vector<uint32_t> refs;      // per block
    std::set<qvx_seq*> seqs;         // every live sequence, for compaction
    bool allocated = false;
    uint64_t layers = 0, synced_rows = 0, full = 0, cow_copies = 0, compaction_moves = 0, bytes_moved = 0;
};

struct LayerMirror {
    std::vector<uint32_t> blocks;  // in position order
    size_t synced = 0;             // positions of this layer the pool holds
};

}  // namespace

struct qvx_kvpool {
    std::shared_ptr<PoolCore> core;
};

struct qvx_seq {
    std::shared_ptr<PoolCore> core;  // the mirror's own hold on the free list (Mirror.free, :260)
    uint64_t epoch = 0;
    std::vector<LayerMirror> layers;
};

struct qvx_plan {
    std::vector<uint32_t> pos, table_at, blocks, sync_to, sync_seq, sync_pos, copy_src, copy_dst;
};

namespace {

// Drops one reference; a block nobody holds goes back on the free list.
void unref(PoolCore& c, uint32_t b) {
    if (--c.refs[b] == 0) c.free.push_back(b);
}

// Mirror::release (discrete.rs:266-273): every block back, synced to 0.  Caller holds c.mu.
void release_locked(PoolCore& c, qvx_seq* q) {
    for (auto& l : q->layers) {
        for (uint32_t b : l.blocks) unref(c, b);
        l.blocks.clear();
        l.synced = 0;
    }
}

}  // namespace

extern "C" {

uint64_t qvx_kvpool_blocks_for(const qvx_geometry* geo, uint64_t configured, uint64_t budget_left, uint64_t max_arena,
                               int uncapped) {
    if (!geo || !geo->block_tokens || !geo->kv_heads || !geo->head_dim) return 0;
    uint64_t bb = 2ull * geo->block_tokens * geo->kv_heads * geo->head_dim * elem_size(geo->dtype);
    const uint64_t DEFAULT_KV_POOL = 512ull << 20, MAX_KV_POOL = 1ull << 30;  // discrete.rs:209-213
    uint64_t room = uncapped ? configured : std::min(configured ? configured : DEFAULT_KV_POOL, MAX_KV_POOL);
    room = std::min(room, std::min(budget_left, max_arena));
    uint64_t blocks = room / bb;
    return std::min<uint64_t>(blocks, 0xffffffffull);
}

qvx_kvpool* qvx_kvpool_new(const qvx_geometry* geo, uint32_t blocks) {
    if (!geo || !blocks) return nullptr;
    auto core = std::make_shared<PoolCore>();
    core->geo = *geo;
    core->block_bytes = 2ull * geo->block_tokens * geo->kv_heads * geo->head_dim * elem_size(geo->dtype);
    core->blocks = blocks;
    core->refs.assign(blocks, 0);
    core->free.resize(blocks);
    for (uint32_t i = 0; i < blocks; i++) core->free[i] = blocks - 1 - i;  // (0..blocks).rev(): first pop is 0
    return new qvx_kvpool{core};
}

void qvx_kvpool_delete(qvx_kvpool* p) { delete p; }

int32_t qvx_kvpool_set_free_order(qvx_kvpool* p, const uint32_t* order, size_t n) {
    if (!p || (!order && n)) return QVX_ERR_SHAPE;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    if (n != c.free.size()) return QVX_ERR_SHAPE;
    std::vector<char> seen(c.blocks, 0);
    for (size_t i = 0; i < n; i++) {
        if (order[i] >= c.blocks || seen[order[i]] || c.refs[order[i]] != 0) return QVX_ERR_SHAPE;
        seen[order[i]] = 1;
    }
    for (size_t i = 0; i < n; i++) c.free[n - 1 - i] = order[i];
    return QVX_OK;
}

int32_t qvx_kvpool_stats_get(qvx_kvpool* p, qvx_kvpool_stats* out) {
    if (!p || !out) return QVX_ERR_SHAPE;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    out->bytes = c.block_bytes * c.blocks;
    out->allocated = c.allocated;
    out->blocks = c.blocks;
    out->free = c.free.size();
    out->layers = c.layers;
    out->synced_rows = c.synced_rows;
    out->full = c.full;
    out->cow_copies = c.cow_copies;
    out->compaction_moves = c.compaction_moves;
    out->bytes_moved = c.bytes_moved;
    uint64_t shared = 0;
    for (uint32_t r : c.refs) shared += r > 1;
    out->shared_blocks = shared;
    return QVX_OK;
}

uint32_t qvx_kvpool_refcount(qvx_kvpool* p, uint32_t block) {
    if (!p) return 0;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    return block < c.blocks ? c.refs[block] : 0;
}

void qvx_kvpool_note_allocated(qvx_kvpool* p, int allocated) {
    if (!p) return;
    std::lock_guard<std::mutex> lk(p->core->mu);
    p->core->allocated = allocated != 0;
}

qvx_seq* qvx_seq_new(qvx_kvpool* p, uint64_t epoch) {
    if (!p) return nullptr;
    qvx_seq* q = new qvx_seq;
    q->core = p->core;
    q->epoch = epoch;
    std::lock_guard<std::mutex> lk(q->core->mu);
    q->core->seqs.insert(q);
    return q;
}

// Drop for Mirror (discrete.rs:276-280).
void qvx_seq_delete(qvx_seq* q) {
    if (!q) return;
    {
        std::lock_guard<std::mutex> lk(q->core->mu);
        release_locked(*q->core, q);
        q->core->seqs.erase(q);
    }
    delete q;
}

size_t qvx_seq_blocks(qvx_seq* q, size_t layer, uint32_t* out, size_t cap) {
    if (!q) return 0;
    std::lock_guard<std::mutex> lk(q->core->mu);
    if (layer >= q->layers.size()) return 0;
    const auto& b = q->layers[layer].blocks;
    if (out) memcpy(out, b.data(), 4 * std::min(cap, b.size()));
    return b.size();
}

size_t qvx_seq_synced(qvx_seq* q, size_t layer) {
    if (!q) return 0;
    std::lock_guard<std::mutex> lk(q->core->mu);
    return layer < q->layers.size() ? q->layers[layer].synced : 0;
}

qvx_seq* qvx_seq_fork(qvx_seq* parent, size_t tokens, uint64_t epoch) {
    if (!parent) return nullptr;
    qvx_seq* q = new qvx_seq;
    q->core = parent->core;
    q->epoch = epoch;
    PoolCore& c = *q->core;
    std::lock_guard<std::mutex> lk(c.mu);
    const size_t B = c.geo.block_tokens;
    q->layers.resize(parent->layers.size());
    for (size_t l = 0; l < parent->layers.size(); l++) {
        const LayerMirror& pl = parent->layers[l];
        size_t have = std::min(tokens, pl.synced);        // only what the pool really holds
        size_t nb = std::min(pl.blocks.size(), (have + B - 1) / B);
        q->layers[l].blocks.assign(pl.blocks.begin(), pl.blocks.begin() + nb);
        for (uint32_t b : q->layers[l].blocks) c.refs[b]++;
        q->layers[l].synced = have;
    }
    c.seqs.insert(q);
    return q;
}

int32_t qvx_plan_build(qvx_kvpool* p, qvx_seq* const* seqs, const uint64_t* epochs, const uint32_t* pos, size_t s,
                       size_t layer, qvx_plan** out) {
    if (!p || !out || (s && (!seqs || !pos))) return QVX_ERR_SHAPE;
    *out = nullptr;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    const size_t B = c.geo.block_tokens;
    for (size_t i = 0; i < s; i++)
        if (!seqs[i] || seqs[i]->core.get() != &c) return QVX_ERR_SHAPE;  // a mirror of another pool

    // First pass (discrete.rs:975-985): epochs and the synced clamp, then count what the pass
    // needs: blocks to grow to pos / B + 1, and one fresh block for every held block that
    // will be written (positions synced..=pos) while somebody else also holds it.
    size_t need_total = 0;
    for (size_t i = 0; i < s; i++) {
        qvx_seq* q = seqs[i];
        if (epochs && q->epoch != epochs[i]) {
            release_locked(c, q);
            q->epoch = epochs[i];
        }
        if (q->layers.size() <= layer) q->layers.resize(layer + 1);
        LayerMirror& lm = q->layers[layer];
        lm.synced = std::min<size_t>(lm.synced, pos[i]);
        size_t need = pos[i] / B + 1;
        if (lm.blocks.size() < need) need_total += need - lm.blocks.size();
        for (size_t bi = lm.synced / B; bi < std::min(need, lm.blocks.size()); bi++)
            if (c.refs[lm.blocks[bi]] > 1) need_total++;
    }
    if (need_total > c.free.size()) {
        // The reference pops until the list is dry and the blocks taken stay with their
        // sequence (discrete.rs:986-992); nothing is copied or swapped on this path.
        for (size_t i = 0; i < s; i++) {
            LayerMirror& lm = seqs[i]->layers[layer];
            size_t need = pos[i] / B + 1;
            while (lm.blocks.size() < need && !c.free.empty()) {
                uint32_t b = c.free.back();
                c.free.pop_back();
                c.refs[b] = 1;
                lm.blocks.push_back(b);
            }
            if (lm.blocks.size() < need) break;
        }
        c.full++;
        return QVX_DECLINED;
    }
    qvx_plan* pl = new qvx_plan;
    for (size_t i = 0; i < s; i++) {
        LayerMirror& lm = seqs[i]->layers[layer];
        size_t need = pos[i] / B + 1;
        for (size_t bi = lm.synced / B; bi < std::min(need, lm.blocks.size()); bi++) {
            uint32_t old = lm.blocks[bi];
            if (c.refs[old] <= 1) continue;
            uint32_t nb = c.free.back();
            c.free.pop_back();
            c.refs[nb] = 1;
            c.refs[old]--;
            lm.blocks[bi] = nb;
            pl->copy_src.push_back(old);
            pl->copy_dst.push_back(nb);
            c.cow_copies++;
            c.bytes_moved += 2 * c.block_bytes;
        }
        while (lm.blocks.size() < need) {
            uint32_t b = c.free.back();
            c.free.pop_back();
            c.refs[b] = 1;
            lm.blocks.push_back(b);
        }
        pl->pos.push_back(pos[i]);
        pl->table_at.push_back((uint32_t)pl->blocks.size());
        pl->blocks.insert(pl->blocks.end(), lm.blocks.begin(), lm.blocks.begin() + need);
        for (size_t pp = lm.synced; pp < pos[i]; pp++) {
            pl->sync_to.push_back((uint32_t)(lm.blocks[pp / B] * B + pp % B));
            pl->sync_seq.push_back((uint32_t)i);
            pl->sync_pos.push_back((uint32_t)pp);
        }
    }
    *out = pl;
    return QVX_OK;
}

void qvx_plan_free(qvx_plan* pl) { delete pl; }

size_t qvx_plan_counts(qvx_plan* pl, size_t* n_blocks, size_t* n_sync, size_t* n_copies) {
    if (!pl) return 0;
    if (n_blocks) *n_blocks = pl->blocks.size();
    if (n_sync) *n_sync = pl->sync_to.size();
    if (n_copies) *n_copies = pl->copy_src.size();
    return pl->pos.size();
}
const uint32_t* qvx_plan_pos(qvx_plan* pl) { return pl->pos.data(); }
const uint32_t* qvx_plan_table_at(qvx_plan* pl) { return pl->table_at.data(); }
const uint32_t* qvx_plan_blocks(qvx_plan* pl) { return pl->blocks.data(); }
const uint32_t* qvx_plan_sync_to(qvx_plan* pl) { return pl->sync_to.data(); }
const uint32_t* qvx_plan_sync_seq(qvx_plan* pl) { return pl->sync_seq.data(); }
const uint32_t* qvx_plan_sync_pos(qvx_plan* pl) { return pl->sync_pos.data(); }
const uint32_t* qvx_plan_copy_src(qvx_plan* pl) { return pl->copy_src.data(); }
const uint32_t* qvx_plan_copy_dst(qvx_plan* pl) { return pl->copy_dst.data(); }

void qvx_plan_commit(qvx_kvpool* p, qvx_plan* pl, qvx_seq* const* seqs, size_t layer) {
    if (!p || !pl) return;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    for (size_t i = 0; i < pl->pos.size(); i++)
        if (seqs[i] && layer < seqs[i]->layers.size()) seqs[i]->layers[layer].synced = (size_t)pl->pos[i] + 1;
    c.layers++;
    c.synced_rows += pl->sync_to.size();
}

int32_t qvx_kvpool_compact(qvx_kvpool* p, uint32_t* src_out, uint32_t* dst_out, size_t cap, size_t* n_moves) {
    if (!p || !n_moves) return QVX_ERR_SHAPE;
    PoolCore& c = *p->core;
    std::lock_guard<std::mutex> lk(c.mu);
    const uint32_t live = c.blocks - (uint32_t)c.free.size();
    std::vector<uint32_t> holes, movers;
    for (uint32_t b = 0; b < live; b++)
        if (c.refs[b] == 0) holes.push_back(b);
    for (uint32_t b = live; b < c.blocks; b++)
        if (c.refs[b] != 0) movers.push_back(b);
    // As many live blocks sit past L as there are holes before it.
    *n_moves = movers.size();
    if (movers.size() > cap || (movers.size() && (!src_out || !dst_out))) return QVX_ERR_SHAPE;
    std::vector<uint32_t> remap(c.blocks);
    for (uint32_t b = 0; b < c.blocks; b++) remap[b] = b;
    for (size_t i = 0; i < movers.size(); i++) {
        src_out[i] = movers[i];
        dst_out[i] = holes[i];
        remap[movers[i]] = holes[i];
        c.refs[holes[i]] = c.refs[movers[i]];
        c.refs[movers[i]] = 0;
    }
    for (qvx_seq* q : c.seqs)
        for (auto& l : q->layers)
            for (uint32_t& b : l.blocks) b = remap[b];
    c.free.resize(c.blocks - live);
    for (uint32_t i = 0; i < c.blocks - live; i++) c.free[i] = c.blocks - 1 - i;  // lowest id popped first
    c.compaction_moves += movers.size();
    c.bytes_moved += 2 * c.block_bytes * movers.size();
    return QVX_OK;
}

}  // extern "C"

// =================================================================================================
// PrefixCache (crates/qubivex-kv-cache/src/lib.rs:67-209)
// =================================================================================================
namespace {

// Arc<V>: the index and every hit hold one count; the release callback runs at zero.
struct Held {
    uint64_t value;
    uint64_t refs;
};

struct Entry {
    bool scoped;
    std::string scope;
    std::vector<uint32_t> tokens;
    uint64_t cost;
    Held* value;
    uint64_t used;
};

bool same_scope(const Entry& e, const char* scope) {
    return scope ? (e.scoped && e.scope == scope) : !e.scoped;
}

size_t common_prefix(const std::vector<uint32_t>& a, const uint32_t* b, size_t nb) {
    size_t n = std::min(a.size(), nb), i = 0;
    while (i < n && a[i] == b[i]) i++;
    return i;
}

}  // namespace

struct qvx_prefix_cache {
    std::mutex mu;
    uint64_t budget;
    std::vector<Entry> entries;
    uint64_t clock = 0;
    qvx_prefix_stats stats{};
    qvx_release_fn release;
    void* user;

    void drop(Held* h) {
        if (--h->refs == 0) {
            if (release) release(h->value, user);
            delete h;
        }
    }
    // evict_oldest, lib.rs:184-199 (swap_remove keeps the reference's entry order).
    bool evict_oldest() {
        if (entries.empty()) return false;
        size_t at = 0;
        for (size_t i = 1; i < entries.size(); i++)
            if (entries[i].used < entries[at].used) at = i;
        Entry e = std::move(entries[at]);
        entries[at] = std::move(entries.back());
        entries.pop_back();
        stats.cost -= e.cost;
        stats.entries -= 1;
        stats.evicted += 1;
        drop(e.value);
        return true;
    }
};

extern "C" {

qvx_prefix_cache* qvx_prefix_new(uint64_t budget, qvx_release_fn release, void* user) {
    qvx_prefix_cache* c = new qvx_prefix_cache;
    c->budget = budget;
    c->release = release;
    c->user = user;
    return c;
}

void qvx_prefix_delete(qvx_prefix_cache* c) {
    if (!c) return;
    {
        std::lock_guard<std::mutex> lk(c->mu);
        for (auto& e : c->entries) c->drop(e.value);
        c->entries.clear();
    }
    delete c;
}

uint64_t qvx_prefix_budget(qvx_prefix_cache* c) { return c ? c->budget : 0; }

int32_t qvx_prefix_lookup(qvx_prefix_cache* c, const char* scope, const uint32_t* prompt, size_t n, uint64_t* value,
                          size_t* reuse, uint64_t* hit) {
    if (!c) return 0;
    std::lock_guard<std::mutex> lk(c->mu);
    c->stats.lookups++;
    if (n == 0) return 0;
    const size_t limit = n - 1;  // the last token always runs
    bool found = false;
    size_t best_n = 0, best_i = 0;
    for (size_t i = 0; i < c->entries.size(); i++) {
        const Entry& e = c->entries[i];
        if (!same_scope(e, scope)) continue;
        size_t shared = std::min(common_prefix(e.tokens, prompt, n), limit);
        if (shared >= QVX_MIN_REUSE && (!found || shared > best_n)) {
            found = true; best_n = shared; best_i = i;
        }
    }
    if (!found) return 0;
    Entry& e = c->entries[best_i];
    e.used = ++c->clock;
    e.value->refs++;
    c->stats.hits++;
    c->stats.tokens_reused += best_n;
    if (value) *value = e.value->value;
    if (reuse) *reuse = best_n;
    if (hit) *hit = (uint64_t)(uintptr_t)e.value;
    else c->drop(e.value);
    return 1;
}

void qvx_prefix_hit_release(qvx_prefix_cache* c, uint64_t hit) {
    if (!c || !hit) return;
    std::lock_guard<std::mutex> lk(c->mu);
    c->drop((Held*)(uintptr_t)hit);
}

int32_t qvx_prefix_insert(qvx_prefix_cache* c, const char* scope, const uint32_t* tokens, size_t n, uint64_t cost,
                          uint64_t value) {
    if (!c) return 0;
    std::lock_guard<std::mutex> lk(c->mu);
    auto refuse = [&]() {
        if (c->release) c->release(value, c->user);
        return 0;
    };
    if (n < QVX_MIN_REUSE || cost > c->budget) return refuse();
    const uint64_t used = ++c->clock;
    // An entry of the scope that already covers these tokens: counts as a use.
    for (auto& e : c->entries) {
        if (same_scope(e, scope) && e.tokens.size() >= n && std::equal(tokens, tokens + n, e.tokens.begin())) {
            e.used = used;
            return refuse();
        }
    }
    // Entries this one covers are replaced (not counted as evictions).
    for (size_t i = 0; i < c->entries.size();) {
        Entry& e = c->entries[i];
        bool covered = same_scope(e, scope) && e.tokens.size() <= n && std::equal(e.tokens.begin(), e.tokens.end(), tokens);
        if (covered) {
            c->stats.cost -= e.cost;
            c->stats.entries -= 1;
            c->drop(e.value);
            c->entries.erase(c->entries.begin() + i);  // Vec::retain keeps the order
        } else {
            i++;
        }
    }
    while (c->stats.cost + cost > c->budget && c->evict_oldest()) {}
    Entry e;
    e.scoped = scope != nullptr;
    if (scope) e.scope = scope;
    e.tokens.assign(tokens, tokens + n);
    e.cost = cost;
    e.value = new Held{value, 1};
    e.used = used;
    c->entries.push_back(std::move(e));
    c->stats.cost += cost;
    c->stats.entries += 1;
    c->stats.inserted += 1;
    return 1;
}

int32_t qvx_prefix_evict_oldest(qvx_prefix_cache* c) {
    if (!c) return 0;
    std::lock_guard<std::mutex> lk(c->mu);
    return c->evict_oldest() ? 1 : 0;
}

void qvx_prefix_clear(qvx_prefix_cache* c) {
    if (!c) return;
    std::lock_guard<std::mutex> lk(c->mu);
    while (c->evict_oldest()) {}
}

void qvx_prefix_stats_get(qvx_prefix_cache* c, qvx_prefix_stats* out) {
    if (!c || !out) return;
    std::lock_guard<std::mutex> lk(c->mu);
    *out = c->stats;
}

}  // extern "C"
