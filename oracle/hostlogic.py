"""Pure-Python restatement of the reference's integer host logic for the paged path.
TEST INFRASTRUCTURE ONLY: the checker for qubivex_b200's C++ block bookkeeping.

  KvFree / LayerMirror / Mirror / attention_plan
      crates/qubivex-runtime/src/discrete.rs:215-290, :951-1009
  PrefixCache
      crates/qubivex-kv-cache/src/lib.rs:67-209

The reference has no shared blocks; `RefPool` follows it exactly for sequences that share
nothing.  Copy-on-write and compaction have no reference counterpart and are restated here
from the rules the build defines (see the C header): parity for them is unpinned.
"""
from __future__ import annotations


class RefPool:
    def __init__(self, blocks: int, block_tokens: int):
        self.B = block_tokens
        self.blocks = blocks
        self.free = list(range(blocks))[::-1]  # (0..blocks).rev(): first pop is block 0 (:447-449)
        self.refs = [0] * blocks
        self.full = 0
        self.layers = 0
        self.synced_rows = 0
        self.cow_copies = 0


class RefMirror:
    def __init__(self, pool: RefPool, epoch: int = 0):
        self.pool, self.epoch = pool, epoch
        self.layers: list[dict] = []  # {"blocks": [...], "synced": n}

    def release(self):  # discrete.rs:266-273
        for l in self.layers:
            for b in l["blocks"]:
                self.pool.refs[b] -= 1
                if self.pool.refs[b] == 0:
                    self.pool.free.append(b)
            l["blocks"] = []
            l["synced"] = 0

    def fork(self, tokens: int, epoch: int = 0) -> "RefMirror":
        m = RefMirror(self.pool, epoch)
        B = self.pool.B
        for l in self.layers:
            have = min(tokens, l["synced"])
            nb = min(len(l["blocks"]), (have + B - 1) // B)
            for b in l["blocks"][:nb]:
                self.pool.refs[b] += 1
            m.layers.append({"blocks": list(l["blocks"][:nb]), "synced": have})
        return m


def attention_plan(pool: RefPool, mirrors, epochs, pos, layer):
    """discrete.rs:951-1009, with the copy-on-write rule added.  None = declined."""
    B = pool.B
    need_total = 0
    for m, ep, p in zip(mirrors, epochs, pos):
        if m.epoch != ep:
            m.release()
            m.epoch = ep
        while len(m.layers) <= layer:
            m.layers.append({"blocks": [], "synced": 0})
        lm = m.layers[layer]
        lm["synced"] = min(lm["synced"], p)
        need = p // B + 1
        need_total += max(0, need - len(lm["blocks"]))
        for bi in range(lm["synced"] // B, min(need, len(lm["blocks"]))):
            if pool.refs[lm["blocks"][bi]] > 1:
                need_total += 1
    if need_total > len(pool.free):
        for m, p in zip(mirrors, pos):
            lm = m.layers[layer]
            need = p // B + 1
            while len(lm["blocks"]) < need and pool.free:
                b = pool.free.pop()
                pool.refs[b] = 1
                lm["blocks"].append(b)
            if len(lm["blocks"]) < need:
                break
        pool.full += 1
        return None
    plan = {"pos": [], "table_at": [], "blocks": [], "sync_to": [], "sync_seq": [], "sync_pos": [],
            "copy_src": [], "copy_dst": []}
    for i, (m, p) in enumerate(zip(mirrors, pos)):
        lm = m.layers[layer]
        need = p // B + 1
        for bi in range(lm["synced"] // B, min(need, len(lm["blocks"]))):
            old = lm["blocks"][bi]
            if pool.refs[old] <= 1:
                continue
            nb = pool.free.pop()
            pool.refs[nb] = 1
            pool.refs[old] -= 1
            lm["blocks"][bi] = nb
            plan["copy_src"].append(old)
            plan["copy_dst"].append(nb)
            pool.cow_copies += 1
        while len(lm["blocks"]) < need:
            b = pool.free.pop()
            pool.refs[b] = 1
            lm["blocks"].append(b)
        plan["pos"].append(p)
        plan["table_at"].append(len(plan["blocks"]))
        plan["blocks"].extend(lm["blocks"][:need])
        for pp in range(lm["synced"], p):
            plan["sync_to"].append(lm["blocks"][pp // B] * B + pp % B)
            plan["sync_seq"].append(i)
            plan["sync_pos"].append(pp)
    return plan


def commit(pool: RefPool, plan, mirrors, layer):  # discrete.rs:929-943
    for m, p in zip(mirrors, plan["pos"]):
        m.layers[layer]["synced"] = p + 1
    pool.layers += 1
    pool.synced_rows += len(plan["sync_to"])


def compact(pool: RefPool, mirrors):
    """Live blocks with id >= L, ascending, move to the free ids < L, ascending."""
    live = pool.blocks - len(pool.free)
    holes = [b for b in range(live) if pool.refs[b] == 0]
    movers = [b for b in range(live, pool.blocks) if pool.refs[b] != 0]
    remap = {s: d for s, d in zip(movers, holes)}
    for s, d in remap.items():
        pool.refs[d], pool.refs[s] = pool.refs[s], 0
    for m in mirrors:
        for l in m.layers:
            l["blocks"] = [remap.get(b, b) for b in l["blocks"]]
    pool.free = list(range(live, pool.blocks))[::-1]
    return movers, holes


MIN_REUSE = 32  # crates/qubivex-kv-cache/src/lib.rs:22


class RefPrefixCache:
    """crates/qubivex-kv-cache/src/lib.rs:67-205, line for line in meaning."""

    def __init__(self, budget: int):
        self.budget = budget
        self.entries: list[dict] = []
        self.clock = 0
        self.stats = dict(lookups=0, hits=0, tokens_reused=0, inserted=0, evicted=0, entries=0, cost=0)

    def lookup(self, scope, prompt):
        self.stats["lookups"] += 1
        if not len(prompt):
            return None
        limit = len(prompt) - 1
        best = None
        for i, e in enumerate(self.entries):
            if e["scope"] != scope:
                continue
            n = 0
            for a, b in zip(e["tokens"], prompt):
                if a != b:
                    break
                n += 1
            shared = min(n, limit)
            if shared >= MIN_REUSE and (best is None or shared > best[0]):
                best = (shared, i)
        if best is None:
            return None
        self.clock += 1
        e = self.entries[best[1]]
        e["used"] = self.clock
        self.stats["hits"] += 1
        self.stats["tokens_reused"] += best[0]
        return e["value"], best[0]

    def insert(self, scope, tokens, cost, value) -> bool:
        tokens = list(tokens)
        if len(tokens) < MIN_REUSE or cost > self.budget:
            return False
        self.clock += 1
        used = self.clock
        for e in self.entries:
            if e["scope"] == scope and e["tokens"][:len(tokens)] == tokens:
                e["used"] = used
                return False
        keep = []
        for e in self.entries:
            if e["scope"] == scope and tokens[:len(e["tokens"])] == e["tokens"]:
                self.stats["cost"] -= e["cost"]
                self.stats["entries"] -= 1
            else:
                keep.append(e)
        self.entries = keep
        while self.stats["cost"] + cost > self.budget and self.evict_oldest():
            pass
        self.entries.append(dict(scope=scope, tokens=tokens, cost=cost, value=value, used=used))
        self.stats["cost"] += cost
        self.stats["entries"] += 1
        self.stats["inserted"] += 1
        return True

    def evict_oldest(self) -> bool:
        if not self.entries:
            return False
        i = min(range(len(self.entries)), key=lambda j: self.entries[j]["used"])
        e = self.entries[i]
        self.entries[i] = self.entries[-1]
        self.entries.pop()
        self.stats["cost"] -= e["cost"]
        self.stats["entries"] -= 1
        self.stats["evicted"] += 1
        return True

    def clear(self):
        while self.evict_oldest():
            pass
