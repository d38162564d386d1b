"""Block bookkeeping: the names of crates/qubivex-runtime/src/discrete.rs:215-290, :951-1009
(KvPool, Mirror, AttnPlan, attention_plan) over the C ABI, plus sharing, copy-on-write and
compaction, which the reference lists as not built (docs/decisions/ADR-016-KV-SUBSYSTEM.md:82-89).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import Geometry, KvPoolStats
from .device import ptr

DEFAULT_KV_POOL = 512 << 20  # discrete.rs:210
MAX_KV_POOL = 1 << 30        # discrete.rs:213


def blocks_for(geo: Geometry, configured: int, budget_left: int, max_arena: int, uncapped: bool = False) -> int:
    """The pool's size rule, discrete.rs:429-455."""
    return _lib.load().qvx_kvpool_blocks_for(C.byref(geo), configured, budget_left, max_arena, int(uncapped))


def _arr(p, n) -> np.ndarray:
    return np.ctypeslib.as_array(p, shape=(n,)).copy() if n else np.zeros(0, dtype=np.uint32)


@dataclass
class AttnPlan:
    """discrete.rs:282-290, with the unsynced rows named by (sequence, position) and the copies
    copy-on-write asks for."""
    pos: np.ndarray
    blocks: np.ndarray
    table_at: np.ndarray
    sync_to: np.ndarray
    sync_seq: np.ndarray
    sync_pos: np.ndarray
    copy_src: np.ndarray
    copy_dst: np.ndarray
    handle: int


class Mirror:
    """One sequence's blocks in the pool (discrete.rs:257-280)."""

    def __init__(self, pool: "KvPool", handle: int):
        self.pool, self.h = pool, handle

    def blocks(self, layer: int) -> np.ndarray:
        lib = self.pool.lib
        n = lib.qvx_seq_blocks(self.h, layer, None, 0)
        out = np.zeros(n, dtype=np.uint32)
        lib.qvx_seq_blocks(self.h, layer, ptr(out), n)
        return out

    def synced(self, layer: int) -> int:
        return self.pool.lib.qvx_seq_synced(self.h, layer)

    def fork(self, tokens: int, epoch: int = 0) -> "Mirror":
        """A sequence sharing this one's blocks for positions 0..tokens; nothing is copied."""
        return Mirror(self.pool, self.pool.lib.qvx_seq_fork(self.h, tokens, epoch))

    def drop(self) -> None:
        if self.h:
            self.pool.lib.qvx_seq_delete(self.h)
            self.h = 0


class KvPool:
    """discrete.rs:227-243: the free list (LIFO, block 0 first) and, new here, reference counts."""

    def __init__(self, geo: Geometry, blocks: int):
        self.lib = _lib.load()
        self.geo = geo
        self.h = self.lib.qvx_kvpool_new(C.byref(geo), blocks)
        if not self.h:
            raise ValueError("a pool needs at least one block")

    def delete(self) -> None:
        if self.h:
            self.lib.qvx_kvpool_delete(self.h)
            self.h = 0

    def set_free_order(self, order) -> None:
        order = np.ascontiguousarray(order, dtype=np.uint32)
        if self.lib.qvx_kvpool_set_free_order(self.h, ptr(order), len(order)):
            raise ValueError("the order must list every free block once")

    def stats(self) -> KvPoolStats:
        s = KvPoolStats()
        self.lib.qvx_kvpool_stats_get(self.h, C.byref(s))
        return s

    def refcount(self, block: int) -> int:
        return self.lib.qvx_kvpool_refcount(self.h, block)

    def note_allocated(self, allocated: bool = True) -> None:
        self.lib.qvx_kvpool_note_allocated(self.h, int(allocated))

    def mirror(self, epoch: int = 0) -> Mirror:
        return Mirror(self, self.lib.qvx_seq_new(self.h, epoch))

    def attention_plan(self, seqs, pos, layer: int, epochs=None):
        """discrete.rs:951-1009.  None when the free list ran dry (the op is declined)."""
        s = len(seqs)
        hs = (C.c_void_p * s)(*[q.h for q in seqs])
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        ep = None if epochs is None else np.ascontiguousarray(epochs, dtype=np.uint64)
        out = C.c_void_p()
        rc = self.lib.qvx_plan_build(self.h, hs, ptr(ep), ptr(pos), s, layer, C.byref(out))
        if rc == 1:
            return None
        if rc:
            raise ValueError("a sequence of another pool")
        nb, ns, nc = C.c_size_t(), C.c_size_t(), C.c_size_t()
        n = self.lib.qvx_plan_counts(out, C.byref(nb), C.byref(ns), C.byref(nc))
        L = self.lib
        return AttnPlan(_arr(L.qvx_plan_pos(out), n), _arr(L.qvx_plan_blocks(out), nb.value),
                        _arr(L.qvx_plan_table_at(out), n), _arr(L.qvx_plan_sync_to(out), ns.value),
                        _arr(L.qvx_plan_sync_seq(out), ns.value), _arr(L.qvx_plan_sync_pos(out), ns.value),
                        _arr(L.qvx_plan_copy_src(out), nc.value), _arr(L.qvx_plan_copy_dst(out), nc.value), out.value)

    def commit(self, plan: AttnPlan, seqs, layer: int) -> None:
        """After the device ran the op: synced = pos + 1 (discrete.rs:929-943)."""
        hs = (C.c_void_p * len(seqs))(*[q.h for q in seqs])
        self.lib.qvx_plan_commit(self.h, plan.handle, hs, layer)

    def free_plan(self, plan: AttnPlan) -> None:
        if plan.handle:
            self.lib.qvx_plan_free(plan.handle)
            plan.handle = 0

    def compact(self):
        """Moves (src, dst) that gather the live blocks to ids 0..L; tables are rewritten."""
        cap = int(self.stats().blocks)
        src = np.zeros(cap, dtype=np.uint32)
        dst = np.zeros(cap, dtype=np.uint32)
        n = C.c_size_t()
        if self.lib.qvx_kvpool_compact(self.h, ptr(src), ptr(dst), cap, C.byref(n)):
            raise RuntimeError("compaction failed")
        return src[: n.value].copy(), dst[: n.value].copy()


class PrefixCache:
    """crates/qubivex-kv-cache/src/lib.rs:67-205 with Python objects as the values."""

    MIN_REUSE = 32

    def __init__(self, budget: int, on_release=None):
        self.lib = _lib.load()
        self._values: dict[int, object] = {}
        self._next = 1
        self._on_release = on_release

        def _release(value, _user):
            v = self._values.pop(value, None)
            if self._on_release is not None and v is not None:
                self._on_release(v)

        self._cb = _lib.RELEASE_FN(_release)
        self.h = self.lib.qvx_prefix_new(budget, self._cb, None)

    def delete(self) -> None:
        if self.h:
            self.lib.qvx_prefix_delete(self.h)
            self.h = 0

    def budget(self) -> int:
        return self.lib.qvx_prefix_budget(self.h)

    def stats(self):
        s = _lib.PrefixStats()
        self.lib.qvx_prefix_stats_get(self.h, C.byref(s))
        return s

    def cost(self) -> int:
        return int(self.stats().cost)

    def lookup(self, scope, prompt):
        """(value, reuse, hit) or None.  Release the hit when done with the value."""
        t = np.ascontiguousarray(prompt, dtype=np.uint32)
        value, reuse, hit = C.c_uint64(), C.c_size_t(), C.c_uint64()
        sc = None if scope is None else scope.encode()
        if not self.lib.qvx_prefix_lookup(self.h, sc, ptr(t), len(t), C.byref(value), C.byref(reuse), C.byref(hit)):
            return None
        return self._values[value.value], reuse.value, hit.value

    def release(self, hit: int) -> None:
        self.lib.qvx_prefix_hit_release(self.h, hit)

    def insert(self, scope, tokens, cost: int, value) -> bool:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        key = self._next
        self._next += 1
        self._values[key] = value
        sc = None if scope is None else scope.encode()
        return bool(self.lib.qvx_prefix_insert(self.h, sc, ptr(t), len(t), cost, key))

    def evict_oldest(self) -> bool:
        return bool(self.lib.qvx_prefix_evict_oldest(self.h))

    def clear(self) -> None:
        self.lib.qvx_prefix_clear(self.h)
