"""The runtime's side of device attention: the part of `OnDevice::routed_moe`
(crates/qubivex-runtime/src/discrete.rs:840-945) that owns the KV pool, plans the block
tables, lists the host rows the device does not hold, offers the op to the device and records
what the pool holds afterwards.  The projections and the MoE layer itself are the stages before and
after this path and are not here; clip, Q/K norms and RoPE run on the device when the caller hands
over the raw projections with a `prelude`.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .device import ATTN_AUTO, CudaDevice, DeviceBuffer, OutOfDeviceMemory, block_bytes
from .kvpool import KvPool, Mirror, PrefixCache, blocks_for


@dataclass
class AttnSeq:
    """crates/qubivex-compute/src/lib.rs:338-355: one decode sequence, one new token at `pos`."""
    mirror: Mirror | None
    host_k: np.ndarray  # [kv_head][position][head_dim] f32: the host cache's keys of 0..pos
    host_v: np.ndarray
    pos: int
    epoch: int = 0


@dataclass
class Retained:
    """What the prefix index keeps of a finished conversation.  The reference's value is the whole host cache
    (`PrefixCache<KvCache>`, crates/qubivex-runtime/src/engine.rs:1684-1699) and a hit copies it; its stated plan
    for paged KV is that the value "would be a set of pages, and a hit would share pages copy-on-write instead
    of copying them" (docs/decisions/ADR-016-KV-SUBSYSTEM.md:82-89).  This is that value: the sequence's blocks in
    the pool (a `Mirror`, reference-counted) and the host cache's rows, which stay the authority the pool can be
    resynced from."""
    mirror: Mirror
    host_k: np.ndarray   # [kv_head][position][head_dim]
    host_v: np.ndarray
    tokens: int          # positions the entry covers


class OnDevice:
    def __init__(self, device: CudaDevice, geo, heads: int, budget_left: int | None = None, uncapped: bool = False,
                 blocks: int | None = None):
        self.device, self.geo, self.heads = device, geo, heads
        if blocks is None:
            budget = device.usage().capacity - device.usage().used if budget_left is None else budget_left
            blocks = blocks_for(geo, device.kv_pool() or 0, budget, device.max_arena(), uncapped)
        self.kv = KvPool(geo, blocks) if blocks > 0 else None
        self._buffer: DeviceBuffer | None = None
        self._refused = False
        self.routed = 0
        self.retained: PrefixCache | None = None

    def close(self) -> None:
        if self.retained is not None:
            self.retained.clear()      # every retained sequence gives its blocks back
            self.retained.delete()
            self.retained = None
        if self._buffer is not None:
            self._buffer.free()
            self._buffer = None
        if self.kv is not None:
            self.kv.delete()
            self.kv = None

    def kv_buffer(self) -> DeviceBuffer | None:
        """discrete.rs:502-512: allocated on first use; None when the device refused the memory."""
        if self._buffer is None and not self._refused and self.kv is not None:
            try:
                self._buffer = self.device.alloc(int(self.kv.stats().blocks) * block_bytes(self.geo))
                self.kv.note_allocated(True)
            except OutOfDeviceMemory:
                self._refused = True
        return self._buffer

    def new_mirror(self, epoch: int = 0) -> Mirror:
        return self.kv.mirror(epoch)

    def attention(self, seqs: list[AttnSeq], layer: int, q, k_new, v_new, variant: int = ATTN_AUTO, prelude: dict | None = None):
        """The attention stage of one layer for one decode pass.  Returns the outputs
        [token][head][d], or None when declined (no pool, no memory, or no free block: the
        caller runs attention on the host, discrete.rs:870-891).  With `prelude`
        (rope=..., clip=..., qk_norm=..., eps=...: DeviceMoeAttention's fields) q, k_new and v_new are the
        raw projections, and k_new / v_new (float32 arrays) come back clipped, normed and rotated for the
        host cache."""
        if self.kv is None:
            return None
        buf = self.kv_buffer()
        if buf is None:
            return None
        for sq in seqs:
            if sq.mirror is None or sq.mirror.pool is not self.kv:
                sq.mirror = self.new_mirror(sq.epoch)  # a mirror made for another pool is replaced (:961-973)
        mirrors = [sq.mirror for sq in seqs]
        plan = self.kv.attention_plan(mirrors, [sq.pos for sq in seqs], layer, epochs=[sq.epoch for sq in seqs])
        if plan is None:
            return None
        try:
            kv_out = self.geo.kv_heads * self.geo.head_dim
            d = self.geo.head_dim
            sync = np.empty((len(plan.sync_to), 2 * kv_out), dtype=np.float32)
            for r, (si, p) in enumerate(zip(plan.sync_seq, plan.sync_pos)):
                sq = seqs[int(si)]
                sync[r, :kv_out] = sq.host_k[:, int(p), :].reshape(-1)  # per KV head, position p (:1000-1004)
                sync[r, kv_out:] = sq.host_v[:, int(p), :].reshape(-1)
            if len(plan.copy_src):
                self.device.block_copy(buf, self.geo, plan.copy_src, plan.copy_dst)
            if prelude is not None:
                out = self.device.attention_stage(buf, self.geo, self.heads, q, k_new, v_new, prelude["rope"], plan.pos, plan.blocks,
                                                  plan.table_at, clip=prelude.get("clip"), qk_norm=prelude.get("qk_norm"),
                                                  eps=prelude.get("eps", 1e-6), sync=sync, sync_to=plan.sync_to, variant=variant)
            else:
                out = self.device.paged_attention(buf, self.geo, self.heads, q, k_new, v_new, plan.pos, plan.blocks,
                                                  plan.table_at, sync, plan.sync_to, variant=variant)
            self.kv.commit(plan, mirrors, layer)
            self.routed += 1
            self.last_plan = plan
            return out
        finally:
            self.kv.free_plan(plan)

    # -- prefix reuse over shared blocks (Engine::restore / Engine::retain, engine.rs:1659-1699) --------------
    def retain_prefixes(self, budget_blocks: int) -> PrefixCache:
        """Turns prefix reuse on: finished sequences are kept, up to `budget_blocks` blocks of the pool in all
        (an entry's cost is the blocks it holds; the index evicts the oldest entries beyond the budget,
        crates/qubivex-kv-cache/src/lib.rs:146-199).  An evicted entry's blocks go back to the free list once
        the last hit on it has been released -- except those a forked sequence still shares."""
        self.retained = PrefixCache(budget_blocks, on_release=lambda kept: kept.mirror.drop())
        return self.retained

    def retain(self, scope: str | None, tokens, mirror: Mirror, host_k: np.ndarray, host_v: np.ndarray) -> bool:
        """Engine::retain: the finished sequence moves into the index (no copy); the caller lets go of `mirror`.
        False when the index did not keep it (over budget, or an entry already covers it): its blocks are
        released at once."""
        if self.retained is None:
            mirror.drop()
            return False
        layers = 0
        cost = 0
        while True:
            n = len(mirror.blocks(layers))
            if n == 0:
                break
            cost += n
            layers += 1
        n_tok = len(tokens)
        return self.retained.insert(scope, tokens, cost, Retained(mirror, host_k[:, :n_tok].copy(), host_v[:, :n_tok].copy(), n_tok))

    def restore(self, scope: str | None, prompt, host_k: np.ndarray, host_v: np.ndarray, epoch: int = 0):
        """Engine::restore: the longest retained prefix of `prompt` in `scope`, if any.  Returns
        (mirror, reuse): a new sequence that SHARES the blocks holding positions 0..reuse of the retained one
        (a table copy and reference counts: no KV byte moves; the first append into a shared, partly filled
        block copies that block, see KvPool.attention_plan), and the host cache's first `reuse` rows copied
        into host_k / host_v (the host cache stays authoritative, as KvCache::restore_from keeps it,
        crates/qubivex-arch/src/lib.rs:409-432).  (None, 0) on a miss."""
        if self.retained is None:
            return None, 0
        found = self.retained.lookup(scope, prompt)
        if found is None:
            return None, 0
        kept, reuse, hit = found
        try:
            mirror = kept.mirror.fork(reuse, epoch)
            host_k[:, :reuse] = kept.host_k[:, :reuse]
            host_v[:, :reuse] = kept.host_v[:, :reuse]
        finally:
            self.retained.release(hit)   # the fork holds its own references: the entry may be evicted from now on
        return mirror, reuse
