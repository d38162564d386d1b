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
from .kvpool import KvPool, Mirror, blocks_for


@dataclass
class AttnSeq:
    """crates/qubivex-compute/src/lib.rs:338-355: one decode sequence, one new token at `pos`."""
    mirror: Mirror | None
    host_k: np.ndarray  # [kv_head][position][head_dim] f32: the host cache's keys of 0..pos
    host_v: np.ndarray
    pos: int
    epoch: int = 0


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

    def close(self) -> None:
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
