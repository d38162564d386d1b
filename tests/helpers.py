"""Shared by the parity tests: seeded cases, the oracle run and the device run of the same op."""
from __future__ import annotations

import numpy as np

import oracle
from qubivex_b200 import device as qd

DT = {"f32": 0, "bf16": 1, "f16": 2}
# The parity bars: max-abs 2e-3 plus max-rel 1e-2 for 16-bit KV, max-abs 1e-5 for f32.
TOL = {"f32": (1e-5, 0.0), "bf16": (2e-3, 1e-2), "f16": (2e-3, 1e-2)}


def within(got, want, dtype: str):
    """|got - want| <= atol + rtol * |want|, and the worst absolute error for the report."""
    atol, rtol = TOL[dtype]
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    ok = bool(np.all(err <= atol + rtol * np.abs(want)))
    return ok, float(err.max()) if err.size else 0.0


class Case:
    """A batch of sequences with prefilled contexts, one new token each."""

    def __init__(self, heads, kv_heads, d, B, dtype, lengths, seed=0, layout=1, amp_qk=1.0, amp_v=1.0,
                 pool_blocks=None, fill=0):
        self.heads, self.kvh, self.d, self.B, self.dtype = heads, kv_heads, d, B, dtype
        self.lengths = np.asarray(lengths, dtype=np.int64)  # positions held after this op (pos + 1)
        self.geo_o = oracle.geometry(B, kv_heads, d, DT[dtype], layout)
        self.geo_d = qd.geometry(B, kv_heads, d, DT[dtype], layout)
        self.bb = oracle.block_bytes(self.geo_o)
        nb = (self.lengths + B - 1) // B
        need = int(nb.sum())
        self.pool_blocks = pool_blocks or need + 3
        rng = np.random.default_rng(seed)
        perm = rng.permutation(self.pool_blocks).astype(np.uint32)
        self.table_at = np.zeros(len(lengths), dtype=np.uint32)
        self.table_at[1:] = np.cumsum(nb)[:-1]
        self.blocks = perm[:need].copy()
        self.pos = (self.lengths - 1).astype(np.uint32)
        s, kv_out = len(lengths), kv_heads * d
        self.q = (rng.standard_normal((s, heads, d), dtype=np.float32) * amp_qk).astype(np.float32)
        self.k_new = (rng.standard_normal((s, kv_out), dtype=np.float32) * amp_qk).astype(np.float32)
        self.v_new = (rng.standard_normal((s, kv_out), dtype=np.float32) * amp_v).astype(np.float32)
        # The prefilled context arrives as sync rows: every position before pos.
        sync_to, rows = [], []
        for t in range(s):
            for p in range(int(self.pos[t])):
                blk = int(self.blocks[self.table_at[t] + p // B])
                sync_to.append(blk * B + p % B)
        self.sync_to = np.array(sync_to, dtype=np.uint32)
        n = len(sync_to)
        self.sync = np.empty((n, 2 * kv_out), dtype=np.float32)
        self.sync[:, :kv_out] = rng.standard_normal((n, kv_out), dtype=np.float32) * amp_qk
        self.sync[:, kv_out:] = rng.standard_normal((n, kv_out), dtype=np.float32) * amp_v
        self.fill = fill

    def host_pool(self) -> np.ndarray:
        return np.full(self.pool_blocks * self.bb, self.fill, dtype=np.uint8)

    def run_oracle(self):
        pool = self.host_pool()
        rc, att = oracle.paged_attention(pool, self.geo_o, self.heads, self.q, self.k_new, self.v_new, self.pos,
                                         self.blocks, self.table_at, self.sync, self.sync_to)
        assert rc == 0
        return pool, att

    def run_device(self, dev, variant=qd.ATTN_AUTO):
        buf = dev.alloc(self.pool_blocks * self.bb)
        try:
            dev.write(buf, 0, self.host_pool())
            out = dev.paged_attention(buf, self.geo_d, self.heads, self.q, self.k_new, self.v_new, self.pos,
                                      self.blocks, self.table_at, self.sync, self.sync_to, variant=variant)
            pool = dev.read(buf, 0, self.pool_blocks * self.bb)
        finally:
            buf.free()
        return pool, out


class XorShift:
    """The reference's test generator (crates/qubivex-backend-vulkan/tests/attention_spike.rs:236-249)."""

    def __init__(self, seed: int):
        self.s = max((seed * 2654435761) & 0xFFFFFFFF, 1)

    def next(self) -> int:
        s = self.s
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        self.s = s
        return s

    def uni(self, a: float, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        for i in range(n):
            out[i] = (np.float32(self.next() >> 8) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0)) * np.float32(a)
        return out
