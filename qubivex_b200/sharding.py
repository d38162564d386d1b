"""How the path is divided over the GPUs of one box: by sequence, or by KV head.

Attention of one (token, head) needs nothing from any other (crates/qubivex-arch/src/lib.rs:1304-1306),
and a GQA group shares its keys and values with no other group, so neither division puts a
collective inside the path.  Sharding by KV head needs one exchange after it: every rank holds
[token][its heads][d] and the caller wants [token][head][d] — an all-gather and a transpose.
The reference has a single device (crates/qubivex-runtime/src/engine.rs:1290); this is new.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def sequence_shard(n_sequences: int, rank: int, world: int) -> range:
    """The sequences rank `rank` owns: contiguous, sizes differing by at most one."""
    base, extra = divmod(n_sequences, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


@dataclass(frozen=True)
class HeadShard:
    """Rank `rank` owns `kv_heads` KV heads starting at `kv0`, and the query heads of their groups."""
    rank: int
    world: int
    kv0: int
    kv_heads: int
    head0: int
    heads: int
    head_dim: int

    def q(self, q: np.ndarray) -> np.ndarray:
        """[token][head][d] -> this rank's [token][local head][d], contiguous."""
        return np.ascontiguousarray(q[:, self.head0:self.head0 + self.heads, :])

    def kv_rows(self, rows: np.ndarray, total_kv_heads: int) -> np.ndarray:
        """[row][kv_out] -> this rank's [row][local kv_out] (key rows, value rows, k_new, v_new)."""
        r = rows.reshape(rows.shape[0], total_kv_heads, self.head_dim)
        return np.ascontiguousarray(r[:, self.kv0:self.kv0 + self.kv_heads, :]).reshape(rows.shape[0], -1)

    def sync_rows(self, sync: np.ndarray, total_kv_heads: int) -> np.ndarray:
        """[row][key row | value row] -> the same for this rank's KV heads."""
        kv_out = total_kv_heads * self.head_dim
        k, v = sync[:, :kv_out], sync[:, kv_out:]
        return np.ascontiguousarray(np.concatenate([self.kv_rows(k, total_kv_heads), self.kv_rows(v, total_kv_heads)], axis=1))


def head_shard(heads: int, kv_heads: int, head_dim: int, rank: int, world: int) -> HeadShard:
    if kv_heads % world != 0:
        raise ValueError(f"{kv_heads} KV heads do not divide over {world} ranks")
    per = kv_heads // world
    group = heads // kv_heads
    return HeadShard(rank, world, rank * per, per, rank * per * group, per * group, head_dim)


def merge_heads(gathered) -> np.ndarray:
    """[rank][token][local head][d] (what an all-gather leaves) -> [token][head][d]."""
    g = np.asarray(gathered)
    world, s, hl, d = g.shape
    return np.ascontiguousarray(g.transpose(1, 0, 2, 3).reshape(s, world * hl, d))


def comm_unique_id() -> bytes:
    """The 128-byte id rank 0 makes and hands to the other ranks (qvx_comm_unique_id)."""
    import ctypes as C

    from . import _lib
    buf = (C.c_uint8 * 128)()
    rc = _lib.load().qvx_comm_unique_id(buf)
    if rc:
        raise RuntimeError(_lib.load().qvx_last_error(None).decode())
    return bytes(buf)


class HeadGather:
    """The exchange of the head-sharded path behind the C ABI: this rank's attention launch writes into
    `send_slot(s)`; `all_gather` runs ncclAllGather over NVLink and the transpose to [token][head][d] on the
    given stream.  Device pointers throughout; nothing passes through the host."""

    def __init__(self, device, nranks: int, rank: int, unique_id: bytes | None, max_tokens: int, heads_local: int, head_dim: int):
        import ctypes as C
        self.device, self.nranks, self.rank = device, nranks, rank
        self.heads_local, self.head_dim = heads_local, head_dim
        self.h = C.c_void_p()
        idbuf = (C.c_uint8 * 128).from_buffer_copy(unique_id) if unique_id is not None else None
        device.check(device.lib.qvx_comm_init(device.h, nranks, rank, idbuf, max_tokens, heads_local, head_dim, C.byref(self.h)))

    def send_slot(self, s: int) -> int:
        p = self.device.lib.qvx_comm_send_slot(self.h, s, self.heads_local, self.head_dim)
        if not p:
            raise ValueError(f"{s} tokens are more than the gather buffer was made for")
        return p

    def all_gather(self, out_full_ptr, s: int, stream=None) -> None:
        self.device.check(self.device.lib.qvx_allgather_heads(self.device.h, self.h, out_full_ptr, s, self.heads_local, self.head_dim, stream))

    def peer_handle(self) -> bytes:
        """This rank's result buffers, described in 128 bytes for the other ranks (qvx_comm_peer_handle)."""
        import ctypes as C
        buf = (C.c_uint8 * 128)()
        self.device.check(self.device.lib.qvx_comm_peer_handle(self.h, buf))
        return bytes(buf)

    def peer_open(self, handles: list[bytes]) -> None:
        """Every rank's handle, in rank order (qvx_comm_peer_open): from now on all_gather goes over peer memory."""
        import ctypes as C
        blob = b"".join(handles)
        self.device.check(self.device.lib.qvx_comm_peer_open(self.h, (C.c_uint8 * len(blob)).from_buffer_copy(blob)))
        self.over_peer_memory = True

    over_peer_memory = False

    def close(self) -> None:
        if self.h:
            self.device.lib.qvx_comm_destroy(self.h)
            self.h = None


def all_gather_heads(out_local, group=None):
    """The same exchange through torch.distributed (gloo on CPU ranks: the tests of the slicing and the
    transpose that need no GPU): all-gather of this rank's [token][local head][d] tensor, then the
    transpose to [token][head][d].  Every rank gets the whole result."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    gathered = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    dist.all_gather(list(gathered.unbind(0)), out_local.contiguous(), group=group)
    s, hl, d = out_local.shape
    return gathered.permute(1, 0, 2, 3).reshape(s, world * hl, d).contiguous()
