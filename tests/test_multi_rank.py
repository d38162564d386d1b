"""The N > 1 host logic on CPU ranks (gloo, world size 2): the KV-head sharding of configuration
C5 — slice queries and rows by head, attend locally, all-gather, transpose — must give the
unsharded result bit for bit; and the by-sequence division must cover every sequence once.
The per-rank arithmetic here is the CPU oracle (no GPU in this test)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from qubivex_b200 import sharding  # noqa: E402


def test_sequences_are_divided_once_and_evenly():
    for n, world in [(64, 8), (65, 8), (3, 4), (256, 2)]:
        parts = [sharding.sequence_shard(n, r, world) for r in range(world)]
        assert sorted(i for p in parts for i in p) == list(range(n))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1


def test_head_shards_tile_the_heads():
    sh = [sharding.head_shard(64, 8, 128, r, 8) for r in range(8)]
    assert [s.kv0 for s in sh] == list(range(8)) and [s.head0 for s in sh] == list(range(0, 64, 8))
    assert all(s.heads == 8 and s.kv_heads == 1 for s in sh)
    with pytest.raises(ValueError):
        sharding.head_shard(64, 8, 128, 0, 3)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch
    import torch.distributed as dist

    import oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    heads, kvh, d, B = 8, 4, 64, 16
    lengths = np.array([40, 17, 130])
    rng = np.random.default_rng(5)  # every rank draws the same full problem
    nb = (lengths + B - 1) // B
    blocks = rng.permutation(int(nb.sum()) + 2).astype(np.uint32)[: int(nb.sum())]
    table_at = np.concatenate([[0], np.cumsum(nb)[:-1]]).astype(np.uint32)
    pos = (lengths - 1).astype(np.uint32)
    kv_out = kvh * d
    q = rng.standard_normal((3, heads, d), dtype=np.float32)
    k_new = rng.standard_normal((3, kv_out), dtype=np.float32)
    v_new = rng.standard_normal((3, kv_out), dtype=np.float32)
    sync_to = np.array([int(blocks[table_at[t] + p // B]) * B + p % B for t in range(3) for p in range(int(pos[t]))], dtype=np.uint32)
    sync = rng.standard_normal((len(sync_to), 2 * kv_out), dtype=np.float32)
    # this rank's shard: its KV heads' pool, rows and queries
    sh = sharding.head_shard(heads, kvh, d, rank, world)
    geo = oracle.geometry(B, sh.kv_heads, d, oracle.BF16, oracle.LAYOUT_NATIVE)
    pool = np.zeros((int(nb.sum()) + 2) * oracle.block_bytes(geo), dtype=np.uint8)
    rc, local = oracle.paged_attention(pool, geo, sh.heads, sh.q(q), sh.kv_rows(k_new, kvh), sh.kv_rows(v_new, kvh), pos, blocks,
                                       table_at, sh.sync_rows(sync, kvh), sync_to)
    assert rc == 0
    full = sharding.all_gather_heads(torch.from_numpy(local)).numpy()
    if rank == 0:
        geo_all = oracle.geometry(B, kvh, d, oracle.BF16, oracle.LAYOUT_NATIVE)
        pool_all = np.zeros((int(nb.sum()) + 2) * oracle.block_bytes(geo_all), dtype=np.uint8)
        rc, want = oracle.paged_attention(pool_all, geo_all, heads, q, k_new, v_new, pos, blocks, table_at, sync, sync_to)
        assert rc == 0
        np.save(os.path.join(out_dir, "ok.npy"), np.array([np.array_equal(full.view(np.uint32), want.view(np.uint32))]))
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_attention_gathers_to_the_unsharded_result(tmp_path):
    torch = pytest.importorskip("torch")
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert bool(np.load(tmp_path / "ok.npy")[0])


def test_merge_heads_is_the_transpose_of_an_all_gather():
    g = np.arange(2 * 3 * 4 * 5, dtype=np.float32).reshape(2, 3, 4, 5)
    m = sharding.merge_heads(g)
    assert m.shape == (3, 8, 5)
    assert np.array_equal(m[1, 5], g[1, 1, 1]) and np.array_equal(m[2, 0], g[0, 2, 0])
