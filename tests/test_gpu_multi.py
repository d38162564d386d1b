"""Two GPUs of one box: the head-sharded division (configuration C5's) on real devices.  Each rank
holds the pool of its own KV heads, runs the decode op on them, and the per-head outputs are
all-gathered with NCCL; the result must equal the single-GPU result bit for bit (the same
per-head kernel with the same chunk boundaries ran in both)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    import torch
    import torch.distributed as dist

    from qubivex_b200 import device as qd
    from qubivex_b200 import sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    heads, kvh, d, B = 16, 2, 128, 16
    lengths = np.array([700, 33, 1500, 2049])
    rng = np.random.default_rng(17)  # every rank draws the same full problem
    nb = (lengths + B - 1) // B
    n_blocks = int(nb.sum()) + 4
    blocks = rng.permutation(n_blocks).astype(np.uint32)[: int(nb.sum())]
    table_at = np.concatenate([[0], np.cumsum(nb)[:-1]]).astype(np.uint32)
    pos = (lengths - 1).astype(np.uint32)
    kv_out = kvh * d
    s = len(lengths)
    q = rng.standard_normal((s, heads, d), dtype=np.float32)
    k_new = rng.standard_normal((s, kv_out), dtype=np.float32)
    v_new = rng.standard_normal((s, kv_out), dtype=np.float32)
    sync_to = np.array([int(blocks[table_at[t] + p // B]) * B + p % B for t in range(s) for p in range(int(pos[t]))], dtype=np.uint32)
    sync = rng.standard_normal((len(sync_to), 2 * kv_out), dtype=np.float32)

    def run(dev, n_kv, n_heads, q_, k_, v_, sync_):
        geo = qd.geometry(B, n_kv, d, qd.BF16)
        buf = dev.alloc(n_blocks * qd.block_bytes(geo))
        dev.write(buf, 0, np.zeros(n_blocks * qd.block_bytes(geo), dtype=np.uint8))
        out = dev.paged_attention(buf, geo, n_heads, q_, k_, v_, pos, blocks, table_at, sync_, sync_to, variant=qd.ATTN_SPLIT)
        buf.free()
        return out

    dev = qd.CudaDevice(rank)
    sh = sharding.head_shard(heads, kvh, d, rank, world)
    local = run(dev, sh.kv_heads, sh.heads, sh.q(q), sh.kv_rows(k_new, kvh), sh.kv_rows(v_new, kvh), sh.sync_rows(sync, kvh))
    full = sharding.all_gather_heads(torch.from_numpy(local).cuda()).cpu().numpy()
    if rank == 0:
        want = run(dev, kvh, heads, q, k_new, v_new, sync)
        np.save(os.path.join(out_dir, "ok.npy"), np.array([np.array_equal(full.view(np.uint32), want.view(np.uint32))]))
    dev.close()
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_decode_over_two_gpus_equals_one_gpu(tmp_path):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert bool(np.load(tmp_path / "ok.npy")[0])
