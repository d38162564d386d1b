"""Two GPUs of one box: the head-sharded division (configuration C5's) on real devices.  Each rank
holds the pool of its own KV heads, runs the decode op on them writing into its slot of the library's
gather buffer, and qvx_allgather_heads (ncclAllGather over NVLink + the transpose, behind the C ABI, device
memory only) assembles [token][head][d]; the result must equal the single-GPU result bit for bit (the same
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

    def run(dev, n_kv, n_heads, q_, k_, v_, sync_, out_ptr=None):
        """The op through the device-memory calls of the C ABI: sync rows, then append + attention.  With `out_ptr`
        the outputs go there (a rank's slot of the gather buffer); otherwise into a tensor that is returned."""
        import ctypes as C
        from qubivex_b200.device import ptr
        geo = qd.geometry(B, n_kv, d, qd.BF16)
        bb = qd.block_bytes(geo)
        pool = torch.zeros(n_blocks * bb, dtype=torch.uint8, device="cuda")
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        d_sync, d_to = to(sync_), to(sync_to.view(np.int32))
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        dev.check(dev.lib.qvx_kv_sync(dev.h, C.byref(geo), ptr(pool), n_blocks, ptr(d_sync), ptr(d_to), len(sync_to), stream))
        tabs = C.c_void_p()
        dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), n_blocks, n_heads, s, ptr(pos), ptr(blocks), len(blocks), ptr(table_at),
                                            C.byref(tabs)))
        out = None if out_ptr is not None else torch.empty((s, n_heads, d), device="cuda")
        d_k, d_v, d_q = to(k_), to(v_), to(q_)        # (named: a temporary's memory may be handed out again before the launch reads it)
        dev.check(dev.lib.qvx_kv_append_attn_decode(dev.h, tabs, ptr(pool), ptr(d_k), ptr(d_v), ptr(d_q),
                                                    C.c_void_p(out_ptr) if out_ptr is not None else ptr(out), qd.ATTN_SPLIT, stream))
        torch.cuda.synchronize()
        dev.lib.qvx_tables_free(tabs)
        return out

    dev = qd.CudaDevice(rank)
    sh = sharding.head_shard(heads, kvh, d, rank, world)
    # rank 0 makes the communicator's id; the host side hands it round (here: torch.distributed's own broadcast)
    box = [sharding.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    gather = sharding.HeadGather(dev, world, rank, box[0], max_tokens=s, heads_local=sh.heads, head_dim=d)
    run(dev, sh.kv_heads, sh.heads, sh.q(q), sh.kv_rows(k_new, kvh), sh.kv_rows(v_new, kvh), sh.sync_rows(sync, kvh),
        out_ptr=gather.send_slot(s))                         # attention writes straight into the send slot
    full = torch.empty((s, heads, d), device="cuda")
    import ctypes as C
    gather.all_gather(C.c_void_p(full.data_ptr()), s, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    # the same exchange over peer memory: every rank maps the others' result buffers, then stores and flags only
    mine = gather.peer_handle()
    handles = [None] * world
    dist.all_gather_object(handles, mine)
    gather.peer_open(handles)
    peer_ok = True
    for step in range(5):                                   # several in a row: the two result buffers alternate
        again = torch.full((s, heads, d), float(step), device="cuda")
        gather.all_gather(C.c_void_p(again.data_ptr()), s, C.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        peer_ok = peer_ok and torch.equal(again.view(torch.int32), full.view(torch.int32))
    dev.kernel_times()                                      # no bounded wait ran out
    if rank == 0:
        want = run(dev, kvh, heads, q, k_new, v_new, sync)
        same = torch.equal(full.view(torch.int32), want.view(torch.int32))
        np.save(os.path.join(out_dir, "ok.npy"), np.array([same, peer_ok]))
    gather.close()
    dev.close()
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_decode_over_two_gpus_equals_one_gpu(tmp_path):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    ok = np.load(tmp_path / "ok.npy")
    assert bool(ok[0]), "the NCCL gather differs from one GPU"
    assert bool(ok[1]), "the peer-memory gather differs from the NCCL gather"
