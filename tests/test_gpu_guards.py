"""The device-pointer entry points check block ids against the pool size the caller declares.

qvx_kv_sync, qvx_kv_append and qvx_block_copy read their block ids from device memory the host
side of the library never sees, so the kernels compare every id with `pool_blocks`: a row or a move
that names a block at or past it is skipped whole, and the device's status word makes the host's
next wait on the device fail with a message that says so.

Every case here is safe by construction: the buffer really holds N blocks, the call declares
N - 4, and the offending ids lie in [N - 4, N) — outside what the check allows, inside real memory.
"""
import ctypes as C

import numpy as np
import pytest

from qubivex_b200 import device as qd
from qubivex_b200.device import ptr

pytestmark = pytest.mark.gpu

N, GUARD = 24, 4


def _setup(torch, dtype=qd.BF16, B=16, kvh=2, d=64):
    geo = qd.geometry(B, kvh, d, dtype, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    pool = torch.full((N * bb,), 0x5A, dtype=torch.uint8, device="cuda")
    return geo, bb, pool


def _expect_out_of_pool(dev):
    with pytest.raises(qd.DeviceError, match="pool_blocks"):
        dev.kernel_times()
    dev.kernel_times()  # reported once


def _tail_untouched(pool, bb):
    tail = pool[(N - GUARD) * bb:]
    assert bool((tail == 0x5A).all())


@pytest.mark.parametrize("dtype", [qd.BF16, qd.F32])
def test_sync_rows_for_blocks_past_the_declared_pool_are_skipped(dev, dtype):
    torch = pytest.importorskip("torch")
    geo, bb, pool = _setup(torch, dtype)
    B, kv_out = geo.block_tokens, geo.kv_heads * geo.head_dim
    blocks = np.array([1, N - 1, 3, N - GUARD, N - 2], dtype=np.uint32)      # three of five past the declared end
    sync_to = torch.from_numpy((blocks * B + np.arange(5, dtype=np.uint32)).view(np.int32)).cuda()
    rows = torch.randn((5, 2 * kv_out), device="cuda")
    dev.check(dev.lib.qvx_kv_sync(dev.h, C.byref(geo), ptr(pool), N - GUARD, ptr(rows), ptr(sync_to), 5, None))
    torch.cuda.synchronize()
    _tail_untouched(pool, bb)
    head = pool[:(N - GUARD) * bb].view(-1, bb)
    assert bool((head[1] != 0x5A).any()) and bool((head[3] != 0x5A).any())     # the rows inside the pool were written
    _expect_out_of_pool(dev)
    # the same call with the true size writes all five
    dev.check(dev.lib.qvx_kv_sync(dev.h, C.byref(geo), ptr(pool), N, ptr(rows), ptr(sync_to), 5, None))
    torch.cuda.synchronize()
    dev.kernel_times()
    assert bool((pool[(N - 1) * bb:] != 0x5A).any())


@pytest.mark.parametrize("layout", [qd.LAYOUT_NATIVE, qd.LAYOUT_REFERENCE])
def test_appended_rows_for_blocks_past_the_declared_pool_are_skipped(dev, layout):
    torch = pytest.importorskip("torch")
    geo, bb, pool = _setup(torch)
    geo.layout = layout
    bb = qd.block_bytes(geo)
    pool = torch.full((N * bb,), 0x5A, dtype=torch.uint8, device="cuda")
    B, kv_out = geo.block_tokens, geo.kv_heads * geo.head_dim
    # two sequences of one block each: the second one's table names a block past the declared end
    pos = torch.tensor([5, 9], dtype=torch.int32, device="cuda")
    blocks = torch.tensor([2, N - 3], dtype=torch.int32, device="cuda")
    table_at = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    k = torch.randn((2, kv_out), device="cuda")
    v = torch.randn((2, kv_out), device="cuda")
    dev.check(dev.lib.qvx_kv_append(dev.h, C.byref(geo), ptr(pool), N - GUARD, ptr(k), ptr(v), ptr(pos), ptr(blocks), ptr(table_at), 2, None))
    torch.cuda.synchronize()
    _tail_untouched(pool, bb)
    assert bool((pool[2 * bb:3 * bb] != 0x5A).any())
    _expect_out_of_pool(dev)


def test_moves_that_name_a_block_past_the_declared_pool_are_skipped(dev):
    torch = pytest.importorskip("torch")
    geo, bb, pool = _setup(torch)
    pool.view(-1, bb)[0] = 1
    pool.view(-1, bb)[N - 1] = 2
    src = torch.tensor([0, 0, N - 1], dtype=torch.int32, device="cuda")        # into the tail, inside, out of the tail
    dst = torch.tensor([N - 2, 5, 6], dtype=torch.int32, device="cuda")
    dev.check(dev.lib.qvx_block_copy(dev.h, C.byref(geo), ptr(pool), N - GUARD, ptr(src), ptr(dst), 3, None))
    torch.cuda.synchronize()
    rows = pool.view(-1, bb)
    assert bool((rows[N - 2] == 0x5A).all())      # not written
    assert bool((rows[5] == 1).all())             # the move inside the pool happened
    assert bool((rows[6] == 0x5A).all())          # a source past the end is not read either
    _expect_out_of_pool(dev)


def test_a_bounded_wait_that_runs_out_is_reported_and_the_device_recovers(monkeypatch):
    """Every wait in the attention kernel is bounded.  A test build of the library (bounded waits of 4096 polls,
    and a hook that loses one chunk's publication) shows what happens when one runs out: the chunk that
    finishes the sequence waits for an entry that never comes, gives up by itself, the launch ends, the host
    call reports it, and the next op on the same device is right again."""
    from helpers import Case, within
    dev = qd.CudaDevice(0, experiments="short_waits")
    try:
        c = Case(8, 2, 128, 16, "bf16", [1300, 600], seed=77, amp_qk=0.4)       # sequence 0: three chunks, one merge node
        _, want = c.run_oracle()
        _, got = c.run_device(dev, variant=qd.ATTN_SPLIT)                      # the test build itself computes correctly
        assert within(got, want, "bf16")[0]
        monkeypatch.setenv("QVX_TEST_LOSE_A_PUBLICATION", "1")
        with pytest.raises(qd.DeviceError, match="gave up a bounded wait"):
            c.run_device(dev, variant=qd.ATTN_SPLIT)
        monkeypatch.delenv("QVX_TEST_LOSE_A_PUBLICATION")
        _, again = c.run_device(dev, variant=qd.ATTN_SPLIT)                    # counters and queue were reset with the report
        assert within(again, want, "bf16")[0]
        dev.kernel_times()
    finally:
        dev.close()
