"""qvx_attn_decode_static, the entry point that allocates nothing.

Some hosts of this backend hand the whole device to the KV pool up front and account for every
byte of it; they cannot let the library malloc scratch in the middle of a decode step.  This
entry point keeps its scratch in a fixed array inside the library instead.  The test calls it
through the C ABI twice in a row on different inputs (the second call finds the array as the
first left it) and checks both results twice: against the CPU oracle on the same pool bytes,
within the tolerance the other attention tests use, and against the ordinary entry point,
qvx_attn_decode, much more tightly (the two kernels share their arithmetic and their chunks
and differ only in the order the chunks' results are merged in).

The file sorts last on purpose: a run that stops at the first failure has then run every other
test.  It builds its own device and pool, so it passes alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import within
from qubivex_b200 import device as qd
from qubivex_b200.device import ptr

pytestmark = pytest.mark.gpu


def _case(dev, torch, seed, lengths, heads=32, kvh=4, d=128, B=16, dtype=qd.BF16, first_launch=False):
    geo = qd.geometry(B, kvh, d, dtype, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    rng = np.random.default_rng(seed)
    lengths = np.asarray(lengths, dtype=np.int64)
    nb = (lengths + B - 1) // B
    pool_blocks = int(nb.sum()) + 5
    perm = rng.permutation(pool_blocks).astype(np.uint32)
    table_at = np.zeros(len(lengths), dtype=np.uint32)
    table_at[1:] = np.cumsum(nb)[:-1]
    blocks = perm[: int(nb.sum())].copy()
    pos = (lengths - 1).astype(np.uint32)
    g = torch.Generator(device="cuda").manual_seed(seed)
    tdt = torch.bfloat16 if dtype == qd.BF16 else torch.float16
    pool = torch.randn(pool_blocks * bb // 2, device="cuda", generator=g).to(tdt)
    q = torch.randn((len(lengths), heads, d), device="cuda", generator=g)
    # the ordinary entry point
    tabs = C.c_void_p()
    dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), pool_blocks, heads, len(lengths), ptr(pos), ptr(blocks), len(blocks),
                                        ptr(table_at), C.byref(tabs)))
    want = torch.empty_like(q)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    dev.check(dev.lib.qvx_attn_decode(dev.h, tabs, ptr(pool), ptr(q), ptr(want), qd.ATTN_SPLIT, stream))
    # the one that allocates nothing: the caller's own device arrays
    d_pos = torch.from_numpy(pos.view(np.int32)).cuda()
    d_blocks = torch.from_numpy(blocks.view(np.int32)).cuda()
    d_table_at = torch.from_numpy(table_at.view(np.int32)).cuda()
    got = torch.full_like(q, float("nan"))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = dev.lib.qvx_attn_decode_static(dev.h, C.byref(geo), ptr(pool), heads, len(lengths), ptr(q), ptr(d_pos), ptr(d_blocks),
                                        ptr(d_table_at), int(pos.max()), ptr(got), stream)
    dev.check(rc)
    torch.cuda.synchronize()
    # The driver's own count of free device memory: unchanged by the call.  (Not checked on a
    # kernel's first launch, when the driver loads its code and the array that comes with it.)
    if not first_launch:
        assert torch.cuda.mem_get_info()[0] >= free_before
    dev.kernel_times()  # reads the device status word: raises if the kernel refused anything
    dev.lib.qvx_tables_free(tabs)
    # the CPU oracle on the same pool bytes
    geo_o = oracle.geometry(B, kvh, d, dtype, oracle.LAYOUT_NATIVE)
    rc, ref = oracle.attn_decode(pool.view(torch.uint8).cpu().numpy(), geo_o, heads, q.cpu().numpy(), pos, blocks, table_at, threads=8)
    assert rc == 0
    return got.cpu().numpy(), want.cpu().numpy(), ref, "bf16" if dtype == qd.BF16 else "f16"


def _close(case):
    got, want, ref, dtype = case
    assert np.all(np.isfinite(got))
    ok, err = within(got, ref, dtype)           # the parity bar, against the oracle
    assert ok, err
    ok, err = within(want, ref, dtype)
    assert ok, err
    # against the ordinary entry point: same chunks, same arithmetic, another merge order
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(diff <= 2e-5 + 1e-4 * np.abs(want)), float(diff.max())


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    torch = pytest.importorskip("torch")
    dev = qd.CudaDevice(0)
    try:
        # first call: sequences of one chunk and of several, a ragged tail, a single position
        _close(_case(dev, torch, 1, [1, 17, 511, 512, 513, 575, 576, 577, 1300, 4096], first_launch=True))
        # second call at once, other shapes: it finds the array as the first call left it
        _close(_case(dev, torch, 2, [2048, 700, 33, 3000], heads=16, kvh=4, d=64, B=32, dtype=qd.F16, first_launch=True))
        _close(_case(dev, torch, 3, [900, 1025], heads=8, kvh=2))                 # groups of 4 query heads
        _close(_case(dev, torch, 4, [1500, 64, 513], heads=24, kvh=2))            # groups of 12: two head groups per KV head
    finally:
        dev.close()


def test_an_op_beyond_the_fixed_array_is_refused_with_its_sizes():
    torch = pytest.importorskip("torch")
    dev = qd.CudaDevice(0)
    try:
        geo = qd.geometry(16, 8, 128, qd.BF16, qd.LAYOUT_NATIVE)
        x = torch.zeros(1024, device="cuda")
        # 4096 sequences x 8 groups = 32768 (sequence, group) pairs: more than the 16384 counters
        rc = dev.lib.qvx_attn_decode_static(dev.h, C.byref(geo), ptr(x), 64, 4096, ptr(x), ptr(x), ptr(x), ptr(x), 4095, ptr(x), None)
        assert rc == -2
        msg = dev.lib.qvx_last_error(dev.h).decode()
        assert "16384" in msg and "qvx_attn_decode" in msg
        # 64 sequences x 8 groups x 64 chunks of partials: more than 16 MiB
        rc = dev.lib.qvx_attn_decode_static(dev.h, C.byref(geo), ptr(x), 64, 64, ptr(x), ptr(x), ptr(x), ptr(x), 32767, ptr(x), None)
        assert rc == -2 and "bytes of scratch" in dev.lib.qvx_last_error(dev.h).decode()
        f32 = qd.geometry(16, 2, 64, qd.F32, qd.LAYOUT_NATIVE)
        assert dev.lib.qvx_attn_decode_static(dev.h, C.byref(f32), ptr(x), 8, 1, ptr(x), ptr(x), ptr(x), ptr(x), 0, ptr(x), None) == -2
    finally:
        dev.close()


def test_a_position_beyond_the_callers_bound_is_refused_and_reported_once():
    """max_pos is the host's promise about pos[]; the scratch was sized by it.  A sequence that breaks it
    is left alone (the kernel returns before it touches memory), the device's status word says so, the
    host reports it at its next wait on the device — once — and the device is usable afterwards."""
    torch = pytest.importorskip("torch")
    dev = qd.CudaDevice(0)
    try:
        heads, kvh, d, B = 8, 2, 128, 16
        geo = qd.geometry(B, kvh, d, qd.BF16, qd.LAYOUT_NATIVE)
        bb = qd.block_bytes(geo)
        lengths = np.array([300, 1301], dtype=np.int64)          # the second breaks the bound below
        nb = (lengths + B - 1) // B
        pool = torch.randn(int(nb.sum()) * bb // 2, device="cuda").to(torch.bfloat16)
        q = torch.randn((2, heads, d), device="cuda")
        d_pos = torch.from_numpy((lengths - 1).astype(np.int32)).cuda()
        d_blocks = torch.arange(int(nb.sum()), dtype=torch.int32, device="cuda")
        d_table_at = torch.tensor([0, int(nb[0])], dtype=torch.int32, device="cuda")
        out = torch.full_like(q, 7.0)
        call = lambda max_pos: dev.lib.qvx_attn_decode_static(dev.h, C.byref(geo), ptr(pool), heads, 2, ptr(q), ptr(d_pos), ptr(d_blocks),
                                                              ptr(d_table_at), max_pos, ptr(out), None)
        assert call(511) == 0                                   # the launch itself is fine
        torch.cuda.synchronize()
        assert torch.all(out[1] == 7.0)                         # nothing written for the sequence past the bound
        assert not torch.any(out[0] == 7.0)                     # the one inside it was served
        with pytest.raises(qd.DeviceError, match="beyond the bound"):
            dev.kernel_times()
        dev.kernel_times()                                      # reported once: the word is clear again
        assert call(1300) == 0
        torch.cuda.synchronize()
        dev.kernel_times()
        assert not torch.any(out == 7.0)
    finally:
        dev.close()


def test_one_thread_may_drive_two_devices():
    """The kernels' shared-memory opt-in belongs to a device: a thread that opens two must get it on both."""
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU here")
    from helpers import Case
    for ordinal in (0, 1):
        dev = qd.CudaDevice(ordinal)
        try:
            with torch.cuda.device(ordinal):
                # (a device's first launch loads the kernel and the array that comes with it: no free-memory check)
                _close(_case(dev, torch, 5 + ordinal, [700, 1025], heads=8, kvh=2, first_launch=True))
            c = Case(8, 2, 64, 16, "f32", [600, 40, 1100], seed=7)   # the f32 split kernel's opt-in as well
            _, want = c.run_oracle()
            _, got = c.run_device(dev, variant=qd.ATTN_SPLIT)
            assert within(got, want, "f32")[0]
        finally:
            dev.close()
