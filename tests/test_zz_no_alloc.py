"""qvx_attn_decode_static, the entry point that allocates nothing.

Some hosts of this backend hand the whole device to the KV pool up front and account for every
byte of it; they cannot let the library malloc scratch in the middle of a decode step.  This
entry point keeps its scratch in a fixed array inside the library instead.  The test calls it
through the C ABI twice in a row on different inputs (the second call finds the array as the
first left it) and checks both results against the ordinary entry point, qvx_attn_decode, on
the same pool — within the tolerance the other attention tests use.

The file sorts last on purpose: a run that stops at the first failure has then run every other
test.  It builds its own device and pool, so it passes alone in a fresh process as well.
"""
import ctypes as C

import numpy as np
import pytest

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
    return got.cpu().numpy(), want.cpu().numpy()


def _close(got, want):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(np.isfinite(got))
    assert np.all(err <= 2e-3 + 1e-2 * np.abs(want)), float(err.max())
    return float(err.max())


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    torch = pytest.importorskip("torch")
    dev = qd.CudaDevice(0)
    try:
        # first call: sequences of one chunk and of several, a ragged tail, a single position
        got, want = _case(dev, torch, 1, [1, 17, 511, 512, 513, 1300, 4096], first_launch=True)
        _close(got, want)
        # second call at once, other shapes: it finds the array as the first call left it
        got, want = _case(dev, torch, 2, [2048, 700, 33, 3000], heads=16, kvh=4, d=64, B=32, dtype=qd.F16, first_launch=True)
        _close(got, want)
        got, want = _case(dev, torch, 3, [900, 1025], heads=8, kvh=2)
        _close(got, want)
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
