"""CUDA-event times of every kernel of the path on the benchmark configurations' shapes, through
the C ABI, with the algorithmic bytes each moves: `python -m qubivex_b200.measure.kernels [names]`.

  c2   one layer of the MoE-decoder shape (batch 64, contexts U[1024, 4096])
  c3   16 x 32768 positions, 8 sequences sharing an 8192-position prefix (shared blocks counted once)
  c4   32 q / 8 kv heads, block 32: one attention step over ~58k live blocks, and a compaction's moves
  c5   one GPU's share of the head-sharded shape (8 q / 1 kv head, batch 256, contexts U[1024, 16384])
  c1   the f32 reference-runnable shape (split and exact-order kernels)
  rows the sync / append kernel at prefill and decode sizes
  static  the fixed-scratch entry point (qvx_attn_decode_static) on the c2 launch
  f32  the f32 split kernel at size (batch 64, contexts U[1024, 4096], 8 q / 2 kv heads of 64)
  copy  block copies at a size a profiler can hold (1474 moves of 128 KiB in a 2 GiB pool)
  prelude  clip + Q/K norms + RoPE on 64 tokens of the MoE-decoder shape
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np
import torch

from .. import device as qd
from .. import workload as wl
from ..device import ptr

PEAK = 6540.5  # GB/s, measured copy bandwidth of the pool's B200s


def _tables(dev, geo, pool_blocks, heads, pos, blocks, table_at):
    t = C.c_void_p()
    dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), pool_blocks, heads, len(pos), ptr(pos), ptr(blocks), len(blocks),
                                        ptr(table_at), C.byref(t)))
    return t


def _time(dev, fn, kind, reps=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dev.reset_kernel_times()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    n, ns = dev.kernel_times()[kind]
    return ns / max(n, 1) * 1e-9


def _report(name, byts, sec):
    gbs = byts / sec / 1e9
    print(f"{name:58s} {byts / 2**20:9.1f} MiB {sec * 1e6:9.1f} us {gbs:8.0f} GB/s  {gbs / PEAK * 100:5.1f}% of measured  {gbs / 80:5.1f}% of 8000",
          flush=True)


def attention_case(dev, name, shape: wl.Shape, lengths, shared_prefix=0, sharers=0, variant=qd.ATTN_SPLIT, dtype=qd.BF16, seed=1):
    import dataclasses
    shape = dataclasses.replace(shape, dtype={qd.F32: "f32", qd.BF16: "bf16", qd.F16: "f16"}[dtype])  # (the bytes follow the pool's type)
    geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, dtype, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    B = shape.block_tokens
    lengths = np.asarray(lengths, dtype=np.int64)
    nb = (lengths + B - 1) // B
    pre_blocks = shared_prefix // B
    own = nb.copy()
    own[:sharers] -= pre_blocks
    pool_blocks = int(own.sum()) + pre_blocks + 8
    perm = wl.permutation(pool_blocks, seed)
    table_at = np.concatenate([[0], np.cumsum(nb)[:-1]]).astype(np.uint32)
    blocks = np.empty(int(nb.sum()), dtype=np.uint32)
    shared = perm[:pre_blocks]
    cur = pre_blocks
    for i in range(len(lengths)):
        lo = int(table_at[i])
        if i < sharers:
            blocks[lo:lo + pre_blocks] = shared
            blocks[lo + pre_blocks:lo + nb[i]] = perm[cur:cur + own[i]]
        else:
            blocks[lo:lo + nb[i]] = perm[cur:cur + own[i]]
        cur += int(own[i])
    e = 4 if dtype == qd.F32 else 2
    tdt = {qd.F32: torch.float32, qd.BF16: torch.bfloat16, qd.F16: torch.float16}[dtype]
    pool = (torch.randn(pool_blocks * bb // e, device="cuda") * wl.value_scale(shape)).to(tdt)
    s = len(lengths)
    q = torch.randn((s, shape.heads, shape.head_dim), device="cuda") * wl.value_scale(shape)
    out = torch.empty_like(q)
    pos = (lengths - 1).astype(np.uint32)
    t = _tables(dev, geo, pool_blocks, shape.heads, pos, blocks, table_at)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sec = _time(dev, lambda: dev.check(dev.lib.qvx_attn_decode(dev.h, t, ptr(pool), ptr(q), ptr(out), variant, stream)),
                "exact" if variant == qd.ATTN_EXACT else "attn", reps=20 if variant != qd.ATTN_EXACT else 3)
    unique = int(lengths.sum()) - (sharers - 1) * shared_prefix if sharers else int(lengths.sum())
    _report(name, wl.algorithmic_bytes(shape, lengths, unique_positions=unique), sec)
    dev.lib.qvx_tables_free(t)
    del pool


def static_case(dev, name, shape: wl.Shape, lengths, seed=1):
    """The fixed-scratch entry point (qvx_attn_decode_static) on the same kind of launch, timed with stream events."""
    geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, qd.BF16, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    B = shape.block_tokens
    lengths = np.asarray(lengths, dtype=np.int64)
    nb = (lengths + B - 1) // B
    pool_blocks = int(nb.sum()) + 8
    perm = wl.permutation(pool_blocks, seed)
    tabs = wl.tables_for(lengths, B, perm)
    pool = (torch.randn(pool_blocks * bb // 2, device="cuda") * wl.value_scale(shape)).to(torch.bfloat16)
    s = len(lengths)
    q = torch.randn((s, shape.heads, shape.head_dim), device="cuda") * wl.value_scale(shape)
    out = torch.empty_like(q)
    d_pos, d_blocks, d_at = (torch.from_numpy(a.astype(np.int32)).cuda() for a in (tabs.pos, tabs.blocks, tabs.table_at))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        dev.check(dev.lib.qvx_attn_decode_static(dev.h, C.byref(geo), ptr(pool), shape.heads, s, ptr(q), ptr(d_pos), ptr(d_blocks),
                                                 ptr(d_at), int(tabs.pos.max()), ptr(out), stream))
    for _ in range(3):
        call()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        call()
    e1.record()
    torch.cuda.synchronize()
    _report(name, wl.algorithmic_bytes(shape, lengths), e0.elapsed_time(e1) / 20 * 1e-3)


def rows_case(dev, name, shape: wl.Shape, n_rows, dtype=qd.BF16):
    geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, dtype, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    pool_blocks = n_rows // shape.block_tokens + 2
    pool = torch.empty(pool_blocks * bb, dtype=torch.uint8, device="cuda")
    rows = torch.randn((n_rows, 2 * shape.kv_out), device="cuda")
    # rows arrive in position order (a prefill's sync rows); their blocks are scattered over the pool
    B = shape.block_tokens
    block_of = np.random.default_rng(1).permutation(pool_blocks)[: (n_rows + B - 1) // B].astype(np.int64)
    row = np.arange(n_rows, dtype=np.int64)
    to = torch.from_numpy((block_of[row // B] * B + row % B).astype(np.int32)).cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sec = _time(dev, lambda: dev.check(dev.lib.qvx_kv_sync(dev.h, C.byref(geo), ptr(pool), pool_blocks, ptr(rows), ptr(to), n_rows, stream)), "sync")
    e = 4 if dtype == qd.F32 else 2
    _report(name, n_rows * 2 * shape.kv_out * (4 + e), sec)


def copy_case(dev, name, shape: wl.Shape, pool_blocks, moves):
    geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, qd.BF16, qd.LAYOUT_NATIVE)
    bb = qd.block_bytes(geo)
    pool = torch.empty(pool_blocks * bb, dtype=torch.uint8, device="cuda")
    perm = np.random.default_rng(2).permutation(pool_blocks).astype(np.int32)
    src = torch.from_numpy(perm[:moves].copy()).cuda()
    dst = torch.from_numpy(perm[moves:2 * moves].copy()).cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sec = _time(dev, lambda: dev.check(dev.lib.qvx_block_copy(dev.h, C.byref(geo), ptr(pool), pool_blocks, ptr(src), ptr(dst), moves, stream)), "copy")
    _report(name, 2 * moves * bb, sec)


def prelude_case(dev, name, shape: wl.Shape):
    from .._lib import Prelude
    geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, qd.BF16, qd.LAYOUT_NATIVE)
    s, d = shape.batch, shape.head_dim
    q = torch.randn((s, shape.heads, d), device="cuda")
    k = torch.randn((s, shape.kv_out), device="cuda")
    v = torch.randn((s, shape.kv_out), device="cuda")
    rope = torch.randn((s, d), device="cuda")
    qn, kn = torch.ones(shape.heads * d, device="cuda"), torch.ones(shape.kv_out, device="cuda")
    pre = Prelude(1, 8.0, qn.data_ptr(), kn.data_ptr(), 1e-6, rope.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sec = _time(dev, lambda: dev.check(dev.lib.qvx_attn_prelude(dev.h, C.byref(geo), shape.heads, s, ptr(q), ptr(k), ptr(v), C.byref(pre), stream)),
                "prelude")
    _report(name, 2 * 4 * s * (shape.heads * d + 2 * shape.kv_out) + 4 * s * d, sec)


def main(names):
    # QVX_MEASURE_EXPERIMENTS=1: the experiment build of the library (its chunk and order rules follow the environment)
    dev = qd.CudaDevice(0, timing=1, experiments=bool(os.environ.get("QVX_MEASURE_EXPERIMENTS")))
    rng = np.random.default_rng(7)
    if "c2" in names:
        attention_case(dev, "c2 attention: batch 64, ctx U[1024,4096], 32q/4kv, bf16, B16", wl.C2, rng.integers(1024, 4097, size=64))
    if "static" in names:
        static_case(dev, "c2 attention, fixed-scratch entry (20 launches back to back)", wl.C2, np.random.default_rng(7).integers(1024, 4097, size=64))
    if "c3" in names:
        attention_case(dev, "c3 attention: 16 x 32768, 8 share 8192, bf16, B16", wl.C3, [32768] * 16, shared_prefix=8192, sharers=8)
    if "c4" in names:
        lens = []
        while sum((n + 31) // 32 for n in lens) < 58982:  # 90 % of 65536 blocks
            lens.append(int(rng.integers(256, 8193)))
        attention_case(dev, f"c4 attention: {len(lens)} seqs U[256,8192], 32q/8kv, bf16, B32", wl.C4, lens)
        copy_case(dev, "c4 compaction: 5898 moves of 128 KiB in a 65536-block pool", wl.C4, 65536, 5898)
    if "c5" in names:
        one = wl.Shape("c5-one-gpu", 8, 1, 128, 16, "bf16", 256, 1024, 16384)
        attention_case(dev, "c5 attention, one GPU's head: batch 256, ctx U[1024,16384]", one, rng.integers(1024, 16385, size=256))
    if "c1" in names:
        attention_case(dev, "c1 split f32: 8q/2kv d64 B16, ctx 101/192/319/576", wl.C1, [101, 192, 319, 576], dtype=qd.F32)
        attention_case(dev, "c1 exact f32 (reference order)", wl.C1, [101, 192, 319, 576], dtype=qd.F32, variant=qd.ATTN_EXACT)
        big = wl.Shape("f32-big", 8, 2, 64, 16, "f32", 64, 1024, 4096)
        attention_case(dev, "split f32 at size: batch 64, ctx U[1024,4096], 8q/2kv d64", big, rng.integers(1024, 4097, size=64), dtype=qd.F32)
    if "f32" in names:
        big = wl.Shape("f32-big", 8, 2, 64, 16, "f32", 64, 1024, 4096)
        attention_case(dev, "split f32 at size: batch 64, ctx U[1024,4096], 8q/2kv d64", big, rng.integers(1024, 4097, size=64), dtype=qd.F32)
    if "f32c2" in names:
        attention_case(dev, "split f32, c2's shape: batch 64, ctx U[1024,4096], 32q/4kv d128", wl.C2, np.random.default_rng(7).integers(1024, 4097, size=64), dtype=qd.F32)
    if "copy" in names:
        copy_case(dev, "block copy: 1474 moves of 128 KiB in a 16384-block pool", wl.C4, 16384, 1474)
    if "prelude" in names:
        prelude_case(dev, "attention prelude: 64 tokens, 32q/4kv x 128 (clip, norms, RoPE)", wl.C2)
    if "rows" in names:
        rows_case(dev, "kv sync (prefill): 65536 rows, 4kv x 128, bf16", wl.C2, 65536)
        rows_case(dev, "kv append (decode): 64 rows, 4kv x 128, bf16", wl.C2, 64)
        rows_case(dev, "kv sync (prefill): 65536 rows, 8kv x 128, bf16, B32", wl.C4, 65536)
    dev.close()


if __name__ == "__main__":
    main(sys.argv[1:] or ["c2", "static", "c3", "c4", "c5", "c1", "rows"])
