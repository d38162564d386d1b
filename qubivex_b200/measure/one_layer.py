"""One layer of the MoE-decoder configuration: 25 launches of the decode-attention kernel through
the C ABI with its CUDA-event time.  The command ncu profiles (see profiles/).

Environment: BATCH, CTX (fixed context), BT (block tokens), PERM=seq|random."""
import ctypes as C
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from qubivex_b200 import device as qd
from qubivex_b200 import workload as wl
from qubivex_b200.device import ptr

shape = wl.C2
import dataclasses
shape = dataclasses.replace(shape, block_tokens=int(os.environ.get('BT', 16)))
batch = int(os.environ.get("BATCH", shape.batch))
seed = 1
dev = qd.CudaDevice(0, timing=True)
lib = dev.lib
geo = qd.geometry(shape.block_tokens, shape.kv_heads, shape.head_dim, qd.BF16, qd.LAYOUT_NATIVE)
bb = qd.block_bytes(geo)
rng = np.random.default_rng(seed)
lengths = rng.integers(shape.ctx_lo, shape.ctx_hi + 1, size=batch)
if os.environ.get('CTX'): lengths[:] = int(os.environ['CTX'])
nb = (lengths + shape.block_tokens - 1) // shape.block_tokens
pool_blocks = int(nb.sum()) + 64
perm = wl.permutation(pool_blocks, seed) if os.environ.get('PERM', 'random') == 'random' else np.arange(pool_blocks, dtype=np.uint32)
tabs = wl.tables_for(lengths, shape.block_tokens, perm)
pool = torch.empty(pool_blocks * bb, dtype=torch.uint8, device="cuda")
# fill: random bf16 bits straight (fast) -- values N(0,1)/sqrt(d)
vals = (torch.randn(pool_blocks * bb // 2, device="cuda") * (shape.head_dim ** -0.5)).to(torch.bfloat16)
pool.copy_(vals.view(torch.uint8))
del vals
q = (torch.randn(batch, shape.heads, shape.head_dim, device="cuda") * shape.head_dim ** -0.5)
out = torch.empty_like(q)
t = C.c_void_p()
dev.check(lib.qvx_tables_create(dev.h, C.byref(geo), pool_blocks, shape.heads, batch, ptr(tabs.pos), ptr(tabs.blocks),
                                len(tabs.blocks), ptr(tabs.table_at), C.byref(t)))
stream = torch.cuda.current_stream().cuda_stream
for variant in (qd.ATTN_SPLIT,):
    for it in range(5):
        dev.check(lib.qvx_attn_decode(dev.h, t, ptr(pool), ptr(q), ptr(out), variant, C.c_void_p(stream)))
    torch.cuda.synchronize()
    dev.reset_kernel_times()
    n = 20
    t0 = time.perf_counter()
    for it in range(n):
        dev.check(lib.qvx_attn_decode(dev.h, t, ptr(pool), ptr(q), ptr(out), variant, C.c_void_p(stream)))
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / n
    kt = dev.kernel_times()
    byts = wl.algorithmic_bytes(shape, lengths)
    a = kt["attn"][1] / kt["attn"][0] * 1e-9
    print(f"blocks={os.environ.get('PERM', 'random')} B={shape.block_tokens} batch={batch} bytes={byts / 2**20:.1f} MiB attn={a * 1e6:.1f} us "
          f"wall/iter={wall * 1e6:.1f} us -> attn {byts / a / 1e9:.0f} GB/s, wall {byts / wall / 1e9:.0f} GB/s")
dev.close()
