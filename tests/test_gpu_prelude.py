"""The attention prelude (clip, full-width Q/K norms, RoPE) against the oracle's restatement of
SimDevice::attention's lines 333-357: f32 in, f32 out, bit for bit; then the whole stage."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import Case, within
from qubivex_b200 import device as qd
from qubivex_b200._lib import Prelude

pytestmark = pytest.mark.gpu


def rope_rows(rng, s, d):
    ang = rng.uniform(-np.pi, np.pi, size=(s, d // 2)).astype(np.float32)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


def run_device_prelude(dev, geo, heads, q, k, v, rope, clip, norms, eps):
    import torch

    s = k.shape[0]
    tq, tk, tv, tr = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (q, k, v, rope))
    tn = [torch.from_numpy(np.ascontiguousarray(n)).cuda() for n in norms] if norms else [None, None]
    pre = Prelude(0 if clip is None else 1, 0.0 if clip is None else clip, tn[0].data_ptr() if norms else None,
                  tn[1].data_ptr() if norms else None, eps, tr.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = dev.lib.qvx_attn_prelude(dev.h, C.byref(geo), heads, s, qd.ptr(tq), qd.ptr(tk), qd.ptr(tv), C.byref(pre), stream)
    dev.check(rc)
    torch.cuda.synchronize()
    return tq.cpu().numpy(), tk.cpu().numpy(), tv.cpu().numpy()


@pytest.mark.parametrize("heads,kvh,d", [(32, 4, 128), (8, 2, 64), (16, 16, 128), (4, 1, 96), (2, 2, 6), (64, 8, 128)])
@pytest.mark.parametrize("clip,norm", [(None, False), (0.75, False), (None, True), (2.5, True)])
def test_prelude_has_the_oracles_bits(dev, heads, kvh, d, clip, norm):
    rng = np.random.default_rng(heads * 1000 + d + (7 if norm else 0))
    s = 5
    q = rng.standard_normal((s, heads * d), dtype=np.float32) * 1.7
    k = rng.standard_normal((s, kvh * d), dtype=np.float32) * 1.7
    v = rng.standard_normal((s, kvh * d), dtype=np.float32) * 1.7
    # Rust's clamp keeps NaN and -0; infinities clip; tiny values survive the norm's products
    q[0, 1], q[1, 0], k[2, 3], v[0, 0], v[1, 1], k[0, 0] = -0.0, np.inf, -np.inf, -0.0, np.float32(1e-40), np.float32(-3e-39)
    if clip is not None and not norm:
        q[3, 2], v[4, 1] = np.nan, np.nan
    norms = (rng.standard_normal(heads * d, dtype=np.float32), rng.standard_normal(kvh * d, dtype=np.float32)) if norm else None
    rope = rope_rows(rng, s, d)
    eps = 1e-6
    wq, wk, wv = oracle.attn_prelude(q, k, v, heads, kvh, d, rope, clip=clip, qk_norm=norms, eps=eps)
    geo = qd.geometry(16, kvh, d, qd.F32, qd.LAYOUT_REFERENCE)
    gq, gk, gv = run_device_prelude(dev, geo, heads, q, k, v, rope, clip, norms, eps)
    for got, want in ((gq, wq), (gk, wk), (gv, wv)):
        got, want = got.reshape(-1), want.reshape(-1)
        # a NaN is a NaN on both sides (its payload is the hardware's business), everything else has the oracle's bits
        assert np.array_equal(np.isnan(got), np.isnan(want))
        m = ~np.isnan(want)
        assert np.array_equal(got[m].view(np.uint32), want[m].view(np.uint32))


def test_a_bad_prelude_is_refused(dev):
    geo = qd.geometry(16, 2, 64, qd.F32, qd.LAYOUT_REFERENCE)
    import torch

    x = torch.zeros(4 * 64, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for pre in (Prelude(1, -1.0, None, None, 1e-6, x.data_ptr()),            # clamp(-c, c) with c < 0
                Prelude(1, float("nan"), None, None, 1e-6, x.data_ptr()),
                Prelude(0, 0.0, x.data_ptr(), None, 1e-6, x.data_ptr()),     # one norm without the other
                Prelude(0, 0.0, None, None, 1e-6, None)):                    # no RoPE table
        rc = dev.lib.qvx_attn_prelude(dev.h, C.byref(geo), 4, 1, qd.ptr(x), qd.ptr(x), qd.ptr(x), C.byref(pre), stream)
        with pytest.raises(qd.ShapeError):
            dev.check(rc)


@pytest.mark.parametrize("dtype,layout,B", [("f32", 0, 256), ("bf16", 1, 16), ("f16", 1, 32)])
def test_the_whole_stage_from_raw_projections(dev, dtype, layout, B):
    # prelude -> sync rows -> new rows -> attention, host memory in and out
    heads, kvh, d = 16, 2, 128
    c = Case(heads, kvh, d, B, dtype, [1, 17, 300, 700], seed=17, layout=layout, amp_qk=0.6, amp_v=0.6)
    rng = np.random.default_rng(5)
    s = len(c.lengths)
    rope = rope_rows(rng, s, d)
    norms = (rng.standard_normal(heads * d, dtype=np.float32), rng.standard_normal(kvh * d, dtype=np.float32))
    clip, eps = 1.5, 1e-5
    q2, k2, v2 = oracle.attn_prelude(c.q, c.k_new, c.v_new, heads, kvh, d, rope, clip=clip, qk_norm=norms, eps=eps)
    pool = c.host_pool()
    rc, want = oracle.paged_attention(pool, c.geo_o, heads, q2, k2, v2, c.pos, c.blocks, c.table_at, c.sync, c.sync_to)
    assert rc == 0
    buf = dev.alloc(c.pool_blocks * c.bb)
    try:
        dev.write(buf, 0, c.host_pool())
        k_back, v_back = np.array(c.k_new, copy=True), np.array(c.v_new, copy=True)
        got = dev.attention_stage(buf, c.geo_d, heads, c.q, k_back, v_back, rope, c.pos, c.blocks, c.table_at, clip=clip,
                                  qk_norm=norms, eps=eps, sync=c.sync, sync_to=c.sync_to,
                                  variant=qd.ATTN_EXACT if dtype == "f32" else qd.ATTN_SPLIT)
        got_pool = dev.read(buf, 0, c.pool_blocks * c.bb)
    finally:
        buf.free()
    assert np.array_equal(k_back.view(np.uint32), k2.view(np.uint32))
    assert np.array_equal(v_back.view(np.uint32), v2.view(np.uint32))
    assert np.array_equal(got_pool, pool)
    if dtype == "f32":
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    else:
        ok, err = within(got, want, dtype)
        assert ok, err
