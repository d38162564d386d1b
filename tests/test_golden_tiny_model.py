"""The reference's own golden vectors for attention: `fixtures/oracle/forward.json`, transformers'
f32 per-layer attention outputs for the tiny fixture models, which the reference checks at 1e-5
relative (crates/qubivex-runtime/tests/oracle.rs:18-40).  tests/golden/tiny_attention.npz holds the
slice of those fixtures the attention stage needs (made by tests/golden/make_tiny_attention.py).

The stage is rebuilt around the path under test: input RMSNorm, Q/K/V projections, OLMoE's
full-width q/k norms, NeoX RoPE, then *paged decode attention one position at a time* (each prompt
token is a decode step: its row is appended, then it attends 0..=p), then the O projection.
On the CPU the path is the oracle (this pins the oracle); on the GPU it is the CUDA backend in the
reference's layout and block size (KV_BLOCK = 256, f32), which must also match the oracle bit for bit.
"""
from pathlib import Path

import numpy as np
import pytest

import oracle

G = np.load(Path(__file__).resolve().parent / "golden" / "tiny_attention.npz")
TOL = 1e-5  # max |ours - ref| / max |ref| per tensor, as the reference's test
KV_BLOCK = 256


def rel(ours, want):
    return float(np.abs(ours.astype(np.float64) - want.astype(np.float64)).max() / max(np.abs(want).max(), 1e-30))


def rms_rows(x, w, eps):
    out = np.array(x, dtype=np.float32, copy=True)
    w = np.ascontiguousarray(w, dtype=np.float32)
    for r in out:
        oracle.lib().qvo_rms_norm(r.ctypes.data, w.ctypes.data, r.size, float(eps))
    return out


def rope_rows(x, heads, d, theta):
    """NeoX pairs (i, i + d/2), table row [cos.., sin..] per position: math::rope_rotate."""
    out = np.array(x, dtype=np.float32, copy=True).reshape(x.shape[0], heads, d)
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))).astype(np.float32)
    for p in range(out.shape[0]):
        f = (np.float32(p) * inv).astype(np.float32)
        cs = np.concatenate([np.cos(f), np.sin(f)]).astype(np.float32)
        for h in range(heads):
            oracle.lib().qvo_rope_rotate(out[p, h].ctypes.data, cs.ctypes.data, d)
    return out.reshape(x.shape[0], heads * d)


def oracle_decode(heads, kvh, d, q, k, v):
    """T decode steps of one sequence through the paged pool, on the CPU oracle."""
    T = q.shape[0]
    geo = oracle.geometry(KV_BLOCK, kvh, d, oracle.F32, oracle.LAYOUT_REFERENCE)
    pool = np.zeros(2 * oracle.block_bytes(geo), dtype=np.uint8)
    out = np.zeros((T, heads, d), dtype=np.float32)
    for p in range(T):
        rc, att = oracle.paged_attention(pool, geo, heads, q[p:p + 1].reshape(1, heads, d), k[p:p + 1], v[p:p + 1], [p], [1], [0])
        assert rc == 0
        out[p] = att[0]
    return out, pool


def rope_table(T, d, theta):
    """One row [cos.., sin..] per position, as the host hands it to the device (DeviceMoeAttention::rope)."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))).astype(np.float32)
    rows = np.empty((T, d), dtype=np.float32)
    for p in range(T):
        f = (np.float32(p) * inv).astype(np.float32)
        rows[p] = np.concatenate([np.cos(f), np.sin(f)])
    return rows


def attention_stage(name, layer, decode, stage=None):
    """`decode` takes normed, rotated q / k / v; `stage`, if given, takes the raw projections with the
    norm weights and the RoPE table instead (the prelude is then part of what is under test)."""
    hidden, heads, kvh, d, _ = (int(x) for x in G[f"{name}/meta"])
    eps, theta = (float(x) for x in G[f"{name}/eps_theta"])
    x = G[f"{name}/embed"] if layer == 0 else G[f"{name}/{layer - 1}/hidden"]
    key = f"{name}/{layer}/"
    h = rms_rows(x, G[key + "input_layernorm"], eps)
    q = (h @ G[key + "q_proj"].T).astype(np.float32)
    k = (h @ G[key + "k_proj"].T).astype(np.float32)
    v = (h @ G[key + "v_proj"].T).astype(np.float32)
    if stage is not None:
        norms = (G[key + "q_norm"], G[key + "k_norm"]) if key + "q_norm" in G else None
        att = stage(heads, kvh, d, q, k, v, rope_table(q.shape[0], d, theta), norms, eps)
    else:
        if key + "q_norm" in G:
            q, k = rms_rows(q, G[key + "q_norm"], eps), rms_rows(k, G[key + "k_norm"], eps)
        q, k = rope_rows(q, heads, d, theta), rope_rows(k, kvh, d, theta)
        att = decode(heads, kvh, d, q, k, v)
    return (att.reshape(att.shape[0], heads * d) @ G[key + "o_proj"].T).astype(np.float32), G[key + "attention"]


def oracle_stage(heads, kvh, d, q, k, v, rope, norms, eps):
    """The oracle's prelude (clip none, the model's norms, RoPE), then its paged decode."""
    q2, k2, v2 = oracle.attn_prelude(q, k, v, heads, kvh, d, rope, qk_norm=norms, eps=eps)
    return oracle_decode(heads, kvh, d, q2.reshape(-1, heads * d), k2, v2)[0]


CASES = [("dense-tiny", 0), ("dense-tiny", 1), ("olmoe-tiny", 0), ("olmoe-tiny", 1)]


@pytest.mark.parametrize("name,layer", CASES)
def test_the_oracle_reproduces_the_references_attention_outputs(name, layer):
    ours, want = attention_stage(name, layer, lambda *a: oracle_decode(*a)[0])
    assert rel(ours, want) <= TOL, rel(ours, want)


@pytest.mark.parametrize("name,layer", CASES)
def test_the_oracles_prelude_reproduces_them_too(name, layer):
    ours, want = attention_stage(name, layer, None, stage=oracle_stage)
    assert rel(ours, want) <= TOL, rel(ours, want)
    plain, _ = attention_stage(name, layer, lambda *a: oracle_decode(*a)[0])
    assert np.array_equal(ours.view(np.uint32), plain.view(np.uint32))  # one prelude call = norm rows, then rotate rows


@pytest.mark.gpu
@pytest.mark.parametrize("name,layer", CASES)
def test_the_cuda_stage_with_its_prelude_reproduces_them(dev, name, layer):
    from qubivex_b200 import device as qd

    def device_stage(heads, kvh, d, q, k, v, rope, norms, eps):
        geo = qd.geometry(KV_BLOCK, kvh, d, qd.F32, qd.LAYOUT_REFERENCE)
        n = 2 * qd.block_bytes(geo)
        buf = dev.alloc(n)
        dev.write(buf, 0, np.zeros(n, dtype=np.uint8))
        T = q.shape[0]
        out = np.zeros((T, heads, d), dtype=np.float32)
        k_back, v_back = np.array(k, copy=True), np.array(v, copy=True)
        for p in range(T):
            out[p] = dev.attention_stage(buf, geo, heads, q[p:p + 1], k_back[p:p + 1], v_back[p:p + 1], rope[p:p + 1], [p], [1], [0],
                                         qk_norm=norms, eps=eps)[0]
        q2, k2, v2 = oracle.attn_prelude(q, k, v, heads, kvh, d, rope, qk_norm=norms, eps=eps)
        want_att, want_pool = oracle_decode(heads, kvh, d, q2.reshape(-1, heads * d), k2, v2)
        assert np.array_equal(k_back.view(np.uint32), k2.view(np.uint32))       # the rows the host cache keeps
        assert np.array_equal(v_back.view(np.uint32), v2.view(np.uint32))
        assert np.array_equal(out.view(np.uint32), want_att.view(np.uint32))
        assert np.array_equal(dev.read(buf, 0, n), want_pool)
        buf.free()
        return out

    ours, want = attention_stage(name, layer, None, stage=device_stage)
    assert rel(ours, want) <= TOL, rel(ours, want)


@pytest.mark.gpu
@pytest.mark.parametrize("name,layer", CASES)
def test_the_cuda_backend_reproduces_them_in_the_references_layout(dev, name, layer):
    from qubivex_b200 import device as qd

    got_pool = {}

    def device_decode(heads, kvh, d, q, k, v):
        geo = qd.geometry(KV_BLOCK, kvh, d, qd.F32, qd.LAYOUT_REFERENCE)
        n = 2 * qd.block_bytes(geo)
        buf = dev.alloc(n)
        dev.write(buf, 0, np.zeros(n, dtype=np.uint8))
        out = np.zeros((q.shape[0], heads, d), dtype=np.float32)
        for p in range(q.shape[0]):
            out[p] = dev.paged_attention(buf, geo, heads, q[p:p + 1].reshape(1, heads, d), k[p:p + 1], v[p:p + 1], [p], [1], [0])[0]
        got_pool["bytes"] = dev.read(buf, 0, n)
        want_att, want_pool = oracle_decode(heads, kvh, d, q, k, v)
        assert np.array_equal(out.view(np.uint32), want_att.view(np.uint32))   # the bits of math::attend
        assert np.array_equal(got_pool["bytes"], want_pool)
        buf.free()
        return out

    ours, want = attention_stage(name, layer, device_decode)
    assert rel(ours, want) <= TOL, rel(ours, want)
