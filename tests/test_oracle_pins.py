"""Pins the CPU oracle to the reference's own known-answer tests before anything trusts it.

Each test restates one test of the reference (cited) against oracle/qvx_oracle.c.
"""
import math

import numpy as np
import pytest

import oracle


def bits(x) -> int:
    return int(np.float32(x).view(np.uint32))


# crates/qubivex-compute/src/math.rs:215-228 (exp_edges)
def test_exp_edges():
    assert oracle.exp_bits(0.0) == bits(1.0)
    assert oracle.exp_bits(-0.0) == bits(1.0)
    assert math.isnan(oracle.exp(float("nan")))
    assert oracle.exp(float("inf")) == float("inf")
    assert oracle.exp_bits(float("-inf")) == 0
    assert oracle.exp(100.0) == float("inf")
    assert oracle.exp_bits(-100.0) == 0
    assert oracle.exp_bits(-87.5) == 0, "subnormal results are zero"
    assert oracle.exp(88.7) < float("inf")
    assert oracle.exp(-87.3365) >= np.finfo(np.float32).tiny
    assert abs(oracle.exp(1.0) - np.float32(math.e)) <= np.finfo(np.float32).eps * 4.0


# crates/qubivex-compute/src/math.rs:196-213 (exp_is_within_two_ulp_over_the_normal_range):
# the same walk, x += max(|x| * 1e-5, 1e-6) in f32, millions of points.
def test_exp_is_within_two_ulp_over_the_normal_range():
    xs = []
    x = np.float32(-87.33655)
    hi = np.float32(88.72284)
    # The walk itself is sequential in f32; generate it in chunks with numpy scalars.
    buf = np.empty(5_000_000, dtype=np.float32)
    n = 0
    e5, e6 = np.float32(1e-5), np.float32(1e-6)
    while x < hi:
        buf[n] = x
        n += 1
        x = np.float32(x + max(np.float32(abs(x) * e5), e6))
    xs = buf[:n]
    got = oracle.exp_array(xs)
    want64 = np.exp(xs.astype(np.float64))
    ok = (want64 >= float(np.finfo(np.float32).tiny)) & (want64 <= float(np.finfo(np.float32).max))
    want = want64[ok].astype(np.float32)
    g = got[ok]
    ulps = np.abs(g.view(np.uint32).astype(np.int64) - want.view(np.uint32).astype(np.int64))
    assert n > 1_000_000
    assert int(ulps.max()) <= 2, f"worst error {int(ulps.max())} ulp"


# crates/qubivex-arch/src/ops.rs:301-310
def test_attention_of_one_position_is_its_value():
    q = np.ones(4, dtype=np.float32)
    k = np.full(4, 0.5, dtype=np.float32)
    v = np.array([2.0, -1.0, 0.0, 3.0], dtype=np.float32)
    out = oracle.attend(q, k, v, 0)
    assert out.tolist() == v.tolist()


# crates/qubivex-arch/src/ops.rs:312-318
def test_softmax_sums_to_one():
    x = oracle.softmax([1.0, 2.0, 3.0, 1000.0])
    assert abs(float(x.sum(dtype=np.float32)) - 1.0) < 1e-6
    assert x[3] > 0.999


# crates/qubivex-compute/src/reduce.rs:53-73
def test_dot_matches_f64_and_handles_tails():
    for n in [0, 1, 31, 32, 63, 64, 65, 100, 128, 1000, 2048]:
        w = np.array([((i * 37 % 101) - 50.0) / 64.0 for i in range(n)], dtype=np.float32)
        x = np.array([((i * 53 % 97) - 48.0) / 32.0 for i in range(n)], dtype=np.float32)
        want = float(np.dot(w.astype(np.float64), x.astype(np.float64)))
        got = float(oracle.reduce_dot(w, x))
        assert abs(got - want) <= 1e-5 * max(abs(want), 1.0), f"n={n}: {got} vs {want}"


# crates/qubivex-compute/src/discrete.rs:247-256, :317-329: the pool's address function at the
# reference's own block size, written out from its definition.
def test_reference_layout_is_kv_key_word_and_kv_value_word():
    KV_BLOCK = 256
    for kvh, d in [(16, 128), (2, 32), (4, 16)]:
        geo = oracle.geometry(KV_BLOCK, kvh, d, oracle.F32, oracle.LAYOUT_REFERENCE)
        kv_out = kvh * d
        block_words = 2 * KV_BLOCK * kv_out
        assert oracle.block_bytes(geo) == 4 * block_words
        rng = np.random.default_rng(kvh * 1000 + d)
        for _ in range(200):
            at = int(rng.integers(0, 5 * KV_BLOCK))
            g, i = int(rng.integers(0, kvh)), int(rng.integers(0, d))
            b, slot = divmod(at, KV_BLOCK)
            key_word = b * block_words + (g * d + i) * KV_BLOCK + slot
            value_word = b * block_words + KV_BLOCK * kv_out + slot * kv_out + g * d + i
            assert oracle.elem_offset(geo, at, 0, g, i) == 4 * key_word
            assert oracle.elem_offset(geo, at, 1, g, i) == 4 * value_word


# kv_sync.comp:36-50 addresses a row the same way: keys strided by the block size, values contiguous.
def test_reference_layout_rows_as_kv_sync_writes_them():
    geo = oracle.geometry(256, 2, 32, oracle.F32, oracle.LAYOUT_REFERENCE)
    at = 3 * 256 + 17
    k0 = oracle.elem_offset(geo, at, 0, 0, 0)
    assert [oracle.elem_offset(geo, at, 0, 0, i) - k0 for i in range(4)] == [0, 1024, 2048, 3072]
    v0 = oracle.elem_offset(geo, at, 1, 0, 0)
    assert [oracle.elem_offset(geo, at, 1, g, i) - v0 for g in range(2) for i in range(3)] == [0, 4, 8, 128, 132, 136]


def test_native_layout_is_a_bijection_and_rows_are_contiguous():
    for dtype, d in [(oracle.F32, 64), (oracle.BF16, 128), (oracle.F16, 64), (oracle.BF16, 256)]:
        B, kvh = 16, 2
        geo = oracle.geometry(B, kvh, d, dtype, oracle.LAYOUT_NATIVE)
        e = 4 if dtype == oracle.F32 else 2
        bb = oracle.block_bytes(geo)
        assert bb == 2 * B * kvh * d * e
        seen = set()
        for at in range(2 * B):
            for kv in (0, 1):
                for g in range(kvh):
                    offs = [oracle.elem_offset(geo, at, kv, g, i) for i in range(d)]
                    lo = min(offs)
                    assert lo % (d * e) == 0 and max(offs) - lo == (d - 1) * e  # one contiguous row
                    seen.update(offs)
        assert len(seen) == 2 * B * 2 * kvh * d and max(seen) == 2 * bb - e


def test_native_layout_needs_128_byte_rows():
    assert not oracle.lib().qvo_geometry_ok(oracle.geometry(16, 2, 16, oracle.F32, oracle.LAYOUT_NATIVE))
    assert oracle.lib().qvo_geometry_ok(oracle.geometry(16, 2, 16, oracle.F32, oracle.LAYOUT_REFERENCE))


# crates/qubivex-backend-cpu/src/formats.rs:76-80: bf16 widens as bits << 16.
def test_bf16_widening_is_a_shift():
    h = np.arange(0, 65536, 7, dtype=np.uint16)
    w = oracle.widen(h, oracle.BF16)
    assert np.array_equal(w.view(np.uint32), h.astype(np.uint32) << 16)


def test_narrowing_rounds_to_nearest_even_like_an_independent_converter():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    x = np.concatenate([
        rng.standard_normal(200_000).astype(np.float32),
        (rng.standard_normal(50_000) * 1e-6).astype(np.float32),
        (rng.standard_normal(50_000) * 1e5).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65519.9, 65520.0, 1e-8, 6e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                  3.4e38, -3.4e38, 1.0 + 2**-8, 1.0 + 2**-9, 1.0 + 3 * 2**-9], dtype=np.float32)])
    got = oracle.narrow(x, oracle.BF16)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    with np.errstate(over="ignore"):
        want16 = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.narrow(x, oracle.F16), want16)
    # and back
    assert np.array_equal(oracle.widen(want16, oracle.F16), want16.view(np.float16).astype(np.float32))


def test_narrowing_keeps_a_nans_sign_and_quiets_it():
    nan_pos = np.array([0x7f800001, 0x7fc00000, 0x7fffffff], dtype=np.uint32).view(np.float32)
    nan_neg = np.array([0xff800001, 0xffc00000], dtype=np.uint32).view(np.float32)
    for dt, quiet, sign in [(oracle.BF16, 0x0040, 0x8000), (oracle.F16, 0x0200, 0x8000)]:
        p, n = oracle.narrow(nan_pos, dt), oracle.narrow(nan_neg, dt)
        assert np.all(np.isnan(oracle.widen(p, dt))) and np.all(np.isnan(oracle.widen(n, dt)))
        assert np.all(p & quiet) and np.all(n & quiet)
        assert not np.any(p & sign) and np.all(n & sign)
