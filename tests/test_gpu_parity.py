"""Parity of the CUDA path with the CPU oracle, through the C ABI, on identical seeded inputs.

Bars: pool bytes bit-exact after sync / append / copies; exact-order attention bit-exact;
split attention within max-abs 1e-5 (f32) or 2e-3 + 1e-2 * |ref| (bf16 / f16).
"""
import numpy as np
import pytest

import oracle
from helpers import DT, Case, XorShift, within
from qubivex_b200 import device as qd

pytestmark = pytest.mark.gpu


def test_device_is_the_cuda_backend(dev):
    assert dev.name() == "cuda"
    assert "sm_100" in dev.describe() or "B200" in dev.describe()
    assert dev.supports(qd.BF16) and dev.supports(qd.F32) and dev.supports(qd.F16)
    assert dev.routes_moe_attention(64, 8, 1)


# ---- sync + append: pool bytes ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("layout,B,kvh,d", [(1, 16, 2, 64), (1, 32, 4, 128), (0, 256, 2, 32), (0, 16, 3, 24), (1, 16, 1, 256)])
def test_sync_and_append_leave_the_oracles_bytes(dev, dtype, layout, B, kvh, d):
    if layout == 1 and (d * (4 if dtype == "f32" else 2)) % 128:
        pytest.skip("native rows are multiples of 128 bytes")
    c = Case(kvh * 2, kvh, d, B, dtype, [1, B, B + 1, 3 * B - 1, 37], seed=11, layout=layout, fill=0xAB)
    want_pool, _ = c.run_oracle()
    got_pool, _ = c.run_device(dev, variant=qd.ATTN_EXACT)
    assert np.array_equal(got_pool, want_pool)


def test_a_later_duplicate_sync_row_wins(dev):
    c = Case(4, 2, 64, 16, "bf16", [40], seed=3)
    # The same position twice with different rows: list order decides (sim.rs:391-393).
    c.sync_to = np.concatenate([c.sync_to, c.sync_to[5:9]])
    extra = np.random.default_rng(5).standard_normal((4, c.sync.shape[1]), dtype=np.float32)
    c.sync = np.concatenate([c.sync, extra])
    want_pool, want = c.run_oracle()
    got_pool, got = c.run_device(dev)
    assert np.array_equal(got_pool, want_pool)
    assert within(got, want, "bf16")[0]


# ---- exact-order attention: bits ------------------------------------------------------------
@pytest.mark.parametrize("layout,B,heads,kvh,d,lengths", [
    (0, 256, 4, 2, 32, [1, 2, 250, 257, 300]),       # the reference's layout and block size, crossing a block
    (1, 16, 8, 2, 64, [37, 128, 255, 512]),           # C1's shape
    (0, 16, 4, 4, 16, [1, 16, 17, 100]),              # the tiny fixtures' head size
    (1, 32, 16, 16, 128, [139]),                      # OLMoE's heads
])
def test_exact_attention_has_the_oracles_bits_f32(dev, layout, B, heads, kvh, d, lengths):
    c = Case(heads, kvh, d, B, "f32", lengths, seed=21, layout=layout)
    want_pool, want = c.run_oracle()
    got_pool, got = c.run_device(dev, variant=qd.ATTN_EXACT)
    assert np.array_equal(got_pool, want_pool)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_exact_attention_has_the_oracles_bits_16bit_kv(dev, dtype):
    c = Case(8, 2, 64, 16, dtype, [1, 63, 200], seed=22)
    _, want = c.run_oracle()
    _, got = c.run_device(dev, variant=qd.ATTN_EXACT)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# The reference's kernel harness: shapes, (s, p0) cases and amplitudes of
# crates/qubivex-backend-vulkan/tests/attention_spike.rs:406-441, its xorshift generator.
@pytest.mark.parametrize("heads,kvh,d", [(16, 16, 128), (8, 2, 64), (4, 4, 96), (2, 1, 200)])
@pytest.mark.parametrize("amp", [1.0, 4.0, 30.0])
def test_exact_attention_on_the_references_harness_cases(dev, heads, kvh, d, amp):
    for p0 in (0, 1, 63, 64, 137, 1000):
        n = p0 + 1
        r = XorShift(7 + p0)
        q = r.uni(amp, heads * d).reshape(1, heads, d)
        k = r.uni(amp, n * kvh * d).reshape(n, kvh * d)
        v = r.uni(1.0, n * kvh * d).reshape(n, kvh * d)
        native_ok = (d * 4) % 128 == 0
        c = Case(heads, kvh, d, 16, "f32", [n], seed=1, layout=1 if native_ok else 0)
        c.q, c.k_new, c.v_new = q, k[-1:].copy(), v[-1:].copy()
        c.sync = np.concatenate([k[:-1], v[:-1]], axis=1).astype(np.float32)
        _, want = c.run_oracle()
        _, got = c.run_device(dev, variant=qd.ATTN_EXACT)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (heads, kvh, d, amp, p0)
        if native_ok and d in (64, 128):
            _, fast = c.run_device(dev, variant=qd.ATTN_SPLIT)
            ok, err = within(fast, want, "f32")
            # amplitude 30 makes scores of +-1e3: the tolerance is for N(0,1)-scale inputs
            assert ok or amp > 4.0, (heads, kvh, d, amp, p0, err)
            assert np.all(np.isfinite(fast))


def test_nan_and_inf_keys_follow_the_reference(dev):
    # attention_spike.rs feeds NaN / Inf keys: the maximum ignores NaN, the sum does not.
    c = Case(4, 2, 64, 16, "f32", [50], seed=9)
    c.sync[7, :64] = np.nan
    c.sync[9, 3] = np.inf
    _, want = c.run_oracle()
    _, got = c.run_device(dev, variant=qd.ATTN_EXACT)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    m = ~np.isnan(want)
    assert np.array_equal(got[m].view(np.uint32), want[m].view(np.uint32))


# ---- split attention: tolerance ---------------------------------------------------------------
@pytest.mark.parametrize("dtype,heads,kvh,d,B", [
    ("f32", 8, 2, 64, 16), ("f32", 4, 4, 128, 16), ("f32", 16, 2, 64, 32), ("f32", 2, 1, 64, 16),
    ("f32", 6, 2, 64, 16), ("f32", 10, 2, 128, 16), ("f32", 12, 1, 128, 32), ("f32", 7, 1, 64, 16),   # groups of 3, 5, 8 + 4, 7
    ("bf16", 32, 4, 128, 16), ("bf16", 32, 8, 128, 32), ("bf16", 8, 8, 64, 16), ("bf16", 24, 2, 128, 16),
    ("bf16", 8, 1, 256, 16), ("f16", 32, 4, 128, 16), ("f16", 4, 2, 64, 64), ("bf16", 64, 8, 128, 256),
])
def test_split_attention_is_within_tolerance(dev, dtype, heads, kvh, d, B):
    lengths = [1, 2, 15, 16, 17, 255, 256, 257, 511, 575, 576, 577, 700, 1023, 1152, 1153, 1500]
    c = Case(heads, kvh, d, B, dtype, lengths, seed=31, fill=0xFF)  # 0xFF bytes are NaNs: tails must be masked
    want_pool, want = c.run_oracle()
    got_pool, got = c.run_device(dev, variant=qd.ATTN_SPLIT)
    assert np.array_equal(got_pool, want_pool)
    ok, err = within(got, want, dtype)
    assert ok, f"max abs err {err}"
    assert np.all(np.isfinite(got))


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_long_contexts_take_larger_chunks_and_a_merge_tree(dev, dtype):
    # 20000, 40000 and 70000 positions: 1152-position chunks, 18, 35 and 61 of them (two levels of the fan-in-8
    # merge tree, the last with a second-level node of 8 entries).  577: two chunks.
    # 4700 and 9800: 9 and 18 chunks of 576, i.e. merge nodes of 8 + 1 and 8 + 8 + 2 entries.
    c = Case(8, 1, 128, 16, dtype, [20000, 40000, 70000, 577, 4700, 9800], seed=35, amp_qk=0.3)
    _, want = c.run_oracle()
    _, got = c.run_device(dev, variant=qd.ATTN_SPLIT)
    ok, err = within(got, want, dtype)
    assert ok, err
    assert err < (1e-4 if dtype == "bf16" else 1e-5)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_split_attention_with_scaled_inputs(dev, dtype):
    # The benchmark's distribution: values ~ N(0,1) / sqrt(d); outputs are small, so check
    # the relative error directly as well.
    d = 128
    c = Case(32, 4, d, 16, dtype, [1024, 2048, 3000, 4096], seed=41, amp_qk=d ** -0.5, amp_v=d ** -0.5)
    _, want = c.run_oracle()
    _, got = c.run_device(dev, variant=qd.ATTN_SPLIT)
    ok, err = within(got, want, dtype)
    assert ok, err
    scale = float(np.abs(want).max())
    assert err <= (1e-5 if dtype == "f32" else 2e-2 * scale)


def test_a_sequences_result_does_not_depend_on_its_batch(dev):
    # ADR-017 (docs/decisions/ADR-017-BATCHING.md:248-256): batch invariance, bit for bit.
    full = Case(32, 4, 128, 16, "bf16", [900, 300, 2047, 33, 1200], seed=51)
    _, out_full = full.run_device(dev, variant=qd.ATTN_SPLIT)
    for t in (0, 2, 3):
        alone = Case(32, 4, 128, 16, "bf16", [int(full.lengths[t])], seed=52, pool_blocks=full.pool_blocks)
        # the same sequence: same blocks, rows and query, alone in its op
        nb = (int(full.lengths[t]) + 15) // 16
        alone.blocks = full.blocks[full.table_at[t]:full.table_at[t] + nb].copy()
        alone.table_at[:] = 0
        alone.q, alone.k_new, alone.v_new = full.q[t:t + 1], full.k_new[t:t + 1], full.v_new[t:t + 1]
        lo = int(sum(int(x) - 1 for x in full.lengths[:t]))
        alone.sync = full.sync[lo:lo + int(full.lengths[t]) - 1]
        alone.sync_to = full.sync_to[lo:lo + int(full.lengths[t]) - 1]
        _, out_alone = alone.run_device(dev, variant=qd.ATTN_SPLIT)
        assert np.array_equal(out_alone[0].view(np.uint32), out_full[t].view(np.uint32))


# ---- validation: nothing written on a shape error (sim.rs:313-324, :359-376) ---------------------
def test_bad_inputs_are_refused_before_anything_is_written(dev):
    c = Case(8, 2, 64, 16, "f32", [20, 40], seed=61)
    buf = dev.alloc(c.pool_blocks * c.bb)
    zeros = c.host_pool()
    dev.write(buf, 0, zeros)
    args = lambda **kw: dict(dict(pool=buf, geo=c.geo_d, heads=c.heads, q=c.q, k_new=c.k_new, v_new=c.v_new,
                                  pos=c.pos, blocks=c.blocks, table_at=c.table_at, sync=c.sync, sync_to=c.sync_to), **kw)
    bad_blocks = c.blocks.copy(); bad_blocks[1] = c.pool_blocks
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(blocks=bad_blocks))                       # a block past the pool
    bad_sync = c.sync_to.copy(); bad_sync[0] = c.pool_blocks * 16
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(sync_to=bad_sync))                        # a sync row past the pool
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(pos=np.array([20, 400], dtype=np.uint32)))  # no block for the position
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(heads=7, q=c.q[:, :7].copy()))            # heads % kv_heads
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(k_new=c.k_new[:1]))                       # a short k_new
    fixed = dev.upload(zeros)
    with pytest.raises(qd.ShapeError):
        dev.paged_attention(**args(pool=fixed))                              # the pool is not an arena
    with pytest.raises(qd.DeviceError):
        dev.write(fixed, 0, zeros[:16])                                      # only an arena can be written
    with pytest.raises(qd.DeviceError):
        dev.write(buf, len(zeros) - 8, zeros[:16])                           # outside the buffer
    with pytest.raises(qd.Unsupported):                                      # native rows are 128-byte multiples
        dev.paged_attention(**args(geo=qd.geometry(16, 2, 16, qd.F32, qd.LAYOUT_NATIVE), q=c.q[:, :, :16].copy(),
                                   k_new=c.k_new[:, :32].copy(), v_new=c.v_new[:, :32].copy(),
                                   sync=c.sync[:, :64].copy()))
    assert np.array_equal(dev.read(buf, 0, len(zeros)), zeros)
    fixed.free()
    buf.free()


def test_capacity_is_enforced_and_freed(dev):
    # crates/qubivex-backend-cpu/src/sim.rs:721-876: capacity enforced, freed on drop, refusals counted.
    from qubivex_b200.device import CudaDevice
    small = CudaDevice(0, capacity=1 << 20)
    a = small.alloc(600_000)
    with pytest.raises(qd.OutOfDeviceMemory):
        small.alloc(600_000)
    u = small.usage()
    assert (u.capacity, u.used, u.refused) == (1 << 20, 600_000, 1)
    a.free()
    b = small.alloc(1 << 20)
    assert small.usage().used == 1 << 20 and small.usage().peak == 1 << 20
    b.free()
    assert small.usage().used == 0
    small.close()


# ---- block copies -------------------------------------------------------------------------------
@pytest.mark.parametrize("B,kvh,d,dtype,layout", [(16, 4, 128, "bf16", 1), (32, 8, 128, "bf16", 1), (3, 1, 5, "f32", 0)])
def test_block_copies_move_the_oracles_bytes(dev, B, kvh, d, dtype, layout):
    geo_o = oracle.geometry(B, kvh, d, {"f32": 0, "bf16": 1}[dtype], layout)
    geo_d = qd.geometry(B, kvh, d, {"f32": 0, "bf16": 1}[dtype], layout)
    n = 64
    bb = oracle.block_bytes(geo_o)
    rng = np.random.default_rng(71)
    host = rng.integers(0, 256, size=n * bb, dtype=np.uint8)
    perm = rng.permutation(n).astype(np.uint32)
    src, dst = perm[:20], perm[20:40]
    src = np.concatenate([src, [perm[41]]]).astype(np.uint32)  # a move onto itself is a no-op
    dst = np.concatenate([dst, [perm[41]]]).astype(np.uint32)
    want = host.copy()
    assert oracle.block_copy(want, geo_o, src, dst) == 0
    buf = dev.alloc(n * bb)
    dev.write(buf, 0, host)
    dev.block_copy(buf, geo_d, src, dst)
    assert np.array_equal(dev.read(buf, 0, n * bb), want)
    with pytest.raises(qd.ShapeError):
        dev.block_copy(buf, geo_d, [0, 1], [2, 2])      # written twice
    with pytest.raises(qd.ShapeError):
        dev.block_copy(buf, geo_d, [0, 1], [1, 2])      # read and written
    with pytest.raises(qd.ShapeError):
        dev.block_copy(buf, geo_d, [0], [n])            # past the pool
    buf.free()


def test_kernel_times_are_counted(dev):
    dev.reset_kernel_times()
    c = Case(32, 4, 128, 16, "bf16", [600, 100], seed=81)
    c.run_device(dev, variant=qd.ATTN_SPLIT)
    kt = dev.kernel_times()
    c32 = Case(8, 2, 64, 16, "f32", [600, 100], seed=82)
    c32.run_device(dev, variant=qd.ATTN_SPLIT)
    assert dev.kernel_times()["append"][0] == 0   # f32 native pool: the same kernel, the same fused append
    cref = Case(8, 2, 64, 16, "f32", [600, 100], seed=82, layout=qd.LAYOUT_REFERENCE)
    cref.run_device(dev)
    assert dev.kernel_times()["append"][0] == 1   # a pool in the reference's layout: the append is its own launch
    assert kt["sync"][0] == 1 and kt["attn"][0] == 1
    assert kt["append"][0] == 0   # native pool: the append rides in the attention launch
    assert kt["attn"][1] > 0
    t = dev.transfers()
    assert t.submissions >= 1 and t.activations_out >= c.q.nbytes and t.timed >= 2


def test_layers_back_to_back_with_the_pool_settled_flag_give_the_same_bits(dev):
    """Several layers' launches queued back to back, each told that its pool blocks are settled
    (so it may start under the tail of the launch before it), against the same launches one at
    a time: outputs and pool bytes must be identical."""
    torch = pytest.importorskip("torch")
    import ctypes as C
    from qubivex_b200.device import ptr
    heads, kvh, d, B, s, layers, steps = 32, 4, 128, 16, 12, 4, 3
    geo = qd.geometry(B, kvh, d, qd.BF16)
    bb = qd.block_bytes(geo)
    rng = np.random.default_rng(91)
    lengths = rng.integers(500, 1500, size=s)
    nb = (lengths + steps + B - 1) // B
    per_layer = int(nb.sum())
    perm = rng.permutation(per_layer * layers).astype(np.uint32)
    table_at = np.concatenate([[0], np.cumsum(nb)[:-1]]).astype(np.uint32)
    g = torch.Generator(device="cuda").manual_seed(5)
    pool0 = torch.randn(per_layer * layers * bb // 2, device="cuda", generator=g).to(torch.bfloat16)
    q = [torch.randn((s, heads, d), device="cuda", generator=g) for _ in range(steps)]
    kn = [torch.randn((s, kvh * d), device="cuda", generator=g) for _ in range(steps)]
    vn = [torch.randn((s, kvh * d), device="cuda", generator=g) for _ in range(steps)]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(flag, sync_each):
        pool = pool0.clone()
        outs = []
        tabs = []
        for t in range(steps):
            pos = (lengths + t).astype(np.uint32)
            for l in range(layers):
                tb = C.c_void_p()
                blocks = perm[l * per_layer:(l + 1) * per_layer].copy()
                dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), per_layer * layers, heads, s, ptr(pos), ptr(blocks), per_layer,
                                                    ptr(table_at), C.byref(tb)))
                tabs.append(tb)
        i = 0
        for t in range(steps):
            for l in range(layers):
                out = torch.empty((s, heads, d), device="cuda")
                dev.check(dev.lib.qvx_kv_append_attn_decode(dev.h, tabs[i], ptr(pool), ptr(kn[t]), ptr(vn[t]), ptr(q[t]), ptr(out),
                                                            qd.ATTN_SPLIT | flag, stream))
                if sync_each:
                    torch.cuda.synchronize()
                outs.append(out)
                i += 1
        torch.cuda.synchronize()
        dev.kernel_times()
        for tb in tabs:
            dev.lib.qvx_tables_free(tb)
        return torch.stack(outs).cpu().numpy(), pool.cpu().view(torch.int16).numpy()

    want_out, want_pool = run(0, True)
    got_out, got_pool = run(qd.ATTN_POOL_SETTLED, False)
    assert np.array_equal(got_pool, want_pool)
    assert np.array_equal(got_out.view(np.uint32), want_out.view(np.uint32))


def test_a_work_list_kept_from_the_previous_layer_gives_the_same_bits(dev):
    # The host op keeps its last work list: a second op with the same positions (the next layer:
    # other blocks, other rows) reuses it; other positions rebuild it.
    lengths = [700, 33, 2047, 1200, 16]
    a = Case(32, 4, 128, 16, "bf16", lengths, seed=71)
    b = Case(32, 4, 128, 16, "bf16", lengths, seed=72)
    nb = (b.lengths + 15) // 16  # its tables laid out in the opposite order
    b.table_at = (np.concatenate([[0], np.cumsum(nb[::-1])[:-1]])[::-1]).astype(np.uint32)
    sync_to = []
    for t in range(len(lengths)):
        for p in range(int(b.pos[t])):
            sync_to.append(int(b.blocks[b.table_at[t] + p // 16]) * 16 + p % 16)
    b.sync_to = np.array(sync_to, dtype=np.uint32)
    other = Case(32, 4, 128, 16, "bf16", [5, 900], seed=73)
    _, want_b = b.run_oracle()
    a.run_device(dev, variant=qd.ATTN_SPLIT)
    pool_hit, out_hit = b.run_device(dev, variant=qd.ATTN_SPLIT)      # same positions as a: reuse
    other.run_device(dev, variant=qd.ATTN_SPLIT)
    pool_miss, out_miss = b.run_device(dev, variant=qd.ATTN_SPLIT)    # after other positions: rebuilt
    assert np.array_equal(out_hit.view(np.uint32), out_miss.view(np.uint32))
    assert np.array_equal(pool_hit, pool_miss)
    ok, err = within(out_hit, want_b, "bf16")
    assert ok, err


def test_more_ops_in_flight_than_the_staging_ring_holds(dev):
    # 40 ops of ~2.3 MiB staged bytes each, submitted without a wait: the ring gives slices back as
    # the oldest ops finish.  Every op's output equals the same op run alone.
    c = Case(32, 4, 128, 16, "bf16", [300] * 64, seed=81)
    buf = dev.alloc(c.pool_blocks * c.bb)
    try:
        dev.write(buf, 0, c.host_pool())
        first = dev.paged_attention(buf, c.geo_d, c.heads, c.q, c.k_new, c.v_new, c.pos, c.blocks, c.table_at, c.sync, c.sync_to,
                                    variant=qd.ATTN_SPLIT)
        qs = [np.ascontiguousarray(c.q * (1.0 + 0.01 * i)) for i in range(40)]
        alone = [dev.paged_attention(buf, c.geo_d, c.heads, qs[i], c.k_new, c.v_new, c.pos, c.blocks, c.table_at, variant=qd.ATTN_SPLIT)
                 for i in range(40)]
        outs = [np.empty_like(first) for _ in range(40)]
        for i in range(40):
            dev.paged_attention(buf, c.geo_d, c.heads, qs[i], c.k_new, c.v_new, c.pos, c.blocks, c.table_at, out=outs[i],
                                variant=qd.ATTN_SPLIT, wait=False)
        dev.wait()
        for i in range(40):
            assert np.array_equal(outs[i].view(np.uint32), alone[i].view(np.uint32)), i
        assert np.array_equal(alone[0].view(np.uint32), first.view(np.uint32))
    finally:
        buf.free()


@pytest.mark.parametrize("dtype,variant", [("bf16", qd.ATTN_SPLIT), ("f32", qd.ATTN_SPLIT), ("f32", qd.ATTN_EXACT)])
def test_outputs_stored_straight_into_pinned_host_memory_have_the_staged_copys_bits(dev, dtype, variant):
    """A page-locked, aligned `out` is written by the kernel itself over the bus; pageable or misaligned memory
    takes the staged copy.  Same bits on every route, synchronous and queued, and right against the oracle."""
    torch = pytest.importorskip("torch")
    c = Case(8, 2, 64, 16, dtype, [1300, 37, 600, 16, 2049], seed=83)
    _, want = c.run_oracle()
    buf = dev.alloc(c.pool_blocks * c.bb)
    try:
        dev.write(buf, 0, c.host_pool())
        call = lambda **kw: dev.paged_attention(buf, c.geo_d, c.heads, c.q, c.k_new, c.v_new, c.pos, c.blocks, c.table_at, c.sync,
                                                c.sync_to, variant=variant, **kw)
        staged = call()                                                        # numpy's pageable memory
        shape = staged.shape
        pinned = torch.full(shape, float("nan"), dtype=torch.float32).pin_memory()
        call(out=pinned)
        assert np.array_equal(pinned.numpy().view(np.uint32), staged.view(np.uint32))
        queued = [torch.full(shape, float("nan"), dtype=torch.float32).pin_memory() for _ in range(3)]
        for o in queued:
            call(out=o, wait=False)
        dev.wait()
        for o in queued:
            assert np.array_equal(o.numpy().view(np.uint32), staged.view(np.uint32))
        # page-locked but 4 bytes off a 16-byte boundary: the staged route again
        wide = torch.full((staged.size + 4,), float("nan"), dtype=torch.float32).pin_memory()
        off = wide[1:1 + staged.size].view(shape)
        assert off.data_ptr() % 16 != 0
        call(out=off)
        assert np.array_equal(off.numpy().view(np.uint32), staged.view(np.uint32))
        assert torch.isnan(wide[0]) and bool(torch.isnan(wide[1 + staged.size:]).all())
        ok, err = within(staged, want, dtype) if variant != qd.ATTN_EXACT else (np.array_equal(staged.view(np.uint32), want.view(np.uint32)), "bits")
        assert ok, err
    finally:
        buf.free()


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_batch_invariance_when_ctas_stream_many_ragged_items(dev, dtype):
    # More (sequence, group) pairs than resident CTAs, lengths that are no multiple of anything:
    # every CTA streams several items, and most start at an arbitrary place of its tile stream.
    # A sequence's bits must still equal those it gets alone (one item, first in its CTA's stream).
    rng = np.random.default_rng(91)
    lengths = [int(x) for x in rng.integers(1, 900, size=360)]
    full = Case(32, 4, 128, 16, dtype, lengths, seed=92, amp_qk=0.3)
    _, out_full = full.run_device(dev, variant=qd.ATTN_SPLIT)
    assert np.all(np.isfinite(out_full))
    for t in (0, 7, 123, 359, int(np.argmax(full.lengths)), int(np.argmin(full.lengths))):
        n = int(full.lengths[t])
        alone = Case(32, 4, 128, 16, dtype, [n], seed=93, pool_blocks=full.pool_blocks)
        nb = (n + 15) // 16
        alone.blocks = full.blocks[full.table_at[t]:full.table_at[t] + nb].copy()
        alone.table_at[:] = 0
        alone.q, alone.k_new, alone.v_new = full.q[t:t + 1], full.k_new[t:t + 1], full.v_new[t:t + 1]
        lo = int(sum(int(x) - 1 for x in full.lengths[:t]))
        alone.sync = full.sync[lo:lo + n - 1]
        alone.sync_to = full.sync_to[lo:lo + n - 1]
        _, out_alone = alone.run_device(dev, variant=qd.ATTN_SPLIT)
        assert np.array_equal(out_alone[0].view(np.uint32), out_full[t].view(np.uint32)), t


@pytest.mark.parametrize("dtype,heads,kvh,d,B", [("bf16", 32, 4, 128, 16), ("f16", 8, 2, 64, 32), ("bf16", 8, 1, 256, 16),
                                                ("bf16", 24, 2, 128, 64), ("f32", 8, 2, 64, 16), ("f32", 16, 2, 128, 32)])
def test_runs_of_chunks_do_not_change_a_single_bit(dev, dev_x, monkeypatch, dtype, heads, kvh, d, B):
    # Work items are runs of consecutive chunks of a sequence; how long the runs are is the
    # scheduler's choice per op.  Every chunk keeps its own state, so the outputs must not move.
    lengths = [3000, 577, 2304, 1, 1729, 4096, 700, 2305] * 3
    c = Case(heads, kvh, d, B, dtype, lengths, seed=95, amp_qk=0.4)
    outs = {}
    for run in ("1", "2", "3", "4"):
        monkeypatch.setenv("QVX_RUN_CHUNKS", run)   # read by the experiment build only
        outs[run] = c.run_device(dev_x, variant=qd.ATTN_SPLIT)[1]
    monkeypatch.delenv("QVX_RUN_CHUNKS")
    outs["auto"] = c.run_device(dev, variant=qd.ATTN_SPLIT)[1]  # the shipped library, its own choice of runs
    for k, v in outs.items():
        assert np.array_equal(v.view(np.uint32), outs["1"].view(np.uint32)), k
    _, want = c.run_oracle()
    ok, err = within(outs["4"], want, dtype)
    assert ok, err


def test_a_step_appended_inside_a_run_lands_in_the_pool(dev_x, monkeypatch):
    # The fused append stores the step's new row from the item that ends the sequence; with runs that
    # item holds several chunks.  Pool bytes and outputs against the oracle, runs of 1 and of 4.
    import ctypes as C
    import torch
    lengths = [2500, 1153, 4096, 576, 577]
    c = Case(32, 4, 128, 16, "bf16", lengths, seed=97, amp_qk=0.4)
    want_pool, want = c.run_oracle()
    for run in ("1", "4"):
        monkeypatch.setenv("QVX_RUN_CHUNKS", run)
        got_pool, got = c.run_device(dev_x, variant=qd.ATTN_SPLIT)   # the host op: sync, then append + attention in one launch
        assert np.array_equal(got_pool, want_pool), run
        ok, err = within(got, want, "bf16")
        assert ok, (run, err)


def test_hundreds_of_overlapping_launches_leave_no_trace_in_the_scratch(dev):
    """240 launches back to back under programmatic dependent launch, each with more work items than
    resident CTAs (queue, late claims, runs, folding ahead, both scratch halves all in play), against
    the same launches one at a time: every output and the pool bit for bit, and a clean status."""
    torch = pytest.importorskip("torch")
    import ctypes as C
    from qubivex_b200.device import ptr
    heads, kvh, d, B, s, layers, steps = 32, 4, 128, 16, 96, 6, 40
    geo = qd.geometry(B, kvh, d, qd.BF16)
    bb = qd.block_bytes(geo)
    rng = np.random.default_rng(191)
    lengths = rng.integers(600, 3000, size=s)
    nb = (lengths + steps + B - 1) // B
    per_layer = int(nb.sum())
    perm = rng.permutation(per_layer * layers).astype(np.uint32)
    table_at = np.concatenate([[0], np.cumsum(nb)[:-1]]).astype(np.uint32)
    g = torch.Generator(device="cuda").manual_seed(6)
    pool0 = (torch.randn(per_layer * layers * bb // 2, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    q = [torch.randn((s, heads, d), device="cuda", generator=g) * 0.3 for _ in range(4)]
    kn = [torch.randn((s, kvh * d), device="cuda", generator=g) * 0.3 for _ in range(4)]
    vn = [torch.randn((s, kvh * d), device="cuda", generator=g) * 0.3 for _ in range(4)]
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    tabs = []
    for t in range(steps):
        pos = (lengths + t).astype(np.uint32)
        for l in range(layers):
            tb = C.c_void_p()
            blocks = perm[l * per_layer:(l + 1) * per_layer].copy()
            dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), per_layer * layers, heads, s, ptr(pos), ptr(blocks), per_layer,
                                                ptr(table_at), C.byref(tb)))
            tabs.append(tb)

    def run(flag, sync_each):
        pool = pool0.clone()
        outs = torch.empty((steps * layers, s, heads, d), device="cuda")
        i = 0
        for t in range(steps):
            for l in range(layers):
                dev.check(dev.lib.qvx_kv_append_attn_decode(dev.h, tabs[i], ptr(pool), ptr(kn[t % 4]), ptr(vn[t % 4]), ptr(q[t % 4]),
                                                            ptr(outs[i]), qd.ATTN_SPLIT | flag, stream))
                if sync_each:
                    torch.cuda.synchronize()
                i += 1
        torch.cuda.synchronize()
        dev.kernel_times()   # drains the timing events; raises if a kernel reported a status
        return outs, pool

    want_out, want_pool = run(0, True)
    for _ in range(2):
        got_out, got_pool = run(qd.ATTN_POOL_SETTLED, False)
        assert torch.equal(got_pool.view(torch.int16), want_pool.view(torch.int16))
        assert torch.equal(got_out.view(torch.int32), want_out.view(torch.int32))
    assert bool(torch.isfinite(want_out).all())
    for tb in tabs:
        dev.lib.qvx_tables_free(tb)


def test_independent_host_ops_side_by_side_give_the_same_bits(dev):
    # Host ops marked QVX_ATTN_POOL_SETTLED (each on its own pool here, as layers are) alternate between
    # two kernel streams; the same ops one at a time, unmarked, are the reference.  An unmarked op in
    # the middle must still see everything before it.
    cases = [Case(32, 4, 128, 16, "bf16", [900 + 37 * i, 300, 2047 - 11 * i, 1200], seed=120 + i) for i in range(6)]
    bufs = []
    try:
        for c in cases:
            b = dev.alloc(c.pool_blocks * c.bb)
            dev.write(b, 0, c.host_pool())
            bufs.append(b)
        # prefill through one unmarked synchronous op per pool (sync rows + the new row)
        want = [dev.paged_attention(b, c.geo_d, c.heads, c.q, c.k_new, c.v_new, c.pos, c.blocks, c.table_at, c.sync, c.sync_to,
                                    variant=qd.ATTN_SPLIT) for b, c in zip(bufs, cases)]
        outs = [[np.empty_like(w) for w in want] for _ in range(4)]
        for r in range(4):
            for i, (b, c) in enumerate(zip(bufs, cases)):
                flag = 0 if (r == 2 and i == 3) else qd.ATTN_POOL_SETTLED
                dev.paged_attention(b, c.geo_d, c.heads, c.q, c.k_new, c.v_new, c.pos, c.blocks, c.table_at, out=outs[r][i],
                                    variant=qd.ATTN_SPLIT | flag, wait=False)
        dev.wait()
        for r in range(4):
            for i in range(len(cases)):
                assert np.array_equal(outs[r][i].view(np.uint32), want[i].view(np.uint32)), (r, i)
    finally:
        for b in bufs:
            b.free()


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_narrowing_edge_values_have_the_oracles_bytes(dev, dtype):
    # The device narrows with the hardware's conversion (NaNs by the spelled-out rule): zeros, f32
    # subnormals, ties in and around the 16-bit formats' subnormal range, the overflow thresholds,
    # infinities and NaNs of both signs with payloads must give the oracle's bytes.
    kvh, d, B = 2, 64, 16
    bits = [0x00000000, 0x80000000, 0x00000001, 0x807fffff, 0x00800000, 0x3f800000, 0x3f808000, 0x3f818000, 0x3f80ffff,
            0x3f808001, 0x477fe000, 0x477fefff, 0x477ff000, 0x47800000, 0xc77ff000, 0x7f7fffff, 0xff7fffff, 0x7f800000,
            0xff800000, 0x7fc00000, 0xffc00001, 0x7f800001, 0xff80ffff, 0x7fffffff, 0x33000000, 0x33000001, 0x33800000,
            0x33c00000, 0x34000000, 0x387fc000, 0x387fe000, 0x38800000, 0x387fffff, 0x38000000, 0x37ffffff, 0x3effffff,
            0x7f7f8000, 0x7f7f7fff, 0x00008000, 0x00018000, 0x00017fff, 0x80008001]
    rng = np.random.default_rng(3)
    n_rows = 8
    vals = np.array(bits, dtype=np.uint32)
    rows = rng.standard_normal((n_rows, 2 * kvh * d), dtype=np.float32)
    flat = rows.reshape(-1).view(np.uint32)
    flat[:len(vals)] = vals
    flat[len(vals):2 * len(vals)] = vals ^ np.uint32(0x80000000)
    # random bit patterns too (every exponent, many ties are unlikely but signs/NaNs/subnormals are covered)
    flat[2 * len(vals):2 * len(vals) + 512] = rng.integers(0, 2**32, size=512, dtype=np.uint64).astype(np.uint32)
    geo_o, geo_d = oracle.geometry(B, kvh, d, DT[dtype], 1), qd.geometry(B, kvh, d, DT[dtype], 1)
    bb = oracle.block_bytes(geo_o)
    sync_to = np.array([5, 17, 3, 30, 31, 0, 16, 9], dtype=np.uint32)
    pool_o = np.zeros(2 * bb, dtype=np.uint8)
    kv_out = kvh * d
    rc = oracle.kv_write(pool_o, geo_o, np.zeros((0, kv_out), np.float32), np.zeros((0, kv_out), np.float32), [], [], [], rows, sync_to)
    assert rc == 0
    buf = dev.alloc(2 * bb)
    try:
        dev.write(buf, 0, np.zeros(2 * bb, dtype=np.uint8))
        # a sync-only op: no tokens
        dev.paged_attention(buf, geo_d, 4, np.zeros((0, 4, d), np.float32), np.zeros((0, kv_out), np.float32),
                            np.zeros((0, kv_out), np.float32), [], [], [], rows, sync_to)
        got = dev.read(buf, 0, 2 * bb)
    finally:
        buf.free()
    assert np.array_equal(got, pool_o)


# ---- several request threads on one device --------------------------------------------------------
def test_four_threads_submit_ops_on_one_device(dev):
    """crates/qubivex-runtime/tests/discrete.rs:772-801: four request threads share the device.  Each runs its own
    sequences on its own pool buffer through the synchronous host call, eight ops in a row, and checks every
    result (pool bytes and outputs) against the oracle."""
    import threading
    cases = [Case(32, 4, 128, 16, "bf16", [700 + 37 * i, 1025, 64 + i, 2100], seed=300 + i, amp_qk=0.4) for i in range(4)]
    wants = [c.run_oracle() for c in cases]
    errors = []

    def request(i):
        try:
            for rep in range(8):
                got_pool, got = cases[i].run_device(dev, variant=qd.ATTN_SPLIT if rep % 2 else qd.ATTN_AUTO)
                assert np.array_equal(got_pool, wants[i][0]), (i, rep)
                ok, err = within(got, wants[i][1], "bf16")
                assert ok, (i, rep, err)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=request, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    dev.kernel_times()   # the status word is clean


# ---- positive controls: the checks above can tell a wrong result ---------------------------------------
# The reference lists mutations that must each fail a named test (docs/engineering/VULKAN_EXECUTION_AUDIT.md:2499-2510):
# "reading every key from the first block fails the block-crossing test only", a changed write order fails the bytes.
# Here the device runs the true op and the ORACLE is given the mutated inputs: the comparison must then fail,
# exactly where the mutation bites and nowhere else.
def test_control_tables_that_send_every_position_to_the_first_block_are_noticed(dev):
    c = Case(8, 2, 64, 16, "bf16", [9, 16, 40, 300], seed=410)     # two sequences inside one block, two that cross
    got_pool, got = c.run_device(dev, variant=qd.ATTN_SPLIT)
    _, want = c.run_oracle()
    assert within(got, want, "bf16")[0]
    bad = Case(8, 2, 64, 16, "bf16", [9, 16, 40, 300], seed=410)
    for t in range(4):                                               # every entry of a table becomes the table's first
        lo = int(bad.table_at[t])
        hi = int(bad.table_at[t + 1]) if t + 1 < 4 else len(bad.blocks)
        bad.blocks[lo:hi] = bad.blocks[lo]
    for r, at in enumerate(c.sync_to):                               # ... and its rows go where those tables say
        blk, slot = divmod(int(at), 16)
        t = int(np.searchsorted(c.table_at, np.where(c.blocks == blk)[0][0], side="right")) - 1
        bad.sync_to[r] = int(bad.blocks[int(bad.table_at[t])]) * 16 + slot
    bad_pool, bad_want = bad.run_oracle()
    for t, crosses in enumerate([False, False, True, True]):
        ok, _ = within(got[t], bad_want[t], "bf16")
        assert ok != crosses, t                                      # the sequences inside one block still agree
    assert not np.array_equal(got_pool, bad_pool)


def test_control_duplicate_sync_rows_written_in_the_other_order_are_noticed(dev):
    c = Case(4, 2, 64, 16, "bf16", [40], seed=3)
    c.sync_to = np.concatenate([c.sync_to, c.sync_to[5:9]])
    extra = np.random.default_rng(5).standard_normal((4, c.sync.shape[1]), dtype=np.float32)
    c.sync = np.concatenate([c.sync, extra])
    got_pool, got = c.run_device(dev)
    want_pool, _ = c.run_oracle()
    assert np.array_equal(got_pool, want_pool)                       # the later duplicate wins on both sides
    n = len(c.sync_to)
    c.sync_to, c.sync = c.sync_to[::-1].copy(), c.sync[::-1].copy()  # the oracle writes them in the other order
    bad_pool, bad_want = c.run_oracle()
    assert not np.array_equal(got_pool, bad_pool)                    # the earlier duplicate won there: the bytes differ
    assert not within(got, bad_want, "bf16")[0]


# ---- the benchmark configurations at their full sizes, sampled against the oracle ----------------------
def _full_size_case(name):
    rng = np.random.default_rng(8)
    if name == "c2":    # the configuration the metric is quoted on, one layer: batch 64, contexts U[1024, 4096], 32 q / 4 kv heads
        return 32, 4, 128, 16, rng.integers(1024, 4097, size=64)
    if name == "c3":    # 16 x 32768 positions, 32 q / 4 kv heads of 128, block 16 (the prefix sharing is in test_gpu_scenarios)
        return 32, 4, 128, 16, np.full(16, 32768)
    if name == "c4":    # ~58 982 live blocks of 32 positions, 32 q / 8 kv heads: the work items are runs of four chunks
        lens = []
        while sum((n + 31) // 32 for n in lens) < 58982:
            lens.append(int(rng.integers(256, 8193)))
        return 32, 8, 128, 32, np.array(lens)
    if name == "c5":    # one GPU's KV head of the head-sharded shape: batch 256, contexts U[1024, 16384] (runs of two chunks)
        return 8, 1, 128, 16, rng.integers(1024, 16385, size=256)
    raise ValueError(name)


@pytest.mark.parametrize("name", ["c2", "c3", "c4", "c5"])
def test_full_size_configurations_sampled_against_the_oracle(dev, name):
    """One attention step at the configuration's full size (up to 7.2 GiB of KV, hundreds of work items per CTA, runs of
    two to four chunks, merge trees of two levels), and the shortest, the median and the longest sequence checked against
    the oracle on their own blocks of the pool."""
    torch = pytest.importorskip("torch")
    import ctypes as C
    from qubivex_b200.device import ptr
    heads, kvh, d, B, lengths = _full_size_case(name)
    lengths = np.asarray(lengths, dtype=np.int64)
    s = len(lengths)
    geo = qd.geometry(B, kvh, d, qd.BF16)
    bb = qd.block_bytes(geo)
    nb = (lengths + B - 1) // B
    pool_blocks = int(nb.sum()) + 16
    perm = np.random.default_rng(9).permutation(pool_blocks).astype(np.uint32)
    table_at = np.zeros(s, dtype=np.uint32)
    table_at[1:] = np.cumsum(nb)[:-1]
    blocks = perm[: int(nb.sum())].copy()
    pos = (lengths - 1).astype(np.uint32)
    g = torch.Generator(device="cuda").manual_seed(10)
    pool = torch.empty(pool_blocks * bb // 2, dtype=torch.bfloat16, device="cuda")
    step = 1 << 28
    for lo in range(0, pool.numel(), step):                      # N(0,1) / sqrt(d), written as bf16 bits
        n = min(step, pool.numel() - lo)
        pool[lo:lo + n] = (torch.randn(n, device="cuda", generator=g) * d ** -0.5).to(torch.bfloat16)
    q = torch.randn((s, heads, d), device="cuda", generator=g) * d ** -0.5
    out = torch.empty_like(q)
    tabs = C.c_void_p()
    dev.check(dev.lib.qvx_tables_create(dev.h, C.byref(geo), pool_blocks, heads, s, ptr(pos), ptr(blocks), len(blocks), ptr(table_at),
                                        C.byref(tabs)))
    dev.check(dev.lib.qvx_attn_decode(dev.h, tabs, ptr(pool), ptr(q), ptr(out), qd.ATTN_SPLIT,
                                      C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    dev.kernel_times()
    dev.lib.qvx_tables_free(tabs)
    assert bool(torch.isfinite(out).all())
    geo_o = oracle.geometry(B, kvh, d, oracle.BF16)
    order = np.argsort(lengths)
    bytes_view = pool.view(torch.uint8)
    for t in {int(order[0]), int(order[s // 2]), int(order[-1])}:
        ids = blocks[int(table_at[t]):int(table_at[t]) + int(nb[t])].astype(np.int64)
        idx = (torch.from_numpy(ids).cuda()[:, None] * bb + torch.arange(bb, device="cuda")[None, :]).reshape(-1)
        host_pool = bytes_view[idx].cpu().numpy()
        rc, want = oracle.attn_decode(host_pool, geo_o, heads, q[t:t + 1].cpu().numpy(), pos[t:t + 1], np.arange(len(ids), dtype=np.uint32),
                                      np.zeros(1, dtype=np.uint32), threads=8)
        assert rc == 0
        ok, err = within(out[t:t + 1].cpu().numpy(), want, "bf16")
        assert ok, (name, t, int(lengths[t]), err)
        # the values are ~ 1 / sqrt(d) and the outputs an average of thousands of them: the absolute bar alone would pass
        # anything, so the relative error against the largest output counts too
        assert err <= 1e-2 * float(np.abs(want).max()), (name, t, err)
