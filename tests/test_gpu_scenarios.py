"""The path end to end on a B200, as the reference's runtime drives it: the pool and its block
tables (OnDevice), host rows synced once, decode steps, prefix sharing with copy-on-write,
compaction.  Every step is checked against the CPU oracle fed the same tables: attention per
step, pool bytes at the end.  Shapes follow the benchmark configurations, scaled to seconds."""
import numpy as np
import pytest

import oracle
from helpers import within
from qubivex_b200 import device as qd
from qubivex_b200.ondevice import AttnSeq, OnDevice

pytestmark = pytest.mark.gpu

DT = {"f32": 0, "bf16": 1}


class HostCache:
    """The authoritative host copy of one sequence's keys and values: [kv_head][position][d]
    (KvCache, crates/qubivex-arch/src/lib.rs:283-524)."""

    def __init__(self, kvh, d, cap, rng, scale=1.0):
        self.k = (rng.standard_normal((kvh, cap, d), dtype=np.float32) * scale).astype(np.float32)
        self.v = (rng.standard_normal((kvh, cap, d), dtype=np.float32) * scale).astype(np.float32)
        self.len = 0
        self.epoch = 0

    def row(self, p):
        return self.k[:, p, :].reshape(-1), self.v[:, p, :].reshape(-1)


def oracle_step(pool, geo_o, heads, plan, seqs, q, k_new, v_new):
    """The same op on the CPU: the copies copy-on-write asked for, then sync rows, new rows, attention."""
    if len(plan.copy_src):
        assert oracle.block_copy(pool, geo_o, plan.copy_src, plan.copy_dst) == 0
    kv_out = geo_o.kv_heads * geo_o.head_dim
    sync = np.empty((len(plan.sync_to), 2 * kv_out), dtype=np.float32)
    for r, (si, p) in enumerate(zip(plan.sync_seq, plan.sync_pos)):
        sync[r, :kv_out], sync[r, kv_out:] = seqs[int(si)].host.row(int(p))
    rc, att = oracle.paged_attention(pool, geo_o, heads, q, k_new, v_new, plan.pos, plan.blocks, plan.table_at, sync, plan.sync_to)
    assert rc == 0
    return att


class Seq:
    def __init__(self, host):
        self.host = host
        self.mirror = None

    def attn_seq(self):
        return AttnSeq(self.mirror, self.host.k, self.host.v, self.host.len, self.host.epoch)


def decode_step(od, seqs, pool_o, geo_o, heads, rng, dtype, variant, scale=1.0, layer=0):
    """One decode pass over `seqs` at their current lengths: device and oracle, compared."""
    s = len(seqs)
    kvh, d = geo_o.kv_heads, geo_o.head_dim
    q = (rng.standard_normal((s, heads, d), dtype=np.float32) * scale).astype(np.float32)
    k_new = np.stack([sq.host.row(sq.host.len)[0] for sq in seqs])
    v_new = np.stack([sq.host.row(sq.host.len)[1] for sq in seqs])
    aseqs = [sq.attn_seq() for sq in seqs]
    out = od.attention(aseqs, layer, q, k_new, v_new, variant=variant)
    assert out is not None
    for sq, a in zip(seqs, aseqs):
        sq.mirror = a.mirror
    want = oracle_step(pool_o, geo_o, heads, od.last_plan, seqs, q, k_new, v_new)
    for sq in seqs:
        sq.host.len += 1
    if variant == qd.ATTN_EXACT and dtype == "f32":
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    else:
        ok, err = within(out, want, dtype)
        assert ok, err
    return od.last_plan


def read_pool(dev, od, n_bytes):
    return dev.read(od.kv_buffer(), 0, n_bytes)


# ---- C1: the reference-runnable configuration ---------------------------------------------------
@pytest.mark.parametrize("variant", [qd.ATTN_EXACT, qd.ATTN_SPLIT])
def test_c1_prompts_then_64_decode_steps(dev, variant):
    """1 layer, block 16, f32, 8 q / 2 kv heads of 64; prompts 37/128/255/512; 64 decode steps; the
    256-block pool handed out in a seeded random permutation.  Outputs: attention per step and
    the final pool bytes."""
    heads, kvh, d, B, blocks = 8, 2, 64, 16, 256
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.F32), oracle.geometry(B, kvh, d, oracle.F32)
    rng = np.random.default_rng(20261125)
    od = OnDevice(dev, geo_d, heads, blocks=blocks)
    od.kv.set_free_order(rng.permutation(blocks))
    n_bytes = blocks * oracle.block_bytes(geo_o)
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)
    seqs = []
    for n in (37, 128, 255, 512):
        sq = Seq(HostCache(kvh, d, n + 64, rng))
        sq.host.len = n          # the prompt was run on the host: its rows reach the pool by sync
        seqs.append(sq)
    first = decode_step(od, seqs, pool_o, geo_o, heads, rng, "f32", variant)
    assert len(first.sync_to) == 37 + 128 + 255 + 512          # every prompt row synced exactly once
    for _ in range(63):
        plan = decode_step(od, seqs, pool_o, geo_o, heads, rng, "f32", variant)
        assert len(plan.sync_to) == 0
    assert np.array_equal(read_pool(dev, od, n_bytes), pool_o)
    st = od.kv.stats()
    assert st.synced_rows == 932 and st.layers == 64 and st.full == 0
    for sq in seqs:
        sq.mirror.drop()
    assert od.kv.stats().free == blocks                         # tests/discrete.rs:724-727
    od.close()


# ---- the host cache stays authoritative ----------------------------------------------------------
def test_a_cleared_cache_and_a_failed_pass_are_resynced(dev):
    heads, kvh, d, B = 8, 2, 64, 16
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.BF16), oracle.geometry(B, kvh, d, oracle.BF16)
    rng = np.random.default_rng(3)
    od = OnDevice(dev, geo_d, heads, blocks=32)
    n_bytes = 32 * oracle.block_bytes(geo_o)
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)
    sq = Seq(HostCache(kvh, d, 200, rng))
    sq.host.len = 50
    decode_step(od, [sq], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT)
    # a pass that failed after the device stored its row: the host is back at 49 positions
    sq.host.len = 49
    sq.host.k[:, 49:, :] += 1.0
    plan = decode_step(od, [sq], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT)
    assert len(plan.sync_to) == 0 and int(plan.pos[0]) == 49    # the new row rewrites position 49
    # the cache was cleared and another prompt run: a new epoch starts the mirror again
    sq.host = HostCache(kvh, d, 200, rng)
    sq.host.len, sq.host.epoch = 20, 1
    plan = decode_step(od, [sq], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT)
    assert len(plan.sync_to) == 20
    assert np.array_equal(read_pool(dev, od, n_bytes), pool_o)
    sq.mirror.drop()
    od.close()


def test_a_pool_one_block_short_declines_and_counts_it(dev):
    # crates/qubivex-runtime/tests/discrete.rs:735-767
    heads, kvh, d, B = 8, 2, 64, 16
    od = OnDevice(dev, qd.geometry(B, kvh, d, qd.BF16), heads, blocks=3)
    rng = np.random.default_rng(4)
    a, b = Seq(HostCache(kvh, d, 64, rng)), Seq(HostCache(kvh, d, 64, rng))
    a.host.len = b.host.len = 31
    aseqs = [a.attn_seq(), b.attn_seq()]
    q = rng.standard_normal((2, heads, d), dtype=np.float32)
    kv = rng.standard_normal((2, kvh * d), dtype=np.float32)
    assert od.attention(aseqs, 0, q, kv, kv) is None            # declined: the host runs this layer
    assert od.kv.stats().full == 1 and od.routed == 0
    for s_ in aseqs:
        s_.mirror.drop()
    od.close()


# ---- C3: a shared prefix, copy-on-write on the first divergent append ------------------------------
@pytest.mark.parametrize("prefix,copies", [(8 * 16 + 8, 3), (8 * 16, 0)])
def test_c3_shared_prefix_and_copy_on_write(dev, prefix, copies):
    """Three of four sequences share a prefix through reference-counted blocks.  A prefix that
    ends inside a block forces one whole-block copy per sharer on its first append (the retained
    prefix holds the block too, so nobody writes in place); one that ends on a block boundary
    copies nothing."""
    heads, kvh, d, B, blocks = 32, 4, 128, 16, 160
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.BF16), oracle.geometry(B, kvh, d, oracle.BF16)
    rng = np.random.default_rng(33)
    scale = d ** -0.5
    od = OnDevice(dev, geo_d, heads, blocks=blocks)
    od.kv.set_free_order(rng.permutation(blocks))
    n_bytes = blocks * oracle.block_bytes(geo_o)
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)
    # the retained value: a sequence that ran the prefix and stays in the index
    owner = Seq(HostCache(kvh, d, prefix + 8, rng, scale))
    owner.host.len = prefix - 1
    decode_step(od, [owner], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)   # pool now holds 0..prefix-1
    assert owner.mirror.synced(0) == prefix
    sharers = []
    for _ in range(3):
        sq = Seq(HostCache(kvh, d, 600, rng, scale))
        sq.host.k[:, :prefix] = owner.host.k[:, :prefix]           # the same tokens: the same keys and values
        sq.host.v[:, :prefix] = owner.host.v[:, :prefix]
        sq.host.len = prefix
        sq.mirror = owner.mirror.fork(prefix)                      # a table copy and reference counts, no bytes
        sharers.append(sq)
    lone = Seq(HostCache(kvh, d, 600, rng, scale))
    lone.host.len = 300
    free_before = od.kv.stats().free
    plan = decode_step(od, sharers + [lone], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)
    assert len(plan.copy_src) == copies and od.kv.stats().cow_copies == copies
    assert len(plan.sync_to) == 300                                # only the lone sequence's prompt
    shared_blocks = prefix // B
    for sq in sharers:
        assert sq.mirror.blocks(0)[:shared_blocks].tolist() == owner.mirror.blocks(0)[:shared_blocks].tolist()
    assert od.kv.refcount(int(owner.mirror.blocks(0)[0])) == 4
    new_blocks = (300 // B + 1) + 3                                 # lone's table + one block per sharer (copy or growth)
    assert free_before - od.kv.stats().free == new_blocks
    for _ in range(20):
        plan = decode_step(od, sharers + [lone], pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)
        assert len(plan.copy_src) == 0
    assert np.array_equal(read_pool(dev, od, n_bytes), pool_o)
    for sq in sharers + [lone, owner]:
        sq.mirror.drop()
    assert od.kv.stats().free == blocks
    od.close()


# ---- C3 through the prefix index: lookup -> shared blocks -> copy-on-write -> retain -> eviction ----
def test_c3_prefix_hits_share_blocks_through_the_index(dev):
    """The request flow of Engine::restore / Engine::retain (crates/qubivex-runtime/src/engine.rs:1659-1699) with
    the index's value a set of pages (docs/decisions/ADR-016-KV-SUBSYSTEM.md:82-89): a finished conversation of
    8192 + 8 tokens is retained; eight requests in its scope find it by lookup and share its 513 blocks; each
    copies the partly filled block on its first append; another scope does not hit; an entry evicted while a
    hit on it is held lives until the hit goes; finished sequences are retained in turn and the budget evicts the
    oldest, whose own blocks return to the free list.  Attention against the oracle at every step, the pool's
    bytes at the end, free == blocks after everything is dropped."""
    heads, kvh, d, B, blocks = 16, 2, 128, 16, 1200
    prefix, sharers_n = 8192 + 8, 8
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.BF16), oracle.geometry(B, kvh, d, oracle.BF16)
    rng = np.random.default_rng(1659)
    scale = d ** -0.5
    od = OnDevice(dev, geo_d, heads, blocks=blocks)
    od.kv.set_free_order(rng.permutation(blocks))
    index = od.retain_prefixes(budget_blocks=1100)
    n_bytes = blocks * oracle.block_bytes(geo_o)
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)

    def step(seqs):
        """decode_step, with the oracle's attention on all host threads (the contexts are 8200 positions)."""
        s = len(seqs)
        q = (rng.standard_normal((s, heads, d), dtype=np.float32) * scale).astype(np.float32)
        k_new = np.stack([sq.host.row(sq.host.len)[0] for sq in seqs])
        v_new = np.stack([sq.host.row(sq.host.len)[1] for sq in seqs])
        aseqs = [sq.attn_seq() for sq in seqs]
        out = od.attention(aseqs, 0, q, k_new, v_new, variant=qd.ATTN_SPLIT)
        assert out is not None
        plan = od.last_plan
        for sq, a in zip(seqs, aseqs):
            sq.mirror = a.mirror
        if len(plan.copy_src):
            assert oracle.block_copy(pool_o, geo_o, plan.copy_src, plan.copy_dst) == 0
        kv_out = kvh * d
        sync = np.empty((len(plan.sync_to), 2 * kv_out), dtype=np.float32)
        for r, (si, p) in enumerate(zip(plan.sync_seq, plan.sync_pos)):
            sync[r, :kv_out], sync[r, kv_out:] = seqs[int(si)].host.row(int(p))
        assert oracle.kv_write(pool_o, geo_o, k_new, v_new, plan.pos, plan.blocks, plan.table_at, sync, plan.sync_to) == 0
        rc, want = oracle.attn_decode(pool_o, geo_o, heads, q, plan.pos, plan.blocks, plan.table_at, threads=8)
        assert rc == 0
        for sq in seqs:
            sq.host.len += 1
        ok, err = within(out, want, "bf16")
        assert ok, err
        return plan

    # a conversation runs 8192 + 8 prompt tokens on the host and one decode step on the device, then ends
    tokens_a = rng.integers(0, 50000, size=prefix + 1, dtype=np.uint32)
    owner = Seq(HostCache(kvh, d, prefix + 8, rng, scale))
    owner.host.len = prefix
    first = step([owner])
    assert len(first.sync_to) == prefix and owner.mirror.synced(0) == prefix + 1
    owner_blocks = owner.mirror.blocks(0).copy()
    assert len(owner_blocks) == 513
    assert od.retain("chat-1", tokens_a, owner.mirror, owner.host.k, owner.host.v)
    assert index.stats().entries == 1 and index.cost() == 513
    free_after_owner = od.kv.stats().free
    assert free_after_owner == blocks - 513

    # another scope never sees it; nor does a prompt that shares fewer than MIN_REUSE tokens
    probe_k, probe_v = np.zeros((kvh, 16, d), np.float32), np.zeros((kvh, 16, d), np.float32)
    assert od.restore("chat-2", tokens_a, probe_k, probe_v) == (None, 0)
    short = np.concatenate([tokens_a[:20], rng.integers(50000, 60000, size=30, dtype=np.uint32)])
    assert od.restore("chat-1", short, probe_k, probe_v) == (None, 0)
    assert index.stats().hits == 0 and index.stats().lookups == 2

    # eight requests that continue the conversation differently: found through the index, nothing copied
    sharers = []
    for i in range(sharers_n):
        prompt = np.concatenate([tokens_a[:prefix], np.array([60000 + i], dtype=np.uint32)])
        sq = Seq(HostCache(kvh, d, prefix + 32, rng, scale))
        sq.mirror, reuse = od.restore("chat-1", prompt, sq.host.k, sq.host.v)
        assert reuse == prefix                                         # the last prompt token always runs
        assert np.array_equal(sq.host.k[:, :prefix], owner.host.k[:, :prefix])
        sq.host.len = prefix
        sq.tokens = prompt
        sharers.append(sq)
    assert index.stats().hits == sharers_n and index.stats().tokens_reused == sharers_n * prefix
    assert od.kv.stats().free == free_after_owner                     # a hit takes no block
    assert od.kv.refcount(int(owner_blocks[0])) == 1 + sharers_n and od.kv.refcount(int(owner_blocks[512])) == 1 + sharers_n
    lone = Seq(HostCache(kvh, d, 400, rng, scale))                    # the other scope's request runs its own prompt
    lone.host.len = 300

    plan = step(sharers + [lone])
    assert len(plan.copy_src) == sharers_n and set(plan.copy_src.tolist()) == {int(owner_blocks[512])}   # the partly filled block, once per sharer
    assert od.kv.stats().cow_copies == sharers_n and len(plan.sync_to) == 300
    assert od.kv.refcount(int(owner_blocks[512])) == 1                # only the retained entry still holds it
    for sq in sharers:
        assert sq.mirror.blocks(0)[:512].tolist() == owner_blocks[:512].tolist()
    for _ in range(8):                                                # on into a fresh block at position 8208
        plan = step(sharers + [lone])
        assert len(plan.copy_src) == 0 and len(plan.sync_to) == 0
    assert all(len(sq.mirror.blocks(0)) == 514 for sq in sharers)

    # an entry evicted while a hit on it is held lives until the hit is released (lib.rs:330-347)
    kept, reuse, hit = index.lookup("chat-1", sharers[0].tokens)
    assert index.evict_oldest() and index.stats().entries == 0
    late = Seq(HostCache(kvh, d, prefix + 32, rng, scale))
    late.mirror = kept.mirror.fork(reuse)                             # still usable: the hit keeps the value alive
    free_before_release = od.kv.stats().free
    index.release(hit)                                                # now the retained sequence lets go of its blocks
    assert od.kv.stats().free == free_before_release                  # ... all of which somebody still shares
    late.mirror.drop()
    assert od.kv.stats().free == free_before_release + 1              # the owner's partly filled block had one holder left
    plan = step(sharers + [lone])                                     # the sharers decode on over the evicted entry's blocks

    # finished sequences are retained in turn; the budget (1100 blocks) holds two of 514, the third evicts the oldest
    done = sharers[:3]
    for i, sq in enumerate(done):
        toks = np.concatenate([sq.tokens, rng.integers(0, 50000, size=sq.host.len - len(sq.tokens), dtype=np.uint32)])
        free_before = od.kv.stats().free
        assert od.retain("chat-1", toks, sq.mirror, sq.host.k, sq.host.v)
        if i < 2:
            assert od.kv.stats().free == free_before
        else:
            assert index.stats().evicted == 2 and index.stats().entries == 2
            assert od.kv.stats().free == free_before + 2              # the evicted sequence's own two blocks (its copy and the one after)
    assert np.array_equal(read_pool(dev, od, n_bytes), pool_o)
    for sq in sharers[3:] + [lone]:
        sq.mirror.drop()
    index.clear()
    assert od.kv.stats().free == blocks
    od.close()


# ---- C4: churn, compaction, then attention ---------------------------------------------------------
def test_c4_churn_compaction_then_attention(dev):
    """32 q / 8 kv heads of 128, bf16, block 32.  Sequences retire and arrive at random; a compaction
    pass gathers the live blocks to the front of the pool (moves on the device, tables rewritten
    on the host); one decode step over every live sequence follows.  The live prefix of the pool
    and the attention outputs must match the oracle's."""
    heads, kvh, d, B, blocks = 32, 8, 128, 32, 96
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.BF16), oracle.geometry(B, kvh, d, oracle.BF16)
    bb = oracle.block_bytes(geo_o)
    rng = np.random.default_rng(44)
    scale = d ** -0.5
    od = OnDevice(dev, geo_d, heads, blocks=blocks)
    od.kv.set_free_order(rng.permutation(blocks))
    n_bytes = blocks * bb
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)

    def admit():
        sq = Seq(HostCache(kvh, d, 700, rng, scale))
        sq.host.len = int(rng.integers(40, 250))
        return sq

    live = [admit() for _ in range(6)]
    decode_step(od, live, pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)
    moved = 0
    for step in range(6):
        # retire a third, admit as many
        for _ in range(2):
            sq = live.pop(int(rng.integers(0, len(live))))
            sq.mirror.drop()
        fresh = [admit(), admit()]
        live += fresh
        decode_step(od, live, pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)
        src, dst = od.kv.compact()
        L = int(od.kv.stats().blocks - od.kv.stats().free)
        assert np.all(src >= L) and np.all(dst < L) and len(set(dst.tolist())) == len(dst)
        dev.block_copy(od.kv_buffer(), geo_d, src, dst)
        assert oracle.block_copy(pool_o, geo_o, src, dst) == 0
        moved += len(src)
        for sq in live:
            assert np.all(sq.mirror.blocks(0) < L)                 # every live block is in the prefix now
        decode_step(od, live, pool_o, geo_o, heads, rng, "bf16", qd.ATTN_SPLIT, scale)
        got = read_pool(dev, od, n_bytes)
        L = int(od.kv.stats().blocks - od.kv.stats().free)
        assert np.array_equal(got[: L * bb], pool_o[: L * bb])
    assert moved > 0 and od.kv.stats().compaction_moves == moved
    for sq in live:
        sq.mirror.drop()
    assert od.kv.stats().free == blocks
    od.close()


def test_c4_at_full_size_churn_and_compaction_keep_every_live_block(dev):
    """The churn configuration at its own size: a pool of 65 536 blocks of 128 KiB (8 GiB) filled to 90 % by sequences
    of U[256, 8192] positions, 5 % of the blocks retired and as many admitted per step, a compaction pass after each
    step.  Size-independent properties instead of an oracle copy of 8 GiB: every live block's checksum follows it
    to its new id (sequence by sequence, in table order), the live ids are exactly 0..L, nothing outside the moves'
    destinations changes, and the counters add up."""
    torch = pytest.importorskip("torch")
    import ctypes as C
    from qubivex_b200.device import ptr
    from qubivex_b200.kvpool import KvPool
    B, kvh, d, N = 32, 8, 128, 65536
    geo = qd.geometry(B, kvh, d, qd.BF16)
    bb = qd.block_bytes(geo)
    assert bb == 128 * 1024
    rng = np.random.default_rng(404)
    kv = KvPool(geo, N)
    kv.set_free_order(rng.permutation(N))
    pool = torch.empty(N * bb, dtype=torch.uint8, device="cuda")
    words = pool.view(torch.int64)
    g = torch.Generator(device="cuda").manual_seed(405)
    step_words = 1 << 27
    for lo in range(0, words.numel(), step_words):
        n = min(step_words, words.numel() - lo)
        words[lo:lo + n] = torch.randint(-2**62, 2**62, (n,), dtype=torch.int64, device="cuda", generator=g)
    checksums = lambda: words.view(N, -1).sum(dim=1).cpu().numpy()      # per block, wrapping
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def admit(blocks_wanted):
        lens, have = [], 0
        while have < blocks_wanted:
            n = int(rng.integers(256, 8193))
            lens.append(n)
            have += (n + B - 1) // B
        ms = [kv.mirror() for _ in lens]
        plan = kv.attention_plan(ms, [n - 1 for n in lens], 0)
        assert plan is not None
        kv.commit(plan, ms, 0)
        kv.free_plan(plan)
        return ms

    live = admit(int(0.9 * N))
    used = lambda: int(kv.stats().blocks - kv.stats().free)
    assert 0.9 * N <= used() <= 0.9 * N + 256
    moved_total = 0
    for _ in range(3):
        # churn: retire sequences until 5 % of the pool's blocks are back, admit as many blocks again
        target = used() - int(0.05 * N)
        while used() > target:
            live.pop(int(rng.integers(0, len(live)))).drop()
        live += admit(int(0.9 * N) - used())
        before = checksums()
        tables = [m.blocks(0).copy() for m in live]
        L = used()
        src, dst = kv.compact()
        assert len(src) > 0 and np.all(src >= L) and np.all(dst < L) and len(set(dst.tolist())) == len(dst)
        d_src, d_dst = (torch.from_numpy(a.astype(np.int32)).cuda() for a in (src, dst))
        dev.check(dev.lib.qvx_block_copy(dev.h, C.byref(geo), ptr(pool), N, ptr(d_src), ptr(d_dst), len(src), stream))
        torch.cuda.synchronize()
        dev.kernel_times()                                            # no late report
        after = checksums()
        seen = np.zeros(N, dtype=bool)
        for m, old in zip(live, tables):
            new = m.blocks(0)
            assert len(new) == len(old) and np.all(new < L)
            assert np.array_equal(after[new], before[old])           # the bytes went with the block, in table order
            assert not seen[new].any()
            seen[new] = True
        assert seen[:L].all() and not seen[L:].any()                  # the live ids are exactly 0..L
        untouched = np.ones(N, dtype=bool)
        untouched[dst] = False
        assert np.array_equal(after[untouched], before[untouched])    # (sources keep their bytes: they are free now)
        assert used() == L
        moved_total += len(src)
    st = kv.stats()
    assert st.compaction_moves == moved_total and st.bytes_moved == 2 * moved_total * bb   # a read and a write per move
    assert moved_total > 0.05 * N     # (the first pass gathers a pool filled in random order: about a tenth of the live blocks)
    for m in live:
        m.drop()
    assert kv.stats().free == N
    kv.delete()


# ---- the prelude inside the runtime's loop --------------------------------------------------------
def test_decode_steps_from_raw_projections_keep_the_host_cache_in_step(dev):
    """Each pass hands the device the raw projections; clip, norms and RoPE run there and the new
    rows come back for the host cache (sim.rs:325-357).  After a cache reset everything is synced
    from that host cache again, so its rows must be exactly the device's."""
    heads, kvh, d, B, blocks = 16, 2, 128, 16, 96
    geo_d, geo_o = qd.geometry(B, kvh, d, qd.BF16), oracle.geometry(B, kvh, d, oracle.BF16)
    rng = np.random.default_rng(77)
    od = OnDevice(dev, geo_d, heads, blocks=blocks)
    n_bytes = blocks * oracle.block_bytes(geo_o)
    dev.write(od.kv_buffer(), 0, np.zeros(n_bytes, dtype=np.uint8))
    pool_o = np.zeros(n_bytes, dtype=np.uint8)
    seqs = [Seq(HostCache(kvh, d, 300, rng, scale=0.0)) for _ in range(3)]   # empty caches: everything comes from decode steps
    norms = (rng.standard_normal(heads * d, dtype=np.float32), rng.standard_normal(kvh * d, dtype=np.float32))
    clip, eps, theta = 3.0, 1e-5, 10000.0
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d)))).astype(np.float32)

    def rope_for(positions):
        f = np.outer(np.asarray(positions, dtype=np.float32), inv).astype(np.float32)
        return np.concatenate([np.cos(f), np.sin(f)], axis=1).astype(np.float32)

    for step in range(40):
        if step == 25:   # the host cache was cleared and refilled: a new epoch, the device re-syncs all rows
            for sq in seqs:
                sq.host.epoch += 1
        s = len(seqs)
        q = rng.standard_normal((s, heads * d), dtype=np.float32)
        k = rng.standard_normal((s, kvh * d), dtype=np.float32) * 2
        v = rng.standard_normal((s, kvh * d), dtype=np.float32) * 2
        rope = rope_for([sq.host.len for sq in seqs])
        wq, wk, wv = oracle.attn_prelude(q, k, v, heads, kvh, d, rope, clip=clip, qk_norm=norms, eps=eps)
        aseqs = [sq.attn_seq() for sq in seqs]
        k_back, v_back = k.copy(), v.copy()
        out = od.attention(aseqs, 0, q, k_back, v_back, variant=qd.ATTN_SPLIT,
                           prelude={"rope": rope, "clip": clip, "qk_norm": norms, "eps": eps})
        assert out is not None
        assert np.array_equal(k_back.view(np.uint32), wk.view(np.uint32)) and np.array_equal(v_back.view(np.uint32), wv.view(np.uint32))
        for t, (sq, a) in enumerate(zip(seqs, aseqs)):
            sq.mirror = a.mirror
            sq.host.k[:, sq.host.len, :] = k_back[t].reshape(kvh, d)   # what the host cache keeps
            sq.host.v[:, sq.host.len, :] = v_back[t].reshape(kvh, d)
        want = oracle_step(pool_o, geo_o, heads, od.last_plan, seqs, wq, wk, wv)
        if step == 25:
            assert len(od.last_plan.sync_to) == 3 * 25
        for sq in seqs:
            sq.host.len += 1
        ok, err = within(out, want, "bf16")
        assert ok, (step, err)
    for sq in seqs:
        sq.mirror.drop()
    od.close()
