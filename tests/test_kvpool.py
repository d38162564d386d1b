"""Block bookkeeping against the reference's behaviour
(crates/qubivex-runtime/src/discrete.rs:215-290, :951-1009; tests/discrete.rs:641-847) and
against the Python restatement on random traffic.  No GPU."""
import numpy as np
import pytest

from oracle import hostlogic as ref
from qubivex_b200 import device as qd
from qubivex_b200.kvpool import DEFAULT_KV_POOL, MAX_KV_POOL, KvPool, blocks_for

GEO = qd.geometry(16, 2, 64, qd.F32, qd.LAYOUT_NATIVE)


def plan_ok(pool, seqs, pos, layer=0, epochs=None):
    p = pool.attention_plan(seqs, pos, layer, epochs)
    assert p is not None
    pool.commit(p, seqs, layer)
    pool.free_plan(p)
    return p


def test_the_kv_pool_is_512_mib_by_default_and_capped():
    # crates/qubivex-runtime/tests/discrete.rs: the_kv_pool_is_512_mib_by_default_and_capped
    olmoe = qd.geometry(256, 16, 128, qd.F32, qd.LAYOUT_REFERENCE)  # 4 MiB blocks
    big = 1 << 40
    assert blocks_for(olmoe, 0, big, big) == DEFAULT_KV_POOL // (4 << 20) == 128
    assert blocks_for(olmoe, 4 << 30, big, big) == MAX_KV_POOL // (4 << 20) == 256
    assert blocks_for(olmoe, 64 << 20, big, big) == 16
    assert blocks_for(olmoe, 0, 100 << 20, big) == 25          # what the budget leaves
    assert blocks_for(olmoe, 0, big, 40 << 20) == 10           # one buffer the device addresses
    assert blocks_for(olmoe, 0, 3 << 20, big) == 0             # no room for one block
    assert blocks_for(olmoe, 64 << 30, big, big, uncapped=True) == (64 << 30) // (4 << 20)


def test_blocks_are_taken_lazily_lifo_from_block_0_and_all_come_back():
    pool = KvPool(GEO, 8)
    a, b = pool.mirror(), pool.mirror()
    p = plan_ok(pool, [a, b], [0, 17])
    assert p.blocks.tolist() == [0, 1, 2] and p.table_at.tolist() == [0, 1] and p.pos.tolist() == [0, 17]
    assert pool.stats().free == 5
    p = plan_ok(pool, [a, b], [15, 18])       # no boundary crossed: nothing taken
    assert pool.stats().free == 5 and p.blocks.tolist() == [0, 1, 2]
    p = plan_ok(pool, [a, b], [16, 19])       # a crosses into its second block
    assert p.blocks.tolist() == [0, 3, 1, 2]
    a.drop()
    assert pool.stats().free == 6
    c = pool.mirror()
    p = plan_ok(pool, [c], [0])
    assert p.blocks.tolist() == [3]           # the last block given back is the first handed out
    b.drop(); c.drop()
    s = pool.stats()
    assert s.free == s.blocks == 8            # tests/discrete.rs:724-727
    pool.delete()


def test_unsynced_host_rows_are_listed_once_then_never_again():
    # tests/discrete.rs:691-723: the prompt rows are synced exactly once per layer.
    pool = KvPool(GEO, 16)
    m = pool.mirror()
    p = plan_ok(pool, [m], [37], layer=1)
    assert p.sync_pos.tolist() == list(range(37)) and set(p.sync_seq.tolist()) == {0}
    blocks = m.blocks(1)
    assert p.sync_to.tolist() == [int(blocks[i // 16]) * 16 + i % 16 for i in range(37)]
    assert m.synced(1) == 38
    p = plan_ok(pool, [m], [38], layer=1)
    assert len(p.sync_to) == 0
    p = plan_ok(pool, [m], [38], layer=0)      # another layer has its own blocks and rows
    assert len(p.sync_to) == 38 and not set(m.blocks(0)) & set(m.blocks(1))
    assert pool.stats().synced_rows == 37 + 38 and pool.stats().layers == 3
    m.drop(); pool.delete()


def test_a_failed_pass_is_written_again():
    # discrete.rs:983-985: rows past the host's count are from a pass that failed.
    pool = KvPool(GEO, 4)
    m = pool.mirror()
    plan_ok(pool, [m], [20])
    assert m.synced(0) == 21
    p = plan_ok(pool, [m], [18])               # the host cache went back to 18 positions
    assert len(p.sync_to) == 0 and m.synced(0) == 19
    m.drop(); pool.delete()


def test_the_pool_runs_dry_the_op_is_declined_and_blocks_taken_stay():
    # tests/discrete.rs:735-767: pool one block short -> declined, `full` counted.
    pool = KvPool(GEO, 3)
    a, b = pool.mirror(), pool.mirror()
    assert pool.attention_plan([a, b], [31, 31], 0) is None     # needs 4, has 3
    s = pool.stats()
    assert s.full == 1 and s.free == 0
    assert len(a.blocks(0)) == 2 and len(b.blocks(0)) == 1      # taken in order until dry, kept
    b.drop()
    assert pool.stats().free == 1
    p = plan_ok(pool, [a], [31])
    assert len(p.blocks) == 2
    a.drop()
    assert pool.stats().free == 3
    pool.delete()


def test_another_epoch_starts_again():
    # discrete.rs:975-978; tests/discrete.rs `clear()` + other prompt -> epoch reset.
    pool = KvPool(GEO, 8)
    m = pool.mirror(epoch=1)
    plan_ok(pool, [m], [40], epochs=[1])
    assert pool.stats().free == 5
    p = plan_ok(pool, [m], [3], epochs=[2])
    assert pool.stats().free == 7 and len(p.sync_to) == 3 and m.synced(0) == 4
    m.drop(); pool.delete()


def test_a_seeded_free_order():
    pool = KvPool(GEO, 6)
    pool.set_free_order([4, 2, 5, 0, 1, 3])
    m = pool.mirror()
    p = plan_ok(pool, [m], [16 * 4])
    assert p.blocks.tolist() == [4, 2, 5, 0, 1]
    with pytest.raises(ValueError):
        pool.set_free_order([3, 3])
    m.drop(); pool.delete()


def test_sharing_copy_on_write_and_refcounts():
    pool = KvPool(GEO, 16)
    parent = pool.mirror()
    plan_ok(pool, [parent], [39])              # 40 positions: blocks 0,1,2; the third half full
    kids = [parent.fork(40) for _ in range(3)]
    assert [pool.refcount(b) for b in (0, 1, 2)] == [4, 4, 4]
    assert pool.stats().free == 13 and pool.stats().shared_blocks == 3
    assert kids[0].synced(0) == 40
    # Every sharer that appends copies the partly filled block first; none writes in place,
    # because the retained parent still holds it.
    p = pool.attention_plan(kids, [40, 40, 40], 0)
    assert p.copy_src.tolist() == [2, 2, 2] and p.copy_dst.tolist() == [3, 4, 5]
    assert p.blocks.tolist() == [0, 1, 3, 0, 1, 4, 0, 1, 5] and len(p.sync_to) == 0
    pool.commit(p, kids, 0); pool.free_plan(p)
    assert [pool.refcount(b) for b in (0, 1, 2, 3)] == [4, 4, 1, 1]
    assert pool.stats().cow_copies == 3
    p = plan_ok(pool, kids, [41, 41, 41])      # now private: no more copies
    assert len(p.copy_src) == 0
    parent.drop()
    assert pool.refcount(2) == 0 and pool.refcount(0) == 3
    for k in kids:
        k.drop()
    assert pool.stats().free == 16
    pool.delete()


def test_a_prefix_that_ends_on_a_block_boundary_copies_nothing():
    pool = KvPool(GEO, 16)
    parent = pool.mirror()
    plan_ok(pool, [parent], [31])              # 32 positions: two full blocks
    kid = parent.fork(32)
    p = plan_ok(pool, [kid], [32])
    assert len(p.copy_src) == 0 and p.blocks.tolist()[:2] == [0, 1] and pool.stats().cow_copies == 0
    kid.drop(); parent.drop(); pool.delete()


def test_compaction_moves_high_live_blocks_into_low_holes():
    pool = KvPool(GEO, 12)
    ms = [pool.mirror() for _ in range(4)]
    plan_ok(pool, ms, [47, 15, 31, 15])        # blocks: [0,1,2] [3] [4,5] [6]
    ms[1].drop(); ms[2].drop()                 # holes at 3,4,5
    live_before = {i: ms[i].blocks(0).tolist() for i in (0, 3)}
    src, dst = pool.compact()
    assert src.tolist() == [6] and dst.tolist() == [3]
    assert ms[0].blocks(0).tolist() == live_before[0] and ms[3].blocks(0).tolist() == [3]
    s = pool.stats()
    assert s.free == 8 and s.compaction_moves == 1
    m = pool.mirror()
    p = plan_ok(pool, [m], [0])
    assert p.blocks.tolist() == [4]            # the free list restarts at L, lowest first
    for x in (ms[0], ms[3], m):
        x.drop()
    assert pool.stats().free == 12
    pool.delete()


def test_random_traffic_matches_the_restatement():
    rng = np.random.default_rng(11)
    B, N = 16, 96
    pool, rp = KvPool(GEO, N), ref.RefPool(N, B)
    live = []  # (mirror, ref mirror, pos)
    for step in range(400):
        r = rng.random()
        if r < 0.25 and len(live) < 12:
            if live and rng.random() < 0.4:
                m, rm, pos = live[int(rng.integers(0, len(live)))]
                t = int(rng.integers(0, pos + 2))
                live.append([m.fork(t), rm.fork(t), min(t, rm.layers[0]["synced"] if rm.layers else 0)])
            else:
                live.append([pool.mirror(), ref.RefMirror(rp), 0])
        elif r < 0.35 and live:
            m, rm, _ = live.pop(int(rng.integers(0, len(live))))
            m.drop(); rm.release()
        elif r < 0.45:
            src, dst = pool.compact()
            rs, rd = ref.compact(rp, [x[1] for x in live])
            assert src.tolist() == rs and dst.tolist() == rd
        elif live:
            k = int(rng.integers(1, len(live) + 1))
            idx = sorted(rng.choice(len(live), size=k, replace=False).tolist())
            for i in idx:
                live[i][2] += int(rng.integers(0, 40))
            pos = [live[i][2] for i in idx]
            got = pool.attention_plan([live[i][0] for i in idx], pos, 0)
            want = ref.attention_plan(rp, [live[i][1] for i in idx], [0] * k, pos, 0)
            assert (got is None) == (want is None)
            if got is not None:
                for f in ("pos", "table_at", "blocks", "sync_to", "sync_seq", "sync_pos", "copy_src", "copy_dst"):
                    assert getattr(got, f).tolist() == want[f], f
                pool.commit(got, [live[i][0] for i in idx], 0)
                ref.commit(rp, want, [live[i][1] for i in idx], 0)
                pool.free_plan(got)
                for i in idx:
                    live[i][2] += 1
        s = pool.stats()
        assert s.free == len(rp.free) and s.full == rp.full and s.cow_copies == rp.cow_copies
        for m, rm, _ in live:
            assert m.blocks(0).tolist() == (rm.layers[0]["blocks"] if rm.layers else [])
        assert [pool.refcount(b) for b in range(N)] == rp.refs
    for m, rm, _ in live:
        m.drop()
    assert pool.stats().free == N
    pool.delete()


# ---- the prefix index over shared blocks (Engine::restore / Engine::retain, engine.rs:1659-1699) -----
def test_a_prefix_hit_shares_blocks_in_every_layer_and_eviction_gives_them_back():
    """lookup -> fork(reuse) -> decode (copy-on-write of the partly filled block, per layer) -> retain the
    finished sequence -> the budget evicts the oldest entry -> its own blocks return to the free list."""
    from qubivex_b200.ondevice import OnDevice
    B, layers, kvh, d = 16, 2, 2, 64
    od = OnDevice(None, GEO, heads=4, blocks=64)        # bookkeeping only: no device behind it
    index = od.retain_prefixes(budget_blocks=14)
    host = lambda n: (np.zeros((kvh, n, d), np.float32), np.zeros((kvh, n, d), np.float32))
    # a conversation of 40 tokens: positions 0..39, three blocks per layer (the third holds 8 positions)
    tokens = np.arange(1000, 1040, dtype=np.uint32)
    owner = od.new_mirror()
    for l in range(layers):
        plan_ok(od.kv, [owner], [39], layer=l)
    k, v = host(40)
    k[:] = 7.0
    assert od.retain("s", tokens, owner, k, v) and index.cost() == 6 and od.kv.stats().free == 64 - 6
    # a request that shares 36 tokens: 2 full blocks + 4 positions of the third, in both layers
    prompt = np.concatenate([tokens[:36], np.array([5, 6, 7], dtype=np.uint32)])
    rk, rv = host(64)
    assert od.restore("other scope", prompt, rk, rv) == (None, 0)
    m, reuse = od.restore("s", prompt, rk, rv)
    assert reuse == 36 and od.kv.stats().free == 64 - 6 and float(rk[0, 35, 0]) == 7.0 and float(rk[0, 36, 0]) == 0.0
    assert [m.synced(l) for l in range(layers)] == [36, 36]
    for l in range(layers):
        p = od.kv.attention_plan([m], [36], l)
        assert len(p.sync_to) == 0                                   # the pool already holds 0..35
        assert len(p.copy_src) == 1 and p.copy_src[0] == owner_block(od, index, "s", tokens, l, 2)
        od.kv.commit(p, [m], l)
        od.kv.free_plan(p)
    assert od.kv.stats().cow_copies == 2 and od.kv.stats().free == 64 - 8
    for pos in (37, 38):
        for l in range(layers):
            assert len(plan_ok(od.kv, [m], [pos], layer=l).copy_src) == 0
    # the finished request is retained too: 6 + 6 blocks fit the budget of 14 ...
    full = np.concatenate([prompt, np.array([9], dtype=np.uint32)])[:39]
    assert od.retain("s", full, m, rk, rv) and index.stats().entries == 2 and index.cost() == 12
    # ... a third conversation of 3 blocks per layer does not: the oldest entry goes, and the two blocks per layer
    # nobody else shares return to the free list (its third block of each layer; the first two the second entry holds)
    other = od.new_mirror()
    for l in range(layers):
        plan_ok(od.kv, [other], [40], layer=l)
    free_before = od.kv.stats().free
    ok, ov = host(41)
    assert od.retain("s", np.arange(5000, 5041, dtype=np.uint32), other, ok, ov)
    assert index.stats().evicted == 1 and index.stats().entries == 2
    assert od.kv.stats().free == free_before + 2
    od.close()                                                       # clears the index: everything comes back
    

def owner_block(od, index, scope, tokens, layer, i):
    """Block i of layer `layer` of the retained sequence `tokens` names (looked up, not remembered)."""
    kept, _, hit = index.lookup(scope, np.concatenate([tokens, np.array([1], dtype=np.uint32)]))
    try:
        return int(kept.mirror.blocks(layer)[i])
    finally:
        index.release(hit)


def test_four_threads_share_one_pool():
    """crates/qubivex-runtime/tests/discrete.rs:772-801 (concurrent_requests_with_decode_attention): four request
    threads plan, commit, fork and drop on one pool; afterwards every block is free again."""
    import threading
    pool = KvPool(GEO, 256)
    errors = []

    def request(seed):
        try:
            rng = np.random.default_rng(seed)
            for _ in range(30):
                m = pool.mirror()
                n = int(rng.integers(1, 120))
                for pos in range(n - 1, n + 6):
                    p = pool.attention_plan([m], [pos], 0)
                    if p is None:                       # the pool ran dry under the others: declined, nothing broken
                        break
                    assert p.pos.tolist() == [pos] and len(p.blocks) == pos // 16 + 1
                    pool.commit(p, [m], 0)
                    pool.free_plan(p)
                child = m.fork(n // 2)
                m.drop()
                p = pool.attention_plan([child], [n // 2], 0)
                if p is not None:
                    pool.commit(p, [child], 0)
                    pool.free_plan(p)
                child.drop()
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=request, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    s = pool.stats()
    assert s.free == s.blocks == 256 and s.shared_blocks == 0
    pool.delete()
