"""Known-answer tests of the integer bookkeeping, ported from the reference's own unit tests and run against
BOTH the Python oracle (oracle/bookkeeping.py) and the C++ host library (kiln_b200/host.py):

  crates/kiln-engine/src/block.rs:428-688      BlockManager / BlockTable
  crates/kiln-engine/src/drafter.rs:149-198    spec_gamma_at_width
  crates/kiln-engine/src/engine.rs:2798-2853   canonical_prefill_len
  crates/kiln-engine/tests/block_props.rs      shadow-model property test (hypothesis here)
These pin the oracle; the C++ library must agree with it operation for operation.
"""
import pytest
from hypothesis import given, settings, strategies as st

from kiln_b200 import host as H
from oracle import bookkeeping as B


class Impl:
    """Uniform face over the two implementations."""

    def __init__(self, kind):
        self.kind = kind

    def manager(self, cap, bs):
        return B.BlockManager(cap, bs) if self.kind == "oracle" else H.BlockManager(cap, bs)

    def table(self):
        return B.BlockTable() if self.kind == "oracle" else H.BlockTable()

    def err(self):
        return B.BlockError if self.kind == "oracle" else H.HostError

    def gamma(self, *a):
        return B.spec_gamma_at_width(*a) if self.kind == "oracle" else H.spec_gamma_at_width(*a)

    def prefill_len(self, *a):
        return B.canonical_prefill_len(*a) if self.kind == "oracle" else H.canonical_prefill_len(*a)


@pytest.fixture(params=["oracle", "host"])
def impl(request):
    return Impl(request.param)


def raises(impl, kind, fn, **info):
    with pytest.raises(impl.err()) as e:
        fn()
    assert e.value.kind == kind
    for k, v in info.items():
        assert e.value.info[k] == v
    return e.value


def cow_of(plan):
    return plan.cow


def test_rejects_invalid_block_size(impl):
    raises(impl, "InvalidBlockSize", lambda: impl.manager(4, 0))
    raises(impl, "InvalidBlockSize", lambda: impl.manager(4, 24))


def test_rejects_zero_capacity(impl):
    raises(impl, "InvalidCapacity", lambda: impl.manager(0, 32))


def test_allocates_in_order_until_exhausted(impl):
    m = impl.manager(3, 32)
    assert [m.allocate() for _ in range(3)] == [0, 1, 2]
    raises(impl, "OutOfBlocks", m.allocate, capacity=3, needed=1)
    assert m.num_free == 0


def test_refcount_lifecycle_and_reuse(impl):
    m = impl.manager(2, 32)
    b = m.allocate()
    assert m.refcount(b) == 1
    m.retain(b)
    assert m.refcount(b) == 2
    m.release(b)
    assert m.refcount(b) == 1 and m.num_free == 1
    m.release(b)
    assert m.refcount(b) == 0 and m.num_free == 2
    raises(impl, "NotAllocated", lambda: m.release(b))
    raises(impl, "NotAllocated", lambda: m.retain(b))
    raises(impl, "NotAllocated", lambda: m.copy_on_write(b))


def test_foreign_ids_are_rejected(impl):
    m = impl.manager(4, 32)
    assert m.refcount(7) is None
    raises(impl, "NotAllocated", lambda: m.retain(7))
    raises(impl, "NotAllocated", lambda: m.release(7))


def test_cow_sole_owner_writes_in_place(impl):
    m = impl.manager(2, 32)
    b = m.allocate()
    assert m.copy_on_write(b) == ("writable", b, b)
    assert m.refcount(b) == 1 and m.num_free == 1


def test_cow_shared_allocates_copy_and_moves_ownership(impl):
    m = impl.manager(2, 32)
    b = m.allocate()
    m.retain(b)
    kind, src, dst = m.copy_on_write(b)
    assert kind == "copied" and src == b and dst != b
    assert m.refcount(b) == 1 and m.refcount(dst) == 1 and m.num_free == 0


def test_cow_exhausted_pool_leaves_state_unchanged(impl):
    m = impl.manager(1, 32)
    b = m.allocate()
    m.retain(b)
    raises(impl, "OutOfBlocks", lambda: m.copy_on_write(b), capacity=1, needed=1)
    assert m.refcount(b) == 2 and m.num_free == 0


def test_table_append_allocates_blocks_and_tracks_tokens(impl):
    m, t = impl.manager(4, 4), impl.table()
    p = t.append_tokens(m, 0)
    assert cow_of(p) is None and p.appended == []
    p = t.append_tokens(m, 6)
    assert cow_of(p) is None and len(p.appended) == 2 and list(t.blocks) == p.appended and t.num_tokens == 6
    p = t.append_tokens(m, 2)
    assert cow_of(p) is None and p.appended == [] and t.num_tokens == 8
    t.release(m)
    assert m.num_free == 4


def test_table_append_cows_shared_partial_tail(impl):
    m, t = impl.manager(4, 4), impl.table()
    t.append_tokens(m, 6)
    forked = t.fork(m)
    shared = list(t.blocks)[-1]
    assert m.refcount(shared) == 2
    p = t.append_tokens(m, 1)
    assert cow_of(p) is not None and cow_of(p)[0] == shared
    assert list(t.blocks)[-1] == cow_of(p)[1]
    assert list(forked.blocks)[-1] == shared and m.refcount(shared) == 1
    aligned = impl.table()
    aligned.append_tokens(m, 4)
    aligned_fork = aligned.fork(m)
    t.release(m)
    p = aligned.append_tokens(m, 1)        # a shared but full tail is never written, so never copied
    assert cow_of(p) is None and len(p.appended) == 1
    forked.release(m); aligned.release(m); aligned_fork.release(m)
    assert m.num_free == 4


def test_table_truncate_releases_only_past_the_kept_tail(impl):
    m, t = impl.manager(8, 4), impl.table()
    t.append_tokens(m, 14)
    assert m.num_free == 4
    t.truncate(m, 10)
    assert (t.num_tokens, len(t.blocks), m.num_free) == (10, 3, 5)
    t.truncate(m, 8)
    assert (len(t.blocks), m.num_free) == (2, 6)
    t.truncate(m, 8)
    assert (len(t.blocks), m.num_free) == (2, 6)
    raises(impl, "TokenCountOverflow", lambda: t.truncate(m, 9))
    assert t.num_tokens == 8
    t.truncate(m, 0)
    assert (t.num_tokens, len(t.blocks), m.num_free) == (0, 0, 8)


def test_table_truncate_then_append_reuses_the_partial_tail(impl):
    """The verify-round shape (block.rs:639-656): 3 committed rows + a 5-slot speculative append, rollback to 5."""
    m, t = impl.manager(4, 4), impl.table()
    t.append_tokens(m, 3)
    t.append_tokens(m, 5)
    assert t.num_tokens == 8
    t.truncate(m, 5)
    assert len(t.blocks) == 2
    p = t.append_tokens(m, 3)
    assert p.appended == [] and t.num_tokens == 8
    t.release(m)
    assert m.num_free == 4


def test_table_append_is_atomic_on_exhaustion(impl):
    m, t = impl.manager(3, 4), impl.table()
    t.append_tokens(m, 6)
    forked = t.fork(m)
    before = list(t.blocks)
    raises(impl, "OutOfBlocks", lambda: t.append_tokens(m, 3), capacity=3, needed=2)
    assert list(t.blocks) == before and t.num_tokens == 6 and m.num_free == 1
    p = t.append_tokens(m, 2)
    assert cow_of(p) is not None and p.appended == [] and t.num_tokens == 8
    t.release(m); forked.release(m)
    assert m.num_free == 3


def test_rollback_returns_blocks_to_the_free_list_in_table_order(impl):
    """Free-list order fixes the next allocations, so it is part of 'block tables bit-exact' (block.rs:389-394, 167-169)."""
    m, t = impl.manager(8, 4), impl.table()
    t.append_tokens(m, 3)
    t.append_tokens(m, 13)          # blocks 0..3
    t.truncate(m, 5)                # releases 2 then 3
    nxt = [m.allocate(), m.allocate()]
    assert nxt == [3, 2]            # LIFO: the last released is reissued first


def test_width_ramp(impl):
    g = impl.gamma
    assert [g(4, 4, w) for w in (1, 2, 3, 4, 5, 100)] == [4, 3, 2, 1, 0, 0]     # drafter.rs:154-162
    for gamma in range(1, 9):
        for smb in range(1, 9):
            prev = 10 ** 9
            for w in range(1, smb + 1):
                v = g(gamma, smb, w)
                assert 1 <= v <= gamma and v <= prev
                prev = v
            assert g(gamma, smb, smb + 1) == 0
    assert g(0, 4, 1) == 0 and g(4, 0, 1) == 0 and g(4, 4, 0) == 4              # drafter.rs:186-197
    assert (g(3, 4, 1), g(3, 4, 4), g(3, 4, 5)) == (3, 1, 0)


def walk(impl, start, limit, chunk, fine):
    at, segs = start, []
    while at < limit:
        n = impl.prefill_len(at, limit, chunk, fine)
        assert n >= 1 and at + n <= limit
        segs.append((at, n))
        at += n
    return segs


def test_prefill_schedule_shapes_and_boundaries(impl):
    assert walk(impl, 0, 248, 2048, 64) == [(0, 64), (64, 64), (128, 64), (192, 56)]     # engine.rs:2816-2832
    s = walk(impl, 0, 4095, 2048, 64)
    assert s[0] == (0, 2048) and s[1] == (2048, 64) and s[-1] == (4032, 63)
    assert walk(impl, 0, 248, 2048, 2048) == [(0, 248)]
    assert walk(impl, 0, 4095, 2048, 2048) == [(0, 2048), (2048, 2047)]
    assert walk(impl, 0, 4096, 2048, 64) == [(0, 2048), (2048, 2048)]


def test_prefill_schedule_is_resume_invariant(impl):
    for chunk, fine in [(16, 4), (8, 8), (48, 48)]:                                     # engine.rs:2837-2852
        for limit in range(1, 3 * chunk + 6):
            cold = walk(impl, 0, limit, chunk, fine)
            for i, (off, _) in enumerate(cold):
                assert walk(impl, off, limit, chunk, fine) == cold[i:]


OPS = st.lists(st.tuples(st.sampled_from(["append", "truncate", "fork", "release", "new"]), st.integers(0, 40), st.integers(0, 7)),
               min_size=1, max_size=60)


@settings(max_examples=150, deadline=None)
@given(ops=OPS, cap=st.integers(1, 24), bs=st.sampled_from([1, 2, 4, 16]))
def test_host_library_tracks_the_oracle(ops, cap, bs):
    """Property test in the spirit of crates/kiln-engine/tests/block_props.rs: the C++ library and the Python
    restatement stay in lock step — same tables, same refcounts, same free-list order, same errors."""
    om, hm = B.BlockManager(cap, bs), H.BlockManager(cap, bs)
    ot, ht = [B.BlockTable()], [H.BlockTable()]
    for op, a, idx in ops:
        i = idx % len(ot)
        oerr = herr = None
        try:
            if op == "append":
                r1 = ot[i].append_tokens(om, a)
            elif op == "truncate":
                r1 = ot[i].truncate(om, a)
            elif op == "fork":
                ot.append(ot[i].fork(om)); r1 = None
            elif op == "release":
                r1 = ot[i].release(om)
            else:
                ot.append(B.BlockTable()); r1 = None
        except B.BlockError as e:
            oerr = e.kind
        try:
            if op == "append":
                r2 = ht[i].append_tokens(hm, a)
            elif op == "truncate":
                r2 = ht[i].truncate(hm, a)
            elif op == "fork":
                ht.append(ht[i].fork(hm)); r2 = None
            elif op == "release":
                r2 = ht[i].release(hm)
            else:
                ht.append(H.BlockTable()); r2 = None
        except H.HostError as e:
            herr = e.kind
        assert oerr == herr, (op, a)
        if oerr is None and op == "append":
            assert (r1.cow, r1.appended) == (r2.cow, r2.appended)
        assert len(ot) == len(ht)
        for x, y in zip(ot, ht):
            assert list(x.blocks) == list(y.blocks) and x.num_tokens == y.num_tokens
        assert om.free == hm.free_list()
        assert [om.refcount(b) for b in range(cap)] == [hm.refcount(b) for b in range(cap)]
