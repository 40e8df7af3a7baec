"""RadixCache (libkiln_host.so) against the reference's own unit tests (crates/kiln-engine/src/radix.rs:469-578, ported
case for case), a hypothesis version of its property suite (crates/kiln-engine/tests/radix_props.rs: random donation /
match-and-hold / release / eviction against a flat set of block-aligned prefixes, with block conservation), and the
chain hash against hashlib's SHA-256 (radix.rs:145-152: sha256(parent digest ++ tokens as little-endian u32))."""
import hashlib
import struct

from hypothesis import given, settings
from hypothesis import strategies as st

from kiln_b200.host import BlockManager, RadixCache

ROOT = 0


def chunk(base):
    return list(range(base, base + 4))


def sha_chain(parent: bytes, tokens) -> bytes:
    return hashlib.sha256(parent + b"".join(struct.pack("<I", t) for t in tokens)).digest()


def test_chain_hash_is_sha256_of_parent_digest_and_le_tokens():
    seed = bytes(range(32))
    tree = RadixCache(4, seed)
    assert tree.node_hash(ROOT) == seed
    a = tree.insert_child(ROOT, chunk(0))
    b = tree.insert_child(a, [0xFFFFFFFF, 0, 0x80000000, 123456789])
    assert tree.node_hash(a) == sha_chain(seed, chunk(0))
    assert tree.node_hash(b) == sha_chain(sha_chain(seed, chunk(0)), [0xFFFFFFFF, 0, 0x80000000, 123456789])
    # lengths on both sides of the 55/56- and 64-byte padding edges of SHA-256 (32-byte digest + 4 bytes per token)
    for n in (1, 5, 6, 7, 8, 9, 16, 23, 24, 64):
        toks = [(i * 2654435761) & 0xFFFFFFFF for i in range(n)]
        assert RadixCache(n, seed).chain_hash_of(ROOT, toks) == sha_chain(seed, toks)
    # a known digest, independent of any helper in this file: sha256 of 32 zero bytes
    assert RadixCache(4, bytes(32)).chain_hash_of(ROOT, []) == bytes.fromhex(
        "66687aadf862bd776c8fc18b8e9f8e20089714856ee233b3902a591d0d5f2925")


def test_insert_descend_and_hash_chaining():
    tree = RadixCache(4, bytes([7] * 32))
    a = tree.insert_child(ROOT, chunk(0))
    b = tree.insert_child(a, chunk(4))
    assert tree.child(ROOT, chunk(0)) == a
    assert tree.child(a, chunk(4)) == b
    assert tree.child(a, chunk(8)) is None
    assert tree.chain_hash_of(ROOT, chunk(0)) == tree.node_hash(a)
    assert tree.chain_hash_of(a, chunk(4)) == tree.node_hash(b)
    assert tree.node_hash(a) != tree.node_hash(b)
    other = RadixCache(4, bytes([8] * 32))
    assert other.chain_hash_of(ROOT, chunk(0)) != tree.node_hash(a), "seed must isolate models"


def test_eviction_is_lru_leaf_first_and_skips_shared():
    mgr = BlockManager(4, 4)
    tree = RadixCache(4)
    a = tree.insert_child(ROOT, chunk(0))
    b = tree.insert_child(a, chunk(4))
    c = tree.insert_child(ROOT, chunk(8))
    for node in (a, b, c):
        tree.set_resident(node, mgr.allocate())
    assert tree.resident_blocks() == 3
    assert tree.evict_candidate(mgr) == b      # a has a resident child; b is older than c
    tree.touch(b)
    assert tree.evict_candidate(mgr) == c
    mgr.retain(tree.node_block(c))             # a running request shares c's block
    assert tree.evict_candidate(mgr) == b
    mgr.release(tree.node_block(c))
    freed = tree.evict(mgr, b)
    assert mgr.refcount(freed) == 0
    assert tree.child(a, chunk(4)) is None
    assert tree.resident_blocks() == 2
    assert tree.evict_candidate(mgr) in (a, c)


def test_ssd_backed_eviction_keeps_the_node():
    mgr = BlockManager(2, 4)
    tree = RadixCache(4)
    a = tree.insert_child(ROOT, chunk(0))
    tree.set_resident(a, mgr.allocate())
    tree.set_on_ssd(a)
    tree.evict(mgr, a)
    assert mgr.num_free == 2
    assert tree.child(ROOT, chunk(0)) == a
    assert tree.node_on_ssd(a)
    assert tree.node_block(a) is None


def test_generations_guard_recycled_slots():
    mgr = BlockManager(2, 4)
    tree = RadixCache(4)
    a = tree.insert_child(ROOT, chunk(0))
    generation = tree.node_generation(a)
    tree.set_resident(a, mgr.allocate())
    assert tree.is_live(a, generation)
    tree.evict(mgr, a)
    assert not tree.is_live(a, generation)
    b = tree.insert_child(ROOT, chunk(4))
    assert a == b, "slot is recycled"
    assert not tree.is_live(a, generation), "old generation stays dead"
    assert tree.is_live(b, tree.node_generation(b))


def test_prune_subtree_releases_resident_descendants():
    mgr = BlockManager(4, 4)
    tree = RadixCache(4)
    a = tree.insert_child(ROOT, chunk(0))
    b = tree.insert_child(a, chunk(4))
    for node in (a, b):
        tree.set_resident(node, mgr.allocate())
    tree.prune_subtree(mgr, a)
    assert mgr.num_free == 4
    assert tree.resident_blocks() == 0
    assert tree.child(ROOT, chunk(0)) is None


def test_reset_drops_everything_but_keeps_the_seed():
    tree = RadixCache(4, bytes([3] * 32))
    a = tree.insert_child(ROOT, chunk(0))
    digest = tree.node_hash(a)
    tree.reset()
    assert tree.child(ROOT, chunk(0)) is None
    assert tree.resident_blocks() == 0
    assert tree.chain_hash_of(ROOT, chunk(0)) == digest


BLOCK, CAPACITY = 4, 64


def stream(seed, chunks):
    """Chunk i of a stream is one of two variants picked by bit i of the seed: dense prefix sharing."""
    return [i * 16 + ((seed >> i) & 1) * 8 + j for i in range(chunks) for j in range(BLOCK)]


OPS = st.one_of(
    st.tuples(st.just("donate"), st.integers(0, 2 ** 64 - 1), st.integers(1, 5)),
    st.tuples(st.just("match"), st.integers(0, 2 ** 64 - 1), st.integers(1, 5)),
    st.tuples(st.just("release"), st.just(0), st.just(0)),
    st.tuples(st.just("evict"), st.just(0), st.just(0)),
)


@settings(max_examples=200, deadline=None)
@given(st.lists(OPS, min_size=1, max_size=80))
def test_radix_matches_reference_and_conserves_blocks(ops):
    mgr = BlockManager(CAPACITY, BLOCK)
    tree = RadixCache(BLOCK, bytes([0x5A] * 32))
    present = {}          # block-aligned prefix (tuple) -> physical block
    cache_live = 0
    held = []
    for op, seed, chunks in ops:
        if op == "donate":
            tokens = stream(seed, chunks)
            cur = ROOT
            for i in range(chunks):
                ch = tokens[i * BLOCK:(i + 1) * BLOCK]
                try:
                    block = mgr.allocate()
                except Exception:
                    break
                node = tree.child(cur, ch)
                if node is not None:
                    assert tree.node_block(node) is not None, "non-resident node in an SSD-less tree"
                    mgr.release(block)
                    tree.touch(node)
                else:
                    node = tree.insert_child(cur, ch)
                    tree.set_resident(node, block)
                    cache_live += 1
                    present[tuple(tokens[:(i + 1) * BLOCK])] = block
                cur = node
        elif op == "match":
            tokens = stream(seed, chunks)
            cur, got = ROOT, []
            for i in range(chunks):
                node = tree.child(cur, tokens[i * BLOCK:(i + 1) * BLOCK])
                if node is None:
                    break
                block = tree.node_block(node)
                if block is None:
                    break
                mgr.retain(block)
                tree.touch(node)
                got.append(block)
                cur = node
            want = 0
            while (want + 1) * BLOCK <= len(tokens) and tuple(tokens[:(want + 1) * BLOCK]) in present:
                want += 1
            assert len(got) == want, "match length diverged from the reference"
            assert all(mgr.refcount(b) >= 2 for b in got)
            if got:
                held.append(got)
        elif op == "release":
            if held:
                for b in held.pop(0):
                    mgr.release(b)
        else:
            node = tree.evict_candidate(mgr)
            if node is not None:
                block = tree.node_block(node)
                assert mgr.refcount(block) == 1, "only sole-owned blocks are eligible"
                assert tree.evict(mgr, node) == block
                assert mgr.refcount(block) == 0
                cache_live -= 1
                prefix = next(p for p, b in present.items() if b == block)
                del present[prefix]
                assert not any(o[:len(prefix)] == prefix and len(o) > len(prefix) for o in present), "evicted an interior node"
        assert CAPACITY - mgr.num_free == cache_live
        assert tree.resident_blocks() == cache_live == len(present)
    for blocks in held:
        for b in blocks:
            mgr.release(b)
    while (node := tree.evict_candidate(mgr)) is not None:
        tree.evict(mgr, node)
    assert mgr.num_free == CAPACITY, "eviction must drain the tree"
    assert tree.resident_blocks() == 0
