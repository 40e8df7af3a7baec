"""The SSD cold tier of the prefix cache (libkiln_host.so): the reference's slab-store unit tests
(crates/kiln-engine/src/ssd.rs:714-821) against `host.SsdStore`, the on-disk layout checked byte by byte against the
format the reference documents (ssd.rs:21-39), and the engine-level behaviour with the checksum mock: write-behind of
donated blocks, re-discovery of evicted blocks, and a warm restart that finds them hash-first (engine.rs:2559-2640,
2645-2704). CPU only.
"""
import hashlib
import struct

import numpy as np

from kiln_b200 import host as H
from tests.test_engine import BS, VOCAB, ChecksumModel, prompts, reference_generation

G = dict(layers=2, kv_heads=2, head_dim=4, block_size=4)
HEADER_BYTES, SLOTS_PER_FILE = 128, 64


def payload_bytes(dtype_size=2):
    return G["layers"] * 2 * G["kv_heads"] * G["block_size"] * G["head_dim"] * dtype_size


def slot_stride(dtype_size=2):
    return 8 + 32 + 32 + G["block_size"] * 4 + payload_bytes(dtype_size)


def payload(seed):
    return bytes((seed ^ i) & 0xFF for i in range(payload_bytes()))


def open_store(d, fp=b"\x01" * 32, cap=1 << 20):
    return H.SsdStore(str(d), fp, max_bytes=cap, **G)


def test_round_trip_and_restart_scan(tmp_path):
    tokens, h, body = [1, 2, 3, 4], b"\x09" * 32, payload(0x5A)
    store = open_store(tmp_path)
    store.enqueue_write(5, 42, h, tokens, body, dtype_tag=3, dtype_size=2)
    assert not store.contains(h), "a block is readable only once its write has been acknowledged"
    acks = store.sync()
    assert acks == [(5, 42, h, True)]
    assert store.contains(h)
    assert store.read(h, tokens, 3) == (body, 3)
    assert store.read(h, tokens, 4) is None                      # wrong pool dtype: silent miss + counter
    assert store.stats()["fingerprint_rejects_total"] == 1
    store.close()
    store = open_store(tmp_path)                                 # restart: rebuilt from the slab headers alone
    assert store.stats()["blocks_stored"] == 1
    assert store.read(h, tokens, -1) == (body, 3)                # a fresh pool accepts the slab's own dtype tag
    assert store.read(h, [1, 2, 3, 5], 3) is None                # the stored token ids catch a mismatched chunk
    store.close()


def test_slab_layout_is_the_documented_one(tmp_path):
    tokens, h, body = [11, 22, 33, 44], bytes(range(32)), payload(7)
    store = open_store(tmp_path, fp=b"\xAB" * 32)
    store.enqueue_write(0, 1, h, tokens, body, dtype_tag=7, dtype_size=2)
    store.sync()
    store.close()
    raw = (tmp_path / "slab-00000000.kiln").read_bytes()
    assert raw[:8] == b"KILNSLB1"
    assert struct.unpack_from("<7I", raw, 8) == (1, G["layers"], G["kv_heads"], G["head_dim"], G["block_size"], 7, SLOTS_PER_FILE)
    assert raw[36:68] == b"\xAB" * 32 and struct.unpack_from("<I", raw, 68) == (2,) and raw[72:128] == bytes(56)
    slot = raw[HEADER_BYTES:HEADER_BYTES + slot_stride()]
    assert slot[0] == 1 and slot[1:8] == bytes(7) and slot[8:40] == h
    assert slot[40:72] == hashlib.sha256(body).digest()
    assert struct.unpack_from("<4I", slot, 72) == tuple(tokens)
    assert slot[72 + 16:] == body
    assert len(raw) == HEADER_BYTES + slot_stride()


def test_corrupt_header_and_wrong_fingerprint_are_skipped(tmp_path):
    h = b"\x07" * 32
    store = open_store(tmp_path)
    store.enqueue_write(0, 1, h, [1, 2, 3, 4], payload(1), 3, 2)
    store.sync()
    store.close()
    other = open_store(tmp_path, fp=b"\x02" * 32)                # another model: the whole file is ignored
    assert other.stats()["blocks_stored"] == 0 and other.stats()["fingerprint_rejects_total"] == 1
    other.close()
    path = tmp_path / "slab-00000000.kiln"
    raw = bytearray(path.read_bytes())
    raw[0] ^= 0xFF
    path.write_bytes(bytes(raw))                                 # a flipped magic byte: the same silent skip
    store = open_store(tmp_path)
    assert store.stats()["blocks_stored"] == 0 and store.stats()["fingerprint_rejects_total"] == 1
    store.close()
    raw[0] ^= 0xFF
    raw[-1] ^= 0xFF
    path.write_bytes(bytes(raw))                                 # a torn payload: the header scans, the digest fails
    store = open_store(tmp_path)
    assert store.stats()["blocks_stored"] == 1
    assert store.read(h, [1, 2, 3, 4], 3) is None
    assert store.stats()["fingerprint_rejects_total"] == 1 and not store.contains(h)
    store.close()


def test_a_block_queued_twice_settles_both_slots(tmp_path):
    """Two writes of one hash before the first acknowledgement: each acknowledgement settles its own slot and the later
    payload is the one served, also after a restart (later slots win the header scan)."""
    tokens, h = [5, 6, 7, 8], b"\x0a" * 32
    store = open_store(tmp_path)
    store.enqueue_write(1, 1, h, tokens, payload(0x11), 3, 2)
    store.enqueue_write(1, 2, h, tokens, payload(0x22), 3, 2)
    acks = store.sync()
    assert [a[3] for a in acks] == [True, True]
    assert store.stats()["blocks_stored"] == 1 and store.stats()["writes_total"] == 2
    assert store.read(h, tokens, 3) == (payload(0x22), 3)
    assert store.stats()["bytes_stored"] == HEADER_BYTES + 2 * slot_stride()
    store.close()
    store = open_store(tmp_path)
    assert store.read(h, tokens, 3) == (payload(0x22), 3)
    store.close()


def test_byte_cap_drops_lru_slabs(tmp_path):
    cap = HEADER_BYTES + slot_stride() * SLOTS_PER_FILE + slot_stride()
    store = open_store(tmp_path, cap=cap)
    hash_of = lambda i: struct.pack("<I", i) + bytes(28)
    for i in range(SLOTS_PER_FILE):
        store.enqueue_write(i, 1, hash_of(i), [i] * 4, payload(i), 3, 2)
        store.sync()
    assert store.stats()["blocks_stored"] == SLOTS_PER_FILE and store.stats()["bytes_stored"] <= cap
    store.enqueue_write(99, 1, hash_of(999), [9] * 4, payload(0xAA), 3, 2)   # starts slab 1: the cap evicts slab 0 wholesale
    store.sync()
    assert store.contains(hash_of(999)) and not store.contains(hash_of(0))
    assert store.stats()["bytes_stored"] <= cap
    assert not (tmp_path / "slab-00000000.kiln").exists()
    store.close()


# ---- engine level: the checksum mock's pool is a numpy array, block IO reads and writes its rows ----

def make_engine(directory, num_blocks=24, fingerprint=b"\x05" * 32):
    model = ChecksumModel(num_blocks)
    cfg = H.EngineConfig(block_size=BS, num_blocks=num_blocks, prefill_chunk=BS, prefill_fine_chunk=BS, prefix_cache=True,
                         deterministic_decode_width=32, gamma=0, spec_max_batch=4, spec_min_acceptance=0.0, max_key_len=0,
                         batch_verify=True)
    sm = H.StepModel.from_python(model, VOCAB, model.copy_block, pipelined=True)
    eng = H.Engine(cfg, sm)
    row_bytes = BS * 8   # one block of the mock: BS int64 values; geometry chosen so that payload_bytes matches
    eng.set_ssd(str(directory), fingerprint, layers=1, kv_heads=1, head_dim=1, dtype_tag=5, dtype_size=4,
                read_block=lambda b: model.pool[b].astype(np.int64).tobytes()[:row_bytes],
                write_block=lambda b, data: model.pool.__setitem__(b, np.frombuffer(data, dtype=np.int64)))
    return eng, model


def test_engine_mock_geometry_matches():
    # the mock's block is BS int64 = 32 bytes; layers 1 x (K + V) x 1 head x BS rows x 1 feature x 4 bytes = 32 bytes
    assert 1 * 2 * 1 * BS * 1 * 4 == BS * 8


def run(eng, prompt, n):
    a = eng.submit(prompt, n)
    toks, kind = eng.run_to_completion([a])[a]
    return a, toks


def test_donated_blocks_are_written_behind_and_survive_eviction_and_restart(tmp_path):
    p = prompts(1, 41, lo=13, hi=14)[0]          # 13 tokens: 3 full blocks of prompt
    truth = reference_generation(p, 8)
    eng, model = make_engine(tmp_path)
    a, toks = run(eng, p, 8)
    assert toks == truth
    for _ in range(6):
        eng.step()                               # idle steps make write-behind progress (engine.rs:1389-1393)
    eng.ssd_sync()
    st = eng.ssd_stats()
    settled = len(p) - 1 + 8
    assert st["blocks_stored"] == settled // BS and st["writes_total"] == settled // BS and st["flush_queue_depth"] == 0

    # evict everything resident: the nodes stay (SSD-backed), a re-run reloads the blocks instead of recomputing them
    bm = eng.block_manager()
    filler = [eng.submit(q, 2) for q in prompts(4, 43, lo=17, hi=18)]
    eng.run_to_completion(filler)
    forwards_before, reads_before = eng.forwards, eng.ssd_stats()["reads_total"]
    a, toks = run(eng, p, 8)
    assert toks == truth, "a block reloaded from the slab served stale or misplaced rows"
    assert eng.seq_state(a).cached_tokens >= 2 * BS
    assert eng.ssd_stats()["reads_total"] >= reads_before

    # warm restart: a new engine (empty radix tree, zeroed pool) over the same directory discovers the blocks hash-first
    eng.ssd_sync()
    del eng
    eng2, model2 = make_engine(tmp_path)
    assert eng2.ssd_stats()["blocks_stored"] >= settled // BS
    a, toks = run(eng2, p, 8)
    assert toks == truth
    assert eng2.seq_state(a).cached_tokens == (len(p) - 1) // BS * BS
    s2 = eng2.ssd_stats()
    assert s2["reads_total"] == (len(p) - 1) // BS and s2["ssd_hits_total"] == 1
    cold, _ = make_engine(tmp_path / "other")
    a, cold_toks = run(cold, p, 8)
    assert cold_toks == toks and cold.seq_state(a).cached_tokens == 0

    # another model's fingerprint: nothing is trusted
    eng3, _ = make_engine(tmp_path, fingerprint=b"\x06" * 32)
    assert eng3.ssd_stats()["blocks_stored"] == 0 and eng3.ssd_stats()["fingerprint_rejects_total"] >= 1
    a, toks = run(eng3, p, 8)
    assert toks == truth and eng3.seq_state(a).cached_tokens == 0


def test_store_against_a_shadow_dictionary(tmp_path):
    """Random interleavings of writes, acknowledgement drains, reads and restarts against a dictionary: a block is
    readable exactly from the moment its acknowledgement has been applied, survives a restart, and rewriting a hash makes
    the later slot win."""
    from hypothesis import given, settings, strategies as st

    ops = st.lists(st.tuples(st.sampled_from(["write", "sync", "read", "reopen"]), st.integers(0, 11), st.integers(0, 255)),
                   min_size=1, max_size=40)
    counter = [0]

    @settings(max_examples=25, deadline=None)
    @given(ops)
    def run(seq):
        counter[0] += 1
        d = tmp_path / f"case{counter[0]}"
        store = open_store(d)
        committed, pending = {}, {}
        hash_of = lambda i: struct.pack("<I", i) + b"\x33" * 28
        for op, i, seed in seq:
            if op == "write":
                store.enqueue_write(i, 1, hash_of(i), [i, i + 1, i + 2, i + 3], payload(seed), 3, 2)
                pending[i] = seed
            elif op == "sync":
                acks = store.sync()
                assert all(a[3] for a in acks)
                committed.update(pending)
                pending.clear()
            elif op == "read":
                got = store.read(hash_of(i), [i, i + 1, i + 2, i + 3], 3)
                if i in committed and i not in pending:
                    assert got == (payload(committed[i]), 3)
                elif i not in committed and i not in pending:
                    assert got is None
            else:
                store.close()                       # joins the writer: queued writes land, and the scan finds them
                committed.update(pending)
                pending.clear()
                store = open_store(d)
                assert store.stats()["blocks_stored"] == len(committed)
        store.close()

    run()
