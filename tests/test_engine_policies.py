"""Engine policies around the verify round: stand-down, drafter faults, stop tokens, submit validation, the radix
prefix cache with copy-on-write, and the DraftModel bookkeeping (crates/kiln-engine/src/engine.rs:1586-1634,
907-963, 1329-1357, 1868-2033, 601-731; crates/kiln-models/src/draft.rs:286-411). Fake models only."""
import ctypes as C

import numpy as np
import pytest

from kiln_b200 import host as H
from tests.test_engine import BS, VOCAB, ChecksumModel, make_engine, prompts, reference_generation


def test_stand_down_after_sustained_low_acceptance():
    """After >= 16 proposed tokens with acceptance below spec_min_acceptance the request stops speculating for good
    and its draft state is released (engine.rs:1616-1633; drafter.rs:45-50)."""
    released = []
    calls = []

    def propose(seq, committed, gamma):
        calls.append(gamma)
        return [11, 23, 5, 42][:gamma]

    eng, _ = make_engine(spec_min_acceptance=0.125)
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: released.append(s)))
    p = prompts(1, 7)[0]
    a = eng.submit(p, 60)
    out = eng.run_to_completion([a])
    assert out[a][0] == reference_generation(p, 60)
    st = eng.spec_stats()
    assert st["standdowns_total"] == 1
    assert 16 <= st["proposed_total"] < 24          # judged as soon as the warm-up window is full
    assert released.count(a) >= 1
    assert len(calls) * 4 >= st["proposed_total"]


def test_drafter_fault_disables_speculation_for_the_request_only():
    """A DraftError never fails a generation (engine.rs:1586-1594, drafter.rs:72-76)."""
    def propose(seq, committed, gamma):
        if seq == 0:
            raise RuntimeError("draft fault")
        return [1] * gamma

    eng, _ = make_engine()
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: None))
    ps = prompts(2, 8)
    arr = [eng.submit(p, 20) for p in ps]
    out = eng.run_to_completion(arr)
    assert [out[a][0] for a in arr] == [reference_generation(p, 20) for p in ps]
    st = eng.spec_stats()
    assert st["draft_errors_total"] == 1
    assert eng.seq_state(arr[0]).standdown == 2 and eng.seq_state(arr[1]).spec_proposed > 0


def test_stop_tokens_and_length():
    """Stop tokens are counted but not emitted and end the walk mid-round (engine.rs:926-931, 2343-2345)."""
    p = prompts(1, 9)[0]
    truth = reference_generation(p, 30)
    stop = truth[10]
    first = truth.index(stop)
    eng, _ = make_engine()
    sd = H.ScriptedDrafter(1.0, 1, VOCAB)
    eng.set_drafter(sd)
    a = eng.submit(p, 30, stop_tokens=[stop])
    sd.set_continuation(a, truth)
    out = eng.run_to_completion([a])
    assert out[a] == (truth[:first], "stop")
    assert eng.seq_state(a).generated == first + 1
    assert eng.block_manager().num_free == 256


def test_submit_validation():
    """engine.rs:1329-1357: errors finish the request in-band."""
    eng, _ = make_engine(num_blocks=4)
    for prompt, mt in [([], 4), ([1, 2], 0), (list(range(10)), 10)]:
        a = eng.submit(prompt, mt)
        assert eng.take_output(a) == ([], "error")
    assert eng.num_waiting == 0


def test_prefix_cache_hit_shares_blocks_and_copies_on_write():
    """A finished request donates its settled blocks; an identical prompt is served from the cache (containment:
    nothing is recomputed), its first write into the shared partial tail goes through copy-on-write, and the
    checksum model proves the shared rows are intact (engine.rs:601-731, 1868-2033; block.rs:253-312)."""
    eng, model = make_engine(prefix_cache=True)
    p = prompts(1, 11, 22, 23)[0]            # 22 tokens: prefill covers 21 = 5 full blocks + 1 row
    truth = reference_generation(p, 10)
    a = eng.submit(p, 10)
    assert eng.run_to_completion([a])[a][0] == truth
    assert eng.cache_stats()["resident_blocks"] == (len(p) - 1 + 10) // BS + 1     # settled = 20 + 10 rows: 7 full + a partial leaf
    rows_before = sum(model.rows)
    b = eng.submit(p, 10)
    out = eng.run_to_completion([b])
    assert out[b][0] == truth
    st = eng.seq_state(b)
    assert st.cached_tokens == len(p) - 1
    assert eng.cache_stats()["hits_total"] == 1 and eng.cache_stats()["tokens_reused_total"] == len(p) - 1
    assert sum(model.rows) - rows_before == 10          # only decode rows were computed: no prefill at all
    assert len(model.copies) >= 1                       # the shared tail block was copied before the first write
    # partial matches are trimmed to a resumable boundary of the canonical prefill schedule (engine.rs:1975-1985):
    # sharing 2 blocks (8 tokens) of a 21-token prefill with prefill_chunk 16 serves nothing; sharing 4 blocks serves 16
    q = p[:9] + [(t + 1) % VOCAB for t in p[9:]]
    c = eng.submit(q, 6)
    assert eng.run_to_completion([c])[c][0] == reference_generation(q, 6)
    assert eng.seq_state(c).cached_tokens == 0
    q = p[:18] + [(t + 2) % VOCAB for t in p[18:]]
    c = eng.submit(q, 6)
    assert eng.run_to_completion([c])[c][0] == reference_generation(q, 6)
    assert eng.seq_state(c).cached_tokens == 16


def test_cache_eviction_makes_room():
    eng, model = make_engine(num_blocks=24, prefix_cache=True)
    ps = prompts(6, 12, 17, 30)
    for p in ps:                                  # sequentially: each finish donates, later admissions must evict
        a = eng.submit(p, 8)
        assert eng.run_to_completion([a])[a][0] == reference_generation(p, 8)
    assert eng.cache_stats()["resident_blocks"] <= 24


class FakeDraftBackend:
    """kh_draft_backend over the checksum model: forward = catch-up prefill, chain = gamma greedy decode steps."""

    def __init__(self, num_blocks):
        self.model = ChecksumModel(num_blocks)
        self.forward_calls, self.chain_calls = [], []

        def _forward(_m, _kv, ids, n, seqs, n_seqs, rows, ncom, nacc):
            py_ids = [ids[i] for i in range(n)]
            py_seqs = [(seqs[i].len, seqs[i].offset, seqs[i].sample_rows, [seqs[i].blocks[b] for b in range(seqs[i].n_blocks)])
                       for i in range(n_seqs)]
            self.forward_calls.append((n, py_seqs[0][1]))
            self.model(py_ids, py_seqs)
            return 0

        def _chain(_m, _kv, first, offset, blocks, n_blocks, gamma, out):
            bl = [blocks[b] for b in range(n_blocks)]
            self.chain_calls.append((offset, gamma))
            tok = first
            for j in range(gamma):
                tok = self.model([tok], [(1, offset + j, 1, bl)])[0]
                out[j] = tok
            return 0

        self._f, self._c = H.VERIFY_FN(_forward), H.CHAIN_FN(_chain)
        b = H.KhDraftBackend()
        b.model, b.kv, b.forward, b.chain, b.max_chunk = None, None, self._f, self._c, 8
        b.weights_bytes, b.kv_allocated_bytes, b.kv_block_bytes = 1000, num_blocks * 64, 64
        self.handle = H._P()
        H._check(H.lib().kh_draft_model_create(C.byref(b), num_blocks, BS, C.byref(self.handle)))
        d = H.KhDrafter()
        H.lib().kh_draft_model_vtable(self.handle, C.byref(d))
        self.drafter = H.Drafter(d, self)

    def live(self):
        return int(H.lib().kh_draft_model_live_sequences(self.handle))

    def pool(self):
        return H.BlockManager(0, 0, _borrowed=H.lib().kh_draft_model_block_manager(self.handle))


def test_draft_model_self_draft_accepts_everything_and_releases_its_pool():
    """DraftModel with the same (fake) weights as the target = the reference's self-draft probe: every proposal is
    accepted, the draft pool reconciles by truncation, catch-up runs in chunks, and release frees every block
    (draft.rs:286-411)."""
    eng, _ = make_engine()
    fb = FakeDraftBackend(128)
    eng.set_drafter(fb.drafter)
    ps = prompts(2, 13, 20, 30)
    arr = [eng.submit(p, 24) for p in ps]
    out = eng.run_to_completion(arr)
    assert [out[a][0] for a in arr] == [reference_generation(p, 24) for p in ps]
    st = eng.spec_stats()
    assert st["proposed_total"] > 0 and st["accepted_total"] == st["proposed_total"]
    assert any(n == 8 for n, _ in fb.forward_calls)              # catch-up chunks capped at max_chunk
    assert fb.live() == 0 and fb.pool().num_free == 128          # released at finish


def test_drafter_memory_report():
    """Drafter::memory through Engine::drafter_memory (drafter.rs:88-127, engine.rs:1128-1132; draft.rs:259-266): None
    without a drafter, zeros for a drafter with no footprint, and for a DraftModel its weights, its pool and the blocks
    its live sequences hold (live blocks x bytes per block)."""
    eng, _ = make_engine()
    assert eng.drafter_memory() is None
    eng.set_drafter(H.ScriptedDrafter(1.0, 1, VOCAB))
    assert eng.drafter_memory() == {"weights_bytes": 0, "kv_allocated_bytes": 0, "kv_used_bytes": 0}
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, lambda s, c, g: [], lambda s: None, memory=lambda: (7, 8, 9)))
    assert eng.drafter_memory() == {"weights_bytes": 7, "kv_allocated_bytes": 8, "kv_used_bytes": 9}
    fb = FakeDraftBackend(128)
    eng.set_drafter(fb.drafter)
    assert eng.drafter_memory() == {"weights_bytes": 1000, "kv_allocated_bytes": 128 * 64, "kv_used_bytes": 0}
    a = eng.submit(prompts(1, 13, 20, 21)[0], 24)
    used = 0
    for _ in range(6):
        eng.step()
        used = max(used, eng.drafter_memory()["kv_used_bytes"])
    assert used > 0 and used % 64 == 0
    eng.run_to_completion([a])
    assert eng.drafter_memory()["kv_used_bytes"] == 0
