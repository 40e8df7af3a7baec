"""The speculative scheduler step (libkiln_host.so) driven by fake models and scripted drafters — the reference's
own way of testing its engine without weights (crates/kiln-engine/tests/{deterministic_partition,pipeline_discard,
drafter}.rs; crates/kiln-models/tests/spec_decode.rs for the invariants):

  * speculation ON == speculation OFF, token for token, with oracle / adversarial / injected drafters
  * the checksum mock derails on any stale or misplaced KV row, so rollback, COW and prefix sharing are
    tested end to end without a model
  * block tables and free-list order after every round equal the Python restatement of block.rs
  * gamma ramp, key-length envelope, stand-down, drafter faults, stop tokens, submit validation
"""
import ctypes as C

import numpy as np
import pytest

from kiln_b200 import host as H
from oracle import bookkeeping as B

VOCAB, BS = 251, 4


class ChecksumModel:
    """Sampled token = checksum of the KV rows the sequence gathers (position-weighted), so a stale, missing or
    misplaced row changes every later token (the RecordingMock idea, deterministic_partition.rs:41-125)."""

    def __init__(self, num_blocks, block_size=BS):
        self.bs = block_size
        self.pool = np.zeros((num_blocks, block_size), dtype=np.int64)
        self.forwards, self.rows, self.copies = 0, [], []

    def copy_block(self, src, dst):
        self.pool[dst] = self.pool[src]
        self.copies.append((src, dst))

    def __call__(self, ids, seqs):
        self.forwards += 1
        self.rows.append(len(ids))
        out, at = [], 0
        for (ln, off, sr, blocks) in seqs:
            for t in range(ln):
                pos = off + t
                self.pool[blocks[pos // self.bs], pos % self.bs] = ids[at + t] + 1
            for t in range(ln - sr, ln):
                pos = off + t
                acc = 0
                for i in range(pos + 1):
                    acc = (acc * 131 + int(self.pool[blocks[i // self.bs], i % self.bs]) * (i + 1)) % 1000003
                out.append(acc % VOCAB)
            at += ln
        return out


def reference_generation(prompt, n):
    """What a correct engine must emit: the checksum model run token by token on a private contiguous cache."""
    ctx, out = list(prompt), []
    for _ in range(n):
        acc = 0
        for i, t in enumerate(ctx):
            acc = (acc * 131 + (t + 1) * (i + 1)) % 1000003
        tok = acc % VOCAB
        out.append(tok)
        ctx.append(tok)
    return out


def make_engine(num_blocks=256, **kw):
    model = ChecksumModel(num_blocks)
    cfg = H.EngineConfig(block_size=BS, num_blocks=num_blocks, prefill_chunk=16, prefill_fine_chunk=4, prefix_cache=False,
                         deterministic_decode_width=32, gamma=4, spec_max_batch=4, spec_min_acceptance=0.0, max_key_len=0,
                         batch_verify=True)
    for k, v in kw.items():
        setattr(cfg, k, v)
    sm = H.StepModel.from_python(model, VOCAB, model.copy_block)
    return H.Engine(cfg, sm), model


def prompts(n, seed=0, lo=5, hi=40):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, VOCAB, size=int(rng.integers(lo, hi))).tolist() for _ in range(n)]


def oracle_drafter(truth_by_seq):
    """Proposes the true continuation (spec_probe.rs's OracleDrafter)."""
    state = {}

    def begin(seq, prompt):
        state[seq] = 0

    def propose(seq, committed, gamma):
        state[seq] += len(committed)
        return truth_by_seq[seq][state[seq]: state[seq] + gamma]

    return H.Drafter.from_python(begin, propose, lambda seq: state.pop(seq, None)), state


def test_plain_decode_matches_the_model():
    eng, model = make_engine()
    ps = prompts(3, 1)
    arr = [eng.submit(p, 12) for p in ps]
    out = eng.run_to_completion(arr)
    for a, p in zip(arr, ps):
        assert out[a] == (reference_generation(p, 12), "length")
    assert eng.block_manager().num_free == 256


@pytest.mark.parametrize("batch_verify", [True, False])
def test_speculation_on_equals_off_with_three_drafters(batch_verify):
    ps = prompts(3, 2)
    truth = [reference_generation(p, 30) for p in ps]
    # oracle drafter: everything accepted
    eng, model = make_engine(batch_verify=batch_verify)
    d, _ = oracle_drafter({i: t for i, t in enumerate(truth)})
    eng.set_drafter(d)
    arr = [eng.submit(p, 30) for p in ps]
    out = eng.run_to_completion(arr)
    assert [out[a][0] for a in arr] == truth
    st = eng.spec_stats()
    assert st["accepted_total"] == st["proposed_total"] > 0 and st["rollback_rounds_total"] == 0
    # adversarial drafter (spec_decode.rs:147-198): valid but wrong ids; every round corrects and rolls back
    eng, model = make_engine(batch_verify=batch_verify)
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, lambda s, c, g: [11, 23, 5, 42][:g], lambda s: None))
    arr = [eng.submit(p, 30) for p in ps]
    out = eng.run_to_completion(arr)
    assert [out[a][0] for a in arr] == truth
    st = eng.spec_stats()
    assert st["rollback_rounds_total"] > 0 and st["rollback_tokens_total"] >= st["rollback_rounds_total"]
    assert eng.block_manager().num_free == 256
    # injected acceptance at p = 0.7 (the headline drafter)
    eng, model = make_engine(batch_verify=batch_verify)
    sd = H.ScriptedDrafter(0.7, 5, VOCAB)
    eng.set_drafter(sd)
    arr = [eng.submit(p, 30) for p in ps]
    for a, t in zip(arr, truth):
        sd.set_continuation(a, t)
    out = eng.run_to_completion(arr)
    assert [out[a][0] for a in arr] == truth
    st = eng.spec_stats()
    assert 0.4 < st["accepted_total"] / st["proposed_total"] < 0.95


def test_forward_grouping_reference_versus_batched():
    """Reference: one forward per verify segment (engine.rs:2240-2271); row-invariant backend: one per iteration."""
    ps = prompts(3, 3, 9, 10)
    truth = {i: reference_generation(p, 12) for i, p in enumerate(ps)}
    counts = {}
    for bv in (False, True):
        eng, model = make_engine(batch_verify=bv)
        d, _ = oracle_drafter(truth)
        eng.set_drafter(d)
        arr = [eng.submit(p, 12) for p in ps]
        eng.run_to_completion(arr)
        counts[bv] = (eng.forwards, eng.iterations, max(model.rows))
    assert counts[True][0] == counts[True][1]            # exactly one forward per iteration
    assert counts[False][0] > counts[False][1]           # several per iteration
    assert counts[True][2] > counts[False][2]            # and the batched forward is wider


def test_block_tables_and_free_list_match_the_python_restatement():
    """After every iteration the engine's table and the pool's free-list order equal a shadow built from
    oracle/bookkeeping.py — 'block tables and rollback state bit-exact' (block.rs:381-396, 167-169)."""
    p = prompts(1, 4, 9, 10)[0]
    truth = reference_generation(p, 40)
    eng, model = make_engine(num_blocks=64)
    sd = H.ScriptedDrafter(0.5, 9, VOCAB)
    eng.set_drafter(sd)
    a = eng.submit(p, 40)
    sd.set_continuation(a, truth)
    mgr, tab = B.BlockManager(64, BS), B.BlockTable()
    got, prev_stats, finished = [], eng.spec_stats(), None
    while finished is None:
        before = eng.seq_state(a)
        eng.step()
        toks, finished = eng.take_output(a)
        got += toks
        st = eng.spec_stats()
        after = eng.seq_state(a)
        if finished:
            break
        # replay the iteration on the shadow: the engine appended (kv growth + rolled-back slots), then truncated
        rounds = st["rounds_total"] - prev_stats["rounds_total"]
        proposed = st["proposed_total"] - prev_stats["proposed_total"]
        appended = (1 + proposed) if rounds else (after.num_tokens - before.num_tokens)
        tab.append_tokens(mgr, appended)
        tab.truncate(mgr, after.num_tokens)
        assert list(tab.blocks) == after.blocks and tab.num_tokens == after.num_tokens
        assert mgr.free == eng.block_manager().free_list()
        prev_stats = st
    assert got == truth


def test_gamma_ramp_and_envelope_clamps():
    """Per-round gamma = min(width ramp, det_width - 1, remaining - 1, max_key_len - (offset + 1)) (engine.rs:1515-1547)."""
    seen = []

    def propose(seq, committed, gamma):
        seen.append(gamma)
        return [1] * gamma

    # width ramp at spec_max_batch 4, gamma 4: widths 1..5 -> 4, 3, 2, 1, off
    for width, want in [(1, 4), (2, 3), (3, 2), (4, 1), (5, None)]:
        seen.clear()
        eng, _ = make_engine()
        eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: None))
        arr = [eng.submit([3], 50) for _ in range(width)]     # 1-token prompts are admitted together (no prefill)
        for _ in range(6 + width):
            eng.step()
        assert (max(seen) if seen else None) == want
    # deterministic width clamp
    seen.clear()
    eng, _ = make_engine(deterministic_decode_width=3)
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: None))
    eng.submit([3, 4, 5], 50)
    for _ in range(6):
        eng.step()
    assert max(seen) == 2
    # remaining budget clamp: never propose past max_tokens
    seen.clear()
    eng, _ = make_engine()
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: None))
    a = eng.submit([3, 4, 5], 4)
    out = eng.run_to_completion([a])
    assert len(out[a][0]) == 4 and all(g <= 3 for g in seen)
    # key-length envelope (VERIFY_MAX_KEY_LEN semantics, engine.rs:204-213): speculation stops, decoding continues
    seen.clear()
    eng, _ = make_engine(max_key_len=12)
    eng.set_drafter(H.Drafter.from_python(lambda s, p: None, propose, lambda s: None))
    p = prompts(1, 5, 6, 7)[0]
    a = eng.submit(p, 20)
    out = eng.run_to_completion([a])
    assert out[a][0] == reference_generation(p, 20)
    assert seen and min(seen) >= 1
    assert eng.seq_state(a).spec_proposed < 20
