"""Pipelined plain decode in the host engine (crates/kiln-engine/src/engine.rs:1428-1475 pipelined_turn / pipeline_ok,
1656-1744 build_pipelined, 1748-1766 apply_inflight), driven by the checksum mock behind the launch/collect seam.

  * the pipelined engine emits exactly what the synchronous engine emits, and step N + 1 is launched before step N is
    collected (the overlap the path exists for)
  * the reference's discarded-row invariant (crates/kiln-engine/tests/pipeline_discard.rs): a sequence that stops or is
    cancelled at a pipelined apply has one row in flight; its block never enters the prefix cache, and what the cache
    serves afterwards is bit-equal to a cold run
  * the pipeline yields to speculation, to waiting requests and to a full pool
"""
import ctypes as C

import pytest

from kiln_b200 import host as H
from tests.test_engine import BS, VOCAB, ChecksumModel, prompts, reference_generation


def make_engine(num_blocks=32, pipelined=True, **kw):
    model = ChecksumModel(num_blocks)
    # chunk == block, as in pipeline_discard.rs:156-170: matches trim to block-aligned canonical boundaries
    cfg = H.EngineConfig(block_size=BS, num_blocks=num_blocks, prefill_chunk=BS, prefill_fine_chunk=BS, prefix_cache=True,
                         deterministic_decode_width=32, gamma=4, spec_max_batch=4, spec_min_acceptance=0.0, max_key_len=0,
                         batch_verify=True)
    for k, v in kw.items():
        setattr(cfg, k, v)
    sm = H.StepModel.from_python(model, VOCAB, model.copy_block, pipelined=True)
    return H.Engine(cfg, sm, pipelined=pipelined), model, sm


def run(eng, prompt, max_tokens, stop=()):
    a = eng.submit(prompt, max_tokens, stop)
    toks, kind = eng.run_to_completion([a])[a]
    return a, toks, kind


def test_pipelined_equals_synchronous_and_overlaps():
    ps = prompts(5, 7)
    outs = []
    for pipelined in (True, False):
        eng, model, sm = make_engine(num_blocks=128, pipelined=pipelined)
        arr = [eng.submit(p, 9 + 3 * i) for i, p in enumerate(ps)]
        out = eng.run_to_completion(arr)
        outs.append([out[a] for a in arr])
        for i, (a, p) in enumerate(zip(arr, ps)):
            assert out[a] == (reference_generation(p, 9 + 3 * i), "length")
        assert (eng.pipelined_steps > 0) == pipelined
        if pipelined:
            log = sm.pipeline_log
            launches = {e[1]: i for i, e in enumerate(log) if e[0] == "launch"}
            collects = {e[1]: i for i, e in enumerate(log) if e[0] == "collect"}
            fed = [e for e in log if e[0] == "launch" and any(f >= 0 for f in e[2])]
            assert fed, "no step was built from unread tokens"
            for e in fed:   # a fed step is launched before the step it feeds from is read back
                assert launches[e[1]] < collects[e[1] - 1]
        assert eng.block_manager().num_free + eng.cache_stats()["resident_blocks"] == 128
    assert outs[0] == outs[1]


def test_requests_of_different_lengths_leave_the_pipeline_one_by_one():
    """A sequence whose final token is in flight gets no row in the next step (engine.rs:1670-1674); the feed indices
    of the others keep pointing at their own rows."""
    eng, model, sm = make_engine(num_blocks=128)
    ps = prompts(4, 3, lo=4, hi=9)
    lens = (30, 11, 16, 22)
    arr = [eng.submit(p, n) for p, n in zip(ps, lens)]
    out = eng.run_to_completion(arr)
    for a, p, n in zip(arr, ps, lens):
        assert out[a] == (reference_generation(p, n), "length")
    widths = [len(e[2]) for e in sm.pipeline_log if e[0] == "launch"]
    # prefills are admitted one per step, so the pipeline only starts once all four decode; then they leave one by one
    assert max(widths) == 4 and widths[-1] == 1
    tail = widths[widths.index(4):]
    assert sorted(tail, reverse=True) == tail and set(tail) == {4, 3, 2, 1}


def test_pipelined_stop_never_donates_the_inflight_block():
    # 1) A stops through a sampled stop token at a pipelined apply, with prompt + generated landing exactly on a block
    # boundary: the discarded row is the would-be last row of a full block.
    prompt_a = None
    for seed in range(200):
        cand = prompts(1, 100 + seed, lo=6, hi=7)[0]
        truth = reference_generation(cand, 12)
        if truth[5] not in truth[:5]:
            prompt_a, truth_a = cand, truth
            break
    assert prompt_a is not None and len(prompt_a) == 6
    stop = truth_a[5]                      # G = 6 => p + G = 12 = 3 full blocks
    warm, _, _ = make_engine()
    a, toks, kind = run(warm, prompt_a, 20, [stop])
    assert kind == "stop" and toks == truth_a[:5]
    assert warm.seq_state(a).generated == 6
    assert warm.pipelined_steps > 0, "the stop must land on the pipelined path"

    # 2) B extends A's full stream (stop token included). Settled rows = p + G - 1 = 11 -> exactly 2 donatable blocks;
    # the block holding rows 8..11 carried the discarded in-flight row and must not have been donated.
    prompt_b = prompt_a + truth_a[:6] + [(truth_a[6] + 1 + i) % VOCAB for i in range(4)]
    cold, _, _ = make_engine()
    b, cold_toks, _ = run(cold, prompt_b, 4)
    assert cold.seq_state(b).cached_tokens == 0
    assert cold_toks == reference_generation(prompt_b, 4)
    b, warm_toks, _ = run(warm, prompt_b, 4)
    assert warm.seq_state(b).cached_tokens == 8, "the match must cover exactly the settled full blocks"
    assert warm_toks == cold_toks, "a prefix-cache read after a pipelined stop served stale data"

    # 3) the same region again now hits what B donated from its own prefill
    b, again_toks, _ = run(warm, prompt_b, 4)
    assert again_toks == cold_toks and warm.seq_state(b).cached_tokens >= 8

    # 4) cancel variant: the flag is honoured at an apply with a row in flight
    prompt_c = prompts(1, 77, lo=6, hi=7)[0]
    truth_c = reference_generation(prompt_c, 40)
    warm2, _, _ = make_engine()
    c = warm2.submit(prompt_c, 30)
    got = []
    while len(got) < 3:
        warm2.step()
        got += warm2.take_output(c)[0]
    assert warm2.pipelined_steps > 0, "the cancel must interrupt a pipeline"
    warm2.cancel(c)
    out = warm2.run_to_completion([c])[c]
    assert out[1] == "cancelled"
    generated = warm2.seq_state(c).generated
    assert (got + out[0]) == truth_c[:len(got + out[0])] and generated >= len(got + out[0])
    settled = len(prompt_c) - 1 + generated
    prompt_d = prompt_c + truth_c[:generated] + [(truth_c[generated] + 1 + i) % VOCAB for i in range(4)]
    cold2, _, _ = make_engine()
    d, d_cold, _ = run(cold2, prompt_d, 4)
    d, d_warm, _ = run(warm2, prompt_d, 4)
    assert d_warm == d_cold, "a prefix-cache read after a pipelined cancel served stale data"
    matched = warm2.seq_state(d).cached_tokens
    assert matched > 0 and matched % BS == 0 and matched <= settled // BS * BS
    for eng in (warm, warm2):
        assert eng.block_manager().num_free + eng.cache_stats()["resident_blocks"] == 32


def test_pipeline_yields_to_speculation_waiting_requests_and_a_full_pool():
    # a drafter that can still propose keeps every step synchronous (engine.rs:1482-1500)
    eng, model, sm = make_engine(num_blocks=64)
    truth = {}
    state = {}
    drafter = H.Drafter.from_python(lambda s, p: state.__setitem__(s, 0),
                                    lambda s, committed, g: (state.__setitem__(s, state[s] + len(committed)) or truth[s][state[s]:state[s] + g]),
                                    lambda s: state.pop(s, None))
    eng.set_drafter(drafter)
    p = prompts(1, 5)[0]
    truth[0] = reference_generation(p, 16)
    a = eng.submit(p, 16)
    assert eng.run_to_completion([a])[a] == (truth[0], "length")
    assert eng.pipelined_steps == 0 and eng.spec_stats()["rounds_total"] > 0

    # a waiting request ends the pipeline at the next turn; both finish with the model's tokens
    eng, model, sm = make_engine(num_blocks=64)
    p1, p2 = prompts(2, 9)
    a1 = eng.submit(p1, 20)
    for _ in range(len(p1) // BS + 6):
        eng.step()
    before = eng.pipelined_steps
    assert before > 0
    a2 = eng.submit(p2, 5)
    out = eng.run_to_completion([a1, a2])
    assert out[a1] == (reference_generation(p1, 20), "length") and out[a2] == (reference_generation(p2, 5), "length")

    # a pool without a free block for the next append hands the step back to the synchronous path, which evicts
    eng, model, sm = make_engine(num_blocks=8)
    p = prompts(1, 11, lo=5, hi=6)[0]
    a, toks, kind = run(eng, p, 10)                       # fills the cache with donated blocks
    assert toks == reference_generation(p, 10)
    q = prompts(1, 12, lo=5, hi=6)[0]
    a, toks, kind = run(eng, q, 20)
    assert (toks, kind) == (reference_generation(q, 20), "length")


def test_pipelining_can_be_switched_off_and_on_mid_generation():
    eng, model, sm = make_engine(num_blocks=64)
    p = prompts(1, 21)[0]
    a = eng.submit(p, 40)
    got = []
    for phase, on in enumerate((True, False, True)):
        eng.set_pipelined(on)
        before = eng.pipelined_steps
        for _ in range(len(p) // BS + 9):
            eng.step()
            got += eng.take_output(a)[0]
        # one step may still have been in flight when the switch was flipped
        assert (eng.pipelined_steps - before > 1) == on
    out = eng.run_to_completion([a])[a]
    assert got + out[0] == reference_generation(p, 40)
    empty = H.KhDecodePipeline()
    assert H.lib().kh_engine_set_pipeline(eng._h, C.byref(empty)) != 0   # a table without its two calls is refused


def test_reference_grouping_keeps_wide_steps_synchronous():
    """With the reference's forward grouping (batch_verify = 0) a decode step wider than the deterministic width is
    several forwards; the pipeline only spans steps that are one forward."""
    ps = prompts(3, 31, lo=4, hi=9)
    for n_seqs, expect in ((2, True), (3, False)):
        eng, model, sm = make_engine(num_blocks=128, batch_verify=False, deterministic_decode_width=2)
        arr = [eng.submit(p, 14) for p in ps[:n_seqs]]
        out = eng.run_to_completion(arr)
        for a, p in zip(arr, ps):
            assert out[a] == (reference_generation(p, 14), "length")
        widths = [len(e[2]) for e in sm.pipeline_log if e[0] == "launch"]
        assert all(w <= 2 for w in widths)        # three sequences pipeline only once one of them has left
        if expect:
            assert max(widths) == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_pipelined_equals_synchronous(seed):
    """Staggered submissions, stop tokens, different lengths and a small pool (evictions): the pipelined engine and the
    synchronous one emit the same tokens with the same finish kinds; cancelled requests emit a prefix of the model's
    stream; every block comes back."""
    import numpy as np
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.integers(3, 7))
    ps = prompts(n, 200 + seed, lo=3, hi=30)
    script = []
    for i, p in enumerate(ps):
        gen = int(rng.integers(2, 28))
        truth = reference_generation(p, gen)
        stop = [truth[int(rng.integers(0, gen))]] if rng.random() < 0.4 else []
        script.append({"prompt": p, "gen": gen, "stop": stop, "at": int(rng.integers(0, 25)),
                       "cancel_at": int(rng.integers(5, 40)) if rng.random() < 0.25 else None, "truth": truth})
    results = []
    for pipelined in (True, False):
        eng, model, sm = make_engine(num_blocks=48, pipelined=pipelined)
        arr, outs, kinds = {}, {}, {}
        for step in range(400):
            for i, r in enumerate(script):
                if r["at"] == step:
                    arr[i] = eng.submit(r["prompt"], r["gen"], r["stop"])
                    outs[i], kinds[i] = [], None
                if r["cancel_at"] == step and i in arr and kinds[i] is None:
                    eng.cancel(arr[i])
            eng.step()
            for i, a in arr.items():
                if kinds[i] is None:
                    toks, kind = eng.take_output(a)
                    outs[i] += toks
                    kinds[i] = kind
            if len(arr) == len(script) and all(k is not None for k in kinds.values()):
                break
        assert all(k is not None for k in kinds.values()), "requests did not finish"
        for _ in range(3):
            eng.step()   # a dropped row may still be in flight
        assert eng.block_manager().num_free + eng.cache_stats()["resident_blocks"] == 48
        results.append((outs, kinds))
        assert (eng.pipelined_steps > 0) or not pipelined or n == 0
    for i, r in enumerate(script):
        for outs, kinds in results:
            assert outs[i] == r["truth"][:len(outs[i])]
        if r["cancel_at"] is None:
            assert results[0][0][i] == results[1][0][i] and results[0][1][i] == results[1][1][i]
            want = r["truth"]
            if r["stop"]:
                cut = want.index(r["stop"][0])
                assert results[0][0][i] == want[:cut] and results[0][1][i] == "stop"
            else:
                assert results[0][0][i] == want and results[0][1][i] == "length"
