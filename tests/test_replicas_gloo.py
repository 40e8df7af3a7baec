"""The N > 1 form of the verify path on CPU: two `gloo` ranks, each a full replica (own fake model, pool, engine,
rank-seeded requests), no data-path collective; only the measurements are reduced (sum of tokens, max of times, AND of
the speculation-on == off verdicts). Mirrors how the reference scales: one engine per worker process, requests sharded
at the gateway (crates/kiln-gateway; crates/kiln-worker/src/engine.rs)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from kiln_b200 import host as H
    from kiln_b200.replicas import combine_over_ranks, rank_seed, shard_requests
    from tests.test_engine import VOCAB, make_engine, prompts, reference_generation
    # a front end holding 7 requests gives this rank its contiguous share
    all_prompts = prompts(7, rank_seed(40, 0))
    mine = [all_prompts[i] for i in shard_requests(len(all_prompts), rank, world)]
    truth = [reference_generation(p, 20) for p in mine]
    eng, _ = make_engine()
    sd = H.ScriptedDrafter(0.7, rank_seed(9, rank), VOCAB)
    eng.set_drafter(sd)
    arr = []
    for p, t in zip(mine, truth):
        a = eng.submit(p, 20)
        sd.set_continuation(a, t)
        arr.append(a)
    out = eng.run_to_completion(arr)
    identical = [out[a][0] for a in arr] == truth
    if rank == 1:
        identical = identical and os.environ.get("KILN_TEST_FORCE_MISMATCH") != "1"
    tokens = sum(len(out[a][0]) for a in arr)
    tot = combine_over_ranks(dist, "cpu", 10.0 + rank, 20.0 - rank, tokens, identical, world)
    results[rank] = (len(mine), tokens, tot.device_ms, tot.wall_ms, tot.tokens, tot.all_identical)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_replicas_reduce_only_measurements():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
        r0, r1 = results[0], results[1]
    assert (r0[0], r1[0]) == (4, 3)                       # 7 requests: shares differ by at most one
    assert r0[1] == 4 * 20 and r1[1] == 3 * 20
    for r in (r0, r1):                                    # every rank sees the same job totals
        assert r[2] == 11.0 and r[3] == 20.0              # max over ranks of both clocks
        assert r[4] == 7 * 20                             # tokens: sum over ranks
        assert r[5] is True


def test_shards_cover_every_request_once():
    from kiln_b200.replicas import shard_requests
    for n in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            seen = [i for r in range(world) for i in shard_requests(n, r, world)]
            assert seen == list(range(n))
            sizes = [len(shard_requests(n, r, world)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_requests(4, 2, 2)


def test_single_process_passthrough():
    from kiln_b200.replicas import combine_over_ranks
    t = combine_over_ranks(None, "cpu", 1.5, 2.5, 10, True, 1)
    assert (t.device_ms, t.wall_ms, t.tokens, t.all_identical) == (1.5, 2.5, 10, True)
