#!/usr/bin/env python
"""Headline benchmark: verified tokens/s of the speculative-decoding verify step.

Workload (the metric's configuration): Llama-3.1-8B architecture, mlx affine 4-bit group 64, a continuous
batch of 32 sequences with prompt lengths uniform in [512, 2048] of uniform-random ids, k = 5 drafted
tokens per round that equal the target's greedy choice with probability 0.7 (seeded) and are uniform-random
ids otherwise, paged KV with 16-token bf16 blocks, 256 generated tokens each. Weights are random-init
N(0, 0.02) quantised by kiln_b200.synth (no checkpoint or dataset exists where this runs).

One "step" = one engine iteration in steady state: a single (k+1)-rows-per-sequence verify forward over the
paged cache + greedy rows + the acceptance walk + rollback. The host scheduler is the C++ engine of
libkiln_host.so driving kc_verify_step of libkiln_cuda.so through a C function table; Python only starts it.

  value  verified tokens/s from the device time of the timed steps (CUDA events on the launching stream,
         inputs resident in HBM)
  e2e    the same through the public call with HOST buffers: wall time of engine.step(), which holds the
         host scheduling, the host->device copy of the step's token ids / block tables and the device->host
         read of the sampled tokens and acceptance counts

Phases: (1) speculation OFF run to completion: gives the target's greedy continuation (needed to inject
acceptance) and donates every prompt to the radix prefix cache; (2) speculation ON with the scripted drafter:
every prompt is a full prefix-cache hit, so all sequences decode together from the first iteration; its
tokens are checked to be identical to phase 1 (speculation on == off). Timed steps come from phase 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (preset, batch, k, prompt_lo, prompt_hi, generated)
    "llama-3.1-8b-w4g64-verify-k5-bs32": ("llama-3.1-8b", 32, 5, 512, 2048, 256),
    # the reference's own CPU-runnable case: 1B target + its first 4 layers as the draft model (own weights, own pool),
    # batch 1, k = 4: speculation runs through the real draft lane (kc_draft_chain), not the scripted drafter
    "llama-3.2-1b-w4g64-verify-k4-bs1": ("llama-3.2-1b", 1, 4, 128, 128, 64, {"draft_layers": 4}),
    # parity-sized cases (speculation on == off at full size), not headline numbers: 64 requests that share a
    # 1024-token prefix (radix cache + copy-on-write) with 256-token unique suffixes; Gemma-2 with 6144-token prompts
    # (sliding window 4096 on even layers, attention and final-logit softcaps)
    "qwen2.5-7b-w8g32-sharedprefix-k4-bs64": ("qwen2.5-7b", 64, 4, 1280, 1280, 128, {"shared_prefix": 1024}),
    "gemma-2-9b-w4g128-verify-k3-bs16": ("gemma-2-9b", 16, 3, 6144, 6144, 128),
    # the tensor-parallel configuration: under torchrun every rank holds a slice of every layer and all ranks run the
    # SAME requests (strong scaling); on one GPU it runs unsharded
    "llama-3-70b-w4g64-verify-k4-bs64-tp": ("llama-3-70b", 64, 4, 1024, 4096, 256, {"tp": True}),
    "llama-3.1-8b-w4g64-verify-k5-bs32-tp": ("llama-3.1-8b", 32, 5, 512, 2048, 256, {"tp": True}),
    # the 70B configuration's batch, k and prompt lengths (320 rows per step: two row chunks per GEMM) on the 8B model
    "llama-3.1-8b-w4g64-verify-k4-bs64-tp": ("llama-3.1-8b", 64, 4, 1024, 4096, 256, {"tp": True}),
    "llama-3-70b-8l-w4g64-verify-k4-bs64-tp": ("llama-3-70b-8l", 64, 4, 1024, 4096, 256, {"tp": True}),
    "tiny-llama-verify-k4-bs4": ("tiny-llama", 4, 4, 40, 90, 48),
}
METRIC = "verified tok/s/GPU, Llama-3-8B w4g64 k=5 bs32; p50 verify-step ms"


def peaks():
    """Measured peaks of this pool's B200s (MEASURED_PEAKS.json), else the stated fallback."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks, power and clock-event reasons WHILE the timed region runs (reads only, nothing is set):
    NVML from a polling thread; nvidia-smi in a loop when the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}

    def __init__(self, device: int):
        self.device, self.proc, self.lines, self.samples, self.stop_flag, self.nvml = device, None, [], [], False, None
        self.recording = True

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.device < len(ids) and ids[self.device].isdigit():
                return int(ids[self.device])
        return self.device

    def start(self, record: bool = True):
        """record = False: open NVML and start polling without keeping samples (the first queries after nvmlInit can
        take hundreds of milliseconds); arm() then starts the record at the head of the timed region."""
        self.recording = record
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self._physical_index())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n, i, power = self.nvml, 0, 0.0
        while not self.stop_flag:
            try:
                if i % 8 == 0:   # the power query is the slow one
                    power = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                sample = (n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM),
                          n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle), power)
                if self.recording:
                    self.samples.append(sample)
            except Exception:
                pass
            i += 1
            time.sleep(0.002)

    def arm(self):
        self.samples, self.lines = [], []
        self.recording = True

    def _read(self):
        for line in self.proc.stdout:
            if self.recording:
                self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.nvml:
            self.stop_flag = True
            self.thread.join(timeout=2)
            sm = sorted(s[0] for s in self.samples)
            mask = 0
            for s_ in self.samples:
                mask |= int(s_[1])
            reasons = sorted(k for k, bit in self.REASONS.items() if mask & bit)
            return {"sm_mhz": float(sm[len(sm) // 2]) if sm else None, "sm_max_mhz": float(self.max_sm), "reasons": reasons,
                    "samples": len(sm), "power_w_max": max((s_[2] for s_ in self.samples), default=None), "source": "nvml polling thread"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi, 50 ms period"}


def algorithmic(cfg, batch, k, mean_ctx):
    """Algorithmic bytes and flops of one verify step: quantised weights read once (incl. the head), KV read once
    per sequence, KV written, logits written + read; flops = 2*M*params + 4*M*ctx*Hq*D*L."""
    H, L, Hq, Hkv, D, F, V = (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads,
                              cfg.head_dim, cfg.intermediate_size, cfg.vocab_size)

    def qb(o, i):
        return o * i * cfg.bits / 8 + 2 * o * (i // cfg.group_size) * 2
    per_layer = qb(Hq * D, H) + 2 * qb(Hkv * D, H) + qb(H, Hq * D) + 2 * qb(F, H) + qb(H, F)
    params_layer = Hq * D * H + 2 * Hkv * D * H + H * Hq * D + 3 * F * H
    M = batch * (k + 1)
    w = L * per_layer + qb(V, H)
    kv_tok = L * 2 * Hkv * D * 2
    total = w + batch * mean_ctx * kv_tok + M * kv_tok + M * V * 2 * 2
    gemm_flops = 2 * M * (L * params_layer + V * H)
    attn_flops = 4 * M * mean_ctx * Hq * D * L
    return {"bytes": total, "weight_bytes": w, "kv_read_bytes": batch * mean_ctx * kv_tok, "gemm_flops": gemm_flops,
            "attn_flops": attn_flops, "M": M}


# DRAM traffic of the dominant kernel (the quantised GEMM) relative to its algorithmic weight bytes, from one ncu
# capture of a single launch larger than L2 (out 128256 x in 4096, 192 rows; summary committed under profiles/):
# dram__bytes_read.sum + dram__bytes_write.sum = 299.9 MB + 33.6 MB for 295.5 MB of weight records. The traffic of a
# launch grows in proportion to its weight bytes, so the per-launch figure reported is this ratio times the mean
# algorithmic weight bytes per GEMM launch of the step.
GEMM_DRAM_TRAFFIC_PER_WEIGHT_BYTE = (299.9 + 33.6) / 295.5

# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------

class Workload:
    """Model + pools + engine for one rank."""

    def __init__(self, name: str, rank: int, local_rank: int, keep_cpu_sample: bool, world: int = 1, dist=None):
        import numpy as np
        import torch
        from kiln_b200 import api, host
        from kiln_b200.replicas import rank_seed
        from kiln_b200.synth import PRESETS, synth_checkpoint
        preset, self.batch, self.k, lo, hi, self.gen = WORKLOADS[name][:6]
        extras = WORKLOADS[name][6] if len(WORKLOADS[name]) > 6 else {}
        self.name, self.cfg = name, PRESETS[preset]
        cfg = self.cfg
        torch.cuda.set_device(local_rank)
        self.ctx = api.Context(local_rank)
        self.tp = world if (extras.get("tp") and world > 1) else 1
        if self.tp > 1:   # rank 0 creates the NCCL id; the bytes travel through the benchmark's own process group
            ident = torch.zeros(128, dtype=torch.uint8, device=f"cuda:{local_rank}")
            if rank == 0:
                ident.copy_(torch.frombuffer(bytearray(api.Context.tp_unique_id()), dtype=torch.uint8))
            dist.broadcast(ident, src=0)
            self.ctx.tp_init(bytes(ident.cpu().numpy().tobytes()), rank, world)
        t0 = time.time()
        ck = synth_checkpoint(cfg, seed=0, device=f"cuda:{local_rank}")
        self.prefill_chunk = 2048 if cfg.hidden_size >= 2048 else 256
        max_step = self.prefill_chunk + self.batch * (self.k + 1)
        self.model = api.CudaModel(self.ctx, cfg, ck, max_step_tokens=max_step, max_step_seqs=self.batch + 1,
                                   tp_rank=rank if self.tp > 1 else 0, tp_world=self.tp)
        self.tp_exchange = "none"
        if self.tp > 1:
            self.tp_exchange = os.environ.get("KILN_TP_EXCHANGE", "peer")
            if self.tp_exchange == "peer":   # the ranks' outputs are read in place over NVLink instead of all-gathered
                def everyone(b):
                    out = [None] * world
                    dist.all_gather_object(out, b)
                    return out
                self.model.tp_connect(everyone)
        self.cpu_sample = None
        if keep_cpu_sample:   # the checkpoint on the host, for the CPU baseline (packed: about an eighth of bf16)
            self.cpu_sample = {n: t.cpu() for n, t in ck.items()}
        del ck
        torch.cuda.empty_cache()
        self.build_s = time.time() - t0
        rng = np.random.default_rng(rank_seed(1000, 0 if self.tp > 1 else rank))   # tensor-parallel ranks serve the same requests
        lens = rng.integers(lo, hi + 1, size=self.batch)
        self.prompts = [rng.integers(0, cfg.vocab_size, size=int(n), dtype=np.int64).tolist() for n in lens]
        if extras.get("shared_prefix"):
            common = rng.integers(0, cfg.vocab_size, size=int(extras["shared_prefix"]), dtype=np.int64).tolist()
            self.prompts = [common + p[len(common):] for p in self.prompts]
        bs = 16
        per_seq = [-(-(len(p) + self.gen + self.k + 1) // bs) for p in self.prompts]
        self.num_blocks = sum(per_seq) + self.batch * ((self.gen + self.k + 1) // bs + 3) + 64
        self.kv = api.PagedKv(self.ctx, self.model.kv_spec(self.num_blocks, bs, tp_world=self.tp))
        ec = host.EngineConfig(block_size=bs, num_blocks=self.num_blocks, max_batch_tokens=max_step,
                               prefill_chunk=self.prefill_chunk, prefill_fine_chunk=128, prefix_cache=True,
                               deterministic_decode_width=max(32, self.batch), gamma=self.k,
                               spec_max_batch=1 << 20,   # keeps the width ramp (drafter.rs:62-70) at gamma = k for the whole batch
                               spec_min_acceptance=0.0, max_key_len=0, batch_verify=True)
        self.engine = host.Engine(ec, host.StepModel.from_cuda(self.model, self.kv))
        self.host = host
        self.mean_prompt = float(sum(len(p) for p in self.prompts)) / self.batch

    def close(self):
        """Releases the device objects in dependency order (before the process group and the interpreter go away)."""
        self.ctx.sync()
        self.engine = None
        self.model.close()
        self.kv.close()
        self.ctx.close()

    def run_off(self):
        """Phase 1: speculation off, to completion. Returns the greedy continuation of every prompt."""
        arrivals = [self.engine.submit(p, self.gen) for p in self.prompts]
        out = self.engine.run_to_completion(arrivals)
        return [out[a][0] for a in arrivals]

    def plain_decode_pass(self, steps: int = 40):
        """Plain decode at the full batch — the path every request takes when speculation stands down
        (engine.rs:1428-1475). Runs after run_off, so every prompt is a prefix-cache hit and the batch is full from the
        first iteration; `steps` full-batch decode steps pipelined (step N + 1 launched from step N's unread tokens),
        then as many synchronous, each timed from the end of one engine step to the end of the next (host work
        included); the requests are cancelled afterwards."""
        eng = self.engine
        arrivals = [eng.submit(p, self.gen) for p in self.prompts]
        spans = {True: [], False: []}
        for pipelined in (True, False):
            eng.set_pipelined(pipelined)
            last_end, guard = None, 0
            while len(spans[pipelined]) < steps and guard < 20 * steps:
                guard += 1
                eng.step()
                now = time.perf_counter()
                emitted = sum(len(eng.take_output(a)[0]) for a in arrivals)
                if last_end is not None and emitted == len(arrivals):
                    spans[pipelined].append((now - last_end) * 1e3)
                last_end = time.perf_counter()
        eng.set_pipelined(True)
        for a in arrivals:
            eng.cancel(a)
        eng.run_to_completion(arrivals)
        med = lambda v: float(statistics.median(v[2:])) if len(v) > 4 else None
        p_ms, s_ms = med(spans[True]), med(spans[False])
        return {"pipelined_ms_per_step": p_ms, "synchronous_ms_per_step": s_ms,
                "steps_timed": [max(0, len(spans[True]) - 2), max(0, len(spans[False]) - 2)],
                "pipelined_tok_s": len(arrivals) / (p_ms * 1e-3) if p_ms else None,
                "synchronous_tok_s": len(arrivals) / (s_ms * 1e-3) if s_ms else None,
                "rows_per_step": len(arrivals)}

    def prefill_pass(self, n_prompts: int = 3, length: int = 4097):
        """Chunked prefill through the same kernels (engine.rs:2114-2162, canonical_prefill_len :167-179): fresh
        prompts of `length` tokens (no prefix-cache hit), one at a time, one generated token each. With the
        reference's schedule a 4097-token prompt is two 2048-token chunks (each a forward whose GEMMs run in equal
        row chunks of 256). Time = wall clock of the engine steps until the request finishes."""
        import numpy as np
        eng = self.engine
        rng = np.random.default_rng(4242)
        ms, fwd0 = [], eng.forwards
        for _ in range(n_prompts):
            prompt = rng.integers(0, self.cfg.vocab_size, size=length, dtype=np.int64).tolist()
            a = eng.submit(prompt, 1)
            t0 = time.perf_counter()
            eng.run_to_completion([a])
            self.ctx.sync()
            ms.append((time.perf_counter() - t0) * 1e3)
        med = float(statistics.median(ms))
        c = self.cfg
        per_layer = (c.num_attention_heads * c.head_dim + 2 * c.num_key_value_heads * c.head_dim) * c.hidden_size + \
            c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.intermediate_size * c.hidden_size
        flops = 2.0 * c.num_hidden_layers * per_layer * (length - 1) + \
            4.0 * c.num_hidden_layers * c.num_attention_heads * c.head_dim * (length - 1) * (length / 2.0)
        return {"prompt_tokens": length, "prompts": n_prompts, "ms_per_prompt": med, "tok_s": (length - 1) / (med * 1e-3),
                "forwards_per_prompt": (eng.forwards - fwd0) / n_prompts, "tflops": flops / (med * 1e-3) / 1e12,
                "chunk": self.prefill_chunk}

    def submit_on(self, base, p_accept=0.7, seed=0):
        """Phase 2 submission: scripted drafter with injected acceptance; every prompt is a prefix-cache hit."""
        if not hasattr(self, "drafter"):
            self.drafter = self.host.ScriptedDrafter(p_accept, seed, self.cfg.vocab_size)
            self.engine.set_drafter(self.drafter)
        arrivals = []
        for p, cont in zip(self.prompts, base):
            a = self.engine.submit(p, self.gen)
            self.drafter.set_continuation(a, cont)
            arrivals.append(a)
        return arrivals


def timed_steps(w: Workload, base, n_steps: int, warmup: int, barrier=None, sampler=None):
    """Runs warmup + n_steps full-batch verify iterations; returns per-step records and the ON==OFF verdict."""
    import torch
    eng = w.engine
    records, checked, identical = [], 0, True
    if sampler:
        sampler.start(record=False)   # polling warms up during the warm-up steps; the record starts with the timed region
    arrivals, outs = [], {}
    done_warm = 0
    started = False
    guard = 0
    while len(records) < n_steps:
        guard += 1
        if guard > 100000:
            raise RuntimeError("benchmark loop did not converge")
        if eng.num_running == 0 and eng.num_waiting == 0:
            for a in arrivals:   # drain and check the finished round of requests
                toks, _ = eng.take_output(a)
                outs[a] = outs.get(a, []) + toks
            for a, cont in zip(arrivals, base):
                checked += 1
                identical &= outs.get(a, []) == cont
            arrivals = w.submit_on(base)
            outs = {}
        full = False
        running_before = eng.num_running
        s0 = eng.spec_stats()
        if done_warm >= warmup and not started:
            if barrier:
                barrier()
            if sampler:
                sampler.arm()
            torch.cuda.profiler.start()   # lets `ncu --profile-from-start off` list the timed region's launches only
            started = True
        t0 = time.perf_counter()
        eng.step()
        t1 = time.perf_counter()
        dev_ms = w.ctx.last_step_ms()
        s1 = eng.spec_stats()
        rounds = s1["rounds_total"] - s0["rounds_total"]
        full = rounds == w.batch and running_before in (0, w.batch)
        if not full:
            continue
        committed = (s1["accepted_total"] - s0["accepted_total"]) + rounds
        if done_warm < warmup:
            done_warm += 1
            continue
        records.append({"wall_ms": (t1 - t0) * 1e3, "dev_ms": dev_ms, "tokens": committed,
                        "proposed": s1["proposed_total"] - s0["proposed_total"],
                        "accepted": s1["accepted_total"] - s0["accepted_total"]})
    torch.cuda.profiler.stop()
    return records, (checked, identical), arrivals, outs


def roofline_pass(w: Workload, base, steps: int = 4):
    """A separate short pass with per-class CUDA events around every launch (events would perturb the headline timing)."""
    eng = w.engine
    got, cls_ms, cls_n = 0, {}, {}
    w.ctx.profile_read()
    guard = 0
    while got < steps and guard < 2000:
        guard += 1
        if eng.num_running == 0 and eng.num_waiting == 0:
            w.submit_on(base)
        s0 = eng.spec_stats()
        before = eng.num_running
        w.ctx.profile_enable(True)
        eng.step()
        prof = w.ctx.profile_read()
        w.ctx.profile_enable(False)
        s1 = eng.spec_stats()
        if s1["rounds_total"] - s0["rounds_total"] != w.batch or before not in (0, w.batch):
            continue
        got += 1
        for k, (ms, n) in prof.items():
            cls_ms[k] = cls_ms.get(k, 0.0) + ms
            cls_n[k] = cls_n.get(k, 0) + n
    return {k: (cls_ms[k] / max(got, 1), cls_n[k] / max(got, 1)) for k in cls_ms}, got


# --------------------------------------------------------------------------------------
# CPU arm: the oracle (a restatement of the reference's op graph; the reference's own MLX CPU path cannot
# be built or installed where this runs) timed on the host cores over a bounded sample of the same workload
# --------------------------------------------------------------------------------------

def cpu_reference(name: str, tensors, ctxs, steps: int, warmup: int, budget_s: float = 150.0):
    """Times the reference's own shape of the verify step on the host cores: ONE forward per speculating sequence
    (crates/kiln-engine/src/engine.rs:2164-2172, 2240-2271 — the reference never batches verify across sequences),
    i.e. (k + 1) rows of one sequence at its context through every layer, the head and the greedy rows. One timed step
    = one such forward; sequences of the batch are taken in turn. Nothing is extrapolated: a batch round on the CPU is
    `batch` of these forwards one after the other, each using every core. tensors: the whole checkpoint on the host."""
    import numpy as np
    import torch
    from kiln_b200 import api
    from kiln_b200.synth import PRESETS, synth_checkpoint
    from oracle import oracle as O
    preset, batch, k, lo, hi, gen = WORKLOADS[name][:6]
    cfg = PRESETS[preset]
    cores = os.cpu_count() or 1
    threads = O.set_threads(cores)   # launchers export OMP_NUM_THREADS=1 to their ranks: set it explicitly
    if tensors is None:
        dev = "cuda" if torch.cuda.is_available() else "cpu"   # the generator is the same on either device
        tensors = {n: t.cpu() for n, t in synth_checkpoint(cfg, seed=0, device=dev).items()}
        if dev == "cuda":
            torch.cuda.empty_cache()
    om = O.OracleModel(cfg, tensors)
    bs = 16
    if ctxs is None:
        rng = np.random.default_rng(1000)
        ctxs = [int(x) + gen // 2 for x in rng.integers(lo, hi + 1, size=batch)]
    nblk = -(-(max(ctxs) + k + 1) // bs)
    okv = O.OracleKv(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, nblk + 1, bs)
    rng = np.random.default_rng(7)
    times = []
    t_begin = time.perf_counter()
    for i in range(warmup + steps):
        c = ctxs[i % len(ctxs)]
        ids = rng.integers(0, cfg.vocab_size, size=k + 1).tolist()
        step = api.StepBatch(ids, [api.SeqStep(k + 1, c, k + 1, list(range(nblk)))])
        t0 = time.perf_counter()
        logits = om.forward_step(step, okv, want_logits=True)
        O.greedy_rows(logits, True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_begin > budget_s and len(times) >= 1:
            break
    fwd_s = sorted(times)[len(times) // 2]
    return {"forward_s": fwd_s, "mean_forward_s": sum(times) / len(times), "cores": cores, "threads": threads, "timed": len(times),
            "sample": (f"one sequence's verify forward per step ({k + 1} rows at that sequence's context, all {cfg.num_hidden_layers} "
                       f"layers + head + greedy rows): the reference verifies one forward per sequence; {len(times)} forwards timed, "
                       f"median; a batch round = {batch} such forwards, nothing extrapolated")}


GEMM_KERNEL = "qlinear_umma_ta_kernel (affine-dequant GEMM, tcgen05, A operand in TMEM)"
TP_WORKLOAD = "llama-3-70b-8l-w4g64-verify-k4-bs64-tp"


def pin_rank_to_cores(local_rank: int, world: int) -> None:
    """Gives every rank of a multi-GPU run its own contiguous share of the cores this process may use, so that the
    ranks' launch threads do not share cores (each rank issues a few hundred launches per step from one thread)."""
    try:
        cores = sorted(os.sched_getaffinity(0))
        per = len(cores) // world
        if per >= 2:
            os.sched_setaffinity(0, set(cores[local_rank * per:(local_rank + 1) * per]))
    except (AttributeError, OSError):
        pass


def status_word(ctx) -> int:
    """The context's device status word (0 = no bounded wait gave up); never raises."""
    try:
        return int(ctx.device_status())
    except Exception as e:   # the call reports a non-zero word as an error; the word is in its message
        import re
        m = re.search(r"0x([0-9a-fA-F]+)", str(e))
        return int(m.group(1), 16) if m else -1


def check_pass(w: "Workload", base) -> dict:
    """Speculation on, to completion, twice: equal to the speculation-off continuation `base`, and equal to itself."""
    t0 = time.time()
    arrivals = w.submit_on(base)
    fin = w.engine.run_to_completion(arrivals)
    on_s = time.time() - t0
    same = [fin[a][0] == cont for a, cont in zip(arrivals, base)]
    first_bad = [(i, next((j for j, (x, y) in enumerate(zip(fin[a][0], cont)) if x != y), min(len(fin[a][0]), len(cont))),
                  len(fin[a][0]), len(cont), fin[a][1])
                 for i, (a, cont) in enumerate(zip(arrivals, base)) if fin[a][0] != cont][:4]
    arrivals2 = w.submit_on(base)
    fin2 = w.engine.run_to_completion(arrivals2)
    on_twice_equal = all(fin2[b][0] == fin[a][0] for a, b in zip(arrivals, arrivals2))
    st = w.engine.spec_stats()
    return {"spec_on_equals_off": {"sequences_checked": len(same), "identical": all(same), "mismatching": len(same) - sum(same),
                                   "first_mismatches(seq, position, len_on, len_off, finish)": first_bad},
            "speculation_on_twice_equal": on_twice_equal, "launches": w.ctx.launch_count(), "iterations": w.engine.iterations,
            "speculation_on_s": round(on_s, 2), "proposed": st["proposed_total"], "accepted": st["accepted_total"],
            "rollback_rounds": st["rollback_rounds_total"], "cache": w.engine.cache_stats(), "device_status": status_word(w.ctx)}


def tp_record(rank: int, local_rank: int, world: int, dist, barrier) -> dict:
    """The tensor-parallel configuration on all `world` GPUs: the 70B layer shapes (8 of the 80 layers, so that it loads
    in seconds), batch 64, k = 4, prompts 1024-4096. Every rank holds a slice of every layer and all ranks serve the same
    requests. Reports the parity properties (speculation on == off, two speculation-on passes equal, device status) and
    the step time (max over ranks) with its per-class split and the bytes each rank receives from its peers per step."""
    import torch
    from kiln_b200.replicas import combine_over_ranks
    t0 = time.time()
    w = Workload(TP_WORKLOAD, rank, local_rank, keep_cpu_sample=False, world=world, dist=dist)
    base = w.run_off()
    chk = check_pass(w, base)
    records, _, arrivals, _ = timed_steps(w, base, 8, 3, barrier, None)
    dev_ms = sum(r["dev_ms"] for r in records)
    wall_ms = sum(r["wall_ms"] for r in records)
    tokens = sum(r["tokens"] for r in records) if rank == 0 else 0
    prof, _ = roofline_pass(w, base, 2)
    if arrivals:
        w.engine.run_to_completion(arrivals)
    ok = chk["spec_on_equals_off"]["identical"] and chk["speculation_on_twice_equal"] and chk["device_status"] == 0
    tot = combine_over_ranks(dist, f"cuda:{local_rank}", dev_ms, wall_ms, tokens, ok, world)
    st = torch.tensor([float(chk["device_status"])], dtype=torch.float64, device=f"cuda:{local_rank}")
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    cfg = w.cfg
    rows = w.batch * (w.k + 1)
    rec = {"workload": TP_WORKLOAD, "ranks": world, "ms_per_step": tot.device_ms / len(records),
           "verified_tok_s": tot.tokens / (tot.device_ms * 1e-3), "e2e_tok_s": tot.tokens / (tot.wall_ms * 1e-3),
           "kernel_classes_ms_per_step_rank0": {k2: round(v[0], 4) for k2, v in prof.items()},
           "spec_on_equals_off": chk["spec_on_equals_off"]["identical"], "sequences_checked": chk["spec_on_equals_off"]["sequences_checked"],
           "speculation_on_twice_equal": chk["speculation_on_twice_equal"], "all_ranks_ok": tot.all_identical,
           "device_status_max_over_ranks": int(st[0]),
           "exchange": (("peer memory, two phases: every rank sums its column slice of all ranks' bf16 [rows, hidden] sublayer outputs "
                         "(peer loads over NVLink, rank order, fp32, one rounding), the consumer kernel gathers the summed slices"
                         if world >= 4 and os.environ.get("KILN_TP_TWO_PHASE", "1") != "0" else
                         "peer memory: every rank's bf16 [rows, hidden] sublayer output after o_proj and down_proj is read in place over "
                         "NVLink by the consumer kernel (flag per rank and exchange, plain peer loads) and summed in rank order in fp32")
                        if w.tp_exchange == "peer" else
                        "all-gather of every rank's bf16 [rows, hidden] sublayer output after o_proj and down_proj (NCCL), summed "
                        "in rank order in fp32 by the consumer kernel"),
           "peer_bytes_received_per_rank_per_step": int(2 * cfg.num_hidden_layers * (world - 1) * rows * cfg.hidden_size * 2 *
                                                        (2.0 / world if (w.tp_exchange == "peer" and world >= 4 and os.environ.get("KILN_TP_TWO_PHASE", "1") != "0") else 1.0)),
           "seconds": round(time.time() - t0, 1)}
    w.close()
    return rec


def stream_gemv_records(ctx, pk):
    """The weight-streaming lane by itself on the decode shapes (at most 8 activation rows): time per call (the lane's
    kernel plus the reduction of its partials) from CUDA events on the library's stream around a run of back-to-back
    calls, against the weight bytes (mlx layout: packed words + bf16 scales
    and biases) at the measured copy bandwidth. Three copies of each weight are used in turn, so no launch finds its
    weight in L2 (3 x 66 MB > 126 MB); the tensor-core lane is timed beside it on the same inputs."""
    import torch
    from kiln_b200 import api
    out = []
    for label, n, k in (("llama-3.1-8b gate_up 28672x4096 w4g64", 28672, 4096), ("llama-3.1-8b down 4096x14336 w4g64", 4096, 14336),
                        ("llama-3.2-1b gate_up 16384x2048 w4g64", 16384, 2048)):
        g = torch.Generator(device="cuda").manual_seed(n + k)
        copies = max(3, -(-3 * 66_000_000 // (n * k // 2)))
        ws = []
        for _ in range(copies):
            w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device="cuda", generator=g)
            sc = (torch.rand(n, k // 64, device="cuda", generator=g) * 0.01 + 0.001).to(torch.bfloat16)
            bi = (torch.rand(n, k // 64, device="cuda", generator=g) * -0.08).to(torch.bfloat16)
            ws.append(api.QuantizedWeight(ctx, w, sc, bi, 4, 64))
        nbytes = n * k // 2 + 2 * n * (k // 64) * 2
        for rows in (1, 8):
            x = torch.randn(16, k, device="cuda", generator=g).to(torch.bfloat16)
            y = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
            torch.cuda.synchronize()
            rec = {"weight": label, "rows": rows, "weight_bytes": nbytes}
            lib_stream = torch.cuda.ExternalStream(ctx.stream)   # the events must sit on the stream the kernels run on
            for lane, fn in (("stream", "kc_quantized_matmul_stream"), ("tensor", "kc_quantized_matmul")):
                call = getattr(api.L.lib(), fn)
                for i in range(2 * copies):   # warm-up: every copy twice
                    api.check(call(ctx._h, ws[i % copies]._h, x.data_ptr(), rows, y.data_ptr()))
                reps = 8 * copies
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(lib_stream)
                for i in range(reps):
                    api.check(call(ctx._h, ws[i % copies]._h, x.data_ptr(), rows, y.data_ptr()))
                e1.record(lib_stream)
                ctx.sync()
                us = e0.elapsed_time(e1) * 1e3 / reps
                rec[lane] = {"us": round(us, 2), "GB/s": round(nbytes / us * 1e-3, 1), "frac_of_hbm": round(nbytes / us * 1e-3 / pk["hbm_gbs"], 3)}
            out.append(rec)
        for q in ws:
            q.close()
    return out


def injected_acceptance_run(eng, draft, prompt, gen, continuation, vocab, ctx, n_requests, p_accept=0.7):
    """What the real draft lane costs at a realistic acceptance rate. A truncation of a random-weight model never agrees
    with it, so the run above commits one token per round. Here every propose still runs the real draft model (its
    catch-up forward and its chain of k one-row forwards: the full device cost), but the tokens handed to the engine
    come from the scripted drafter (the target's greedy token with probability p, else a random id). The draft model's
    own proposals are therefore never the accepted ones, so each round it also recomputes the K/V of every committed
    token in its catch-up forward — a trained draft would only catch up on the one correction token: the figure is on
    the conservative side."""
    import ctypes as C
    from kiln_b200 import host
    scripted = host.ScriptedDrafter(p_accept, 0, vocab)
    dc, sc = draft.c, scripted.c

    def begin(seq, toks):
        arr = (C.c_uint32 * max(1, len(toks)))(*toks)
        for d in (dc, sc):
            if d.begin(d.user, seq, arr, len(toks)) != 0:
                raise RuntimeError("draft begin failed")

    def propose(seq, committed, gamma):
        arr = (C.c_uint32 * max(1, len(committed)))(*committed)
        out_real, out = (C.c_uint32 * max(1, gamma))(), (C.c_uint32 * max(1, gamma))()
        n_real, n = C.c_int32(0), C.c_int32(0)
        if dc.propose(dc.user, seq, arr, len(committed), gamma, out_real, C.byref(n_real)) != 0:
            raise RuntimeError("draft propose failed")
        if sc.propose(sc.user, seq, arr, len(committed), gamma, out, C.byref(n)) != 0:
            raise RuntimeError("scripted propose failed")
        return [int(out[i]) for i in range(n.value)]

    def release(seq):
        dc.release(dc.user, seq)
        sc.release(sc.user, seq)

    eng.set_drafter(host.Drafter.from_python(begin, propose, release))
    recs, outs = [], []
    for r in range(n_requests + 1):          # the first request warms the new drafter up
        a = eng.submit(prompt, gen)
        scripted.set_continuation(a, continuation)
        toks, fk, first = [], None, True
        while fk is None:
            s0 = eng.spec_stats()
            t0 = time.perf_counter()
            eng.step()
            t1 = time.perf_counter()
            s1 = eng.spec_stats()
            new, fk = eng.take_output(a)
            toks += new
            if r > 0 and not first and new:
                recs.append({"wall_ms": (t1 - t0) * 1e3, "tokens": len(new), "proposed": s1["proposed_total"] - s0["proposed_total"],
                             "accepted": s1["accepted_total"] - s0["accepted_total"]})
            first = False
        outs.append(toks)
    wall, tokens = sum(x["wall_ms"] for x in recs), sum(x["tokens"] for x in recs)
    eng.set_drafter(draft)
    return {"p": p_accept, "tok_s": tokens / (wall * 1e-3) if wall else None, "ms_per_step": wall / max(len(recs), 1), "steps": len(recs),
            "tokens_per_step": tokens / max(len(recs), 1), "proposed": sum(x["proposed"] for x in recs),
            "accepted": sum(x["accepted"] for x in recs), "outputs_identical": all(o == continuation for o in outs),
            "note": "real draft model cost (catch-up + chain) every round; the proposals handed to the engine are scripted"}


def draft_lane_line(args, metric, config, warmup):
    """The 1B configuration with the REAL draft model: the target's first `draft_layers` layers with their own pool
    (crates/kiln-models/src/draft.rs:128-162), proposing k tokens per round through kc_draft_chain. One step = one engine
    iteration = one propose (k chained draft decode forwards) + one (k + 1)-row verify forward + the settle walk.
    Reports verified tok/s with speculation on, the speculation-off rate beside it, and the draft lane's time per
    proposed token against its HBM floor (the draft's weight bytes at the measured copy bandwidth)."""
    import torch
    from kiln_b200 import api, host
    from kiln_b200.synth import PRESETS, synth_checkpoint, truncated
    preset, batch, k, lo, hi, gen = WORKLOADS[args.workload][:6]
    extras = WORKLOADS[args.workload][6]
    cfg = PRESETS[preset]
    dcfg = truncated(cfg, extras["draft_layers"])
    torch.cuda.set_device(0)
    ctx = api.Context(0)
    ck = synth_checkpoint(cfg, seed=0, device="cuda:0")
    dck = {n: t for n, t in ck.items() if not n.startswith("model.layers.") or int(n.split(".")[2]) < dcfg.num_hidden_layers}
    max_step = 256
    model = api.CudaModel(ctx, cfg, ck, max_step_tokens=max_step, max_step_seqs=4)
    dmodel = api.CudaModel(ctx, dcfg, dck, max_step_tokens=max_step, max_step_seqs=4)
    dmodel.set_stream_lane(True)     # the draft's chained decode forwards take the streaming and the small-weight kernels
    del ck, dck
    bs, nb = 16, 64 + (hi + gen + 64) // 16
    kv = api.PagedKv(ctx, model.kv_spec(nb, bs))
    dkv = api.PagedKv(ctx, dmodel.kv_spec(nb, bs))
    ec = host.EngineConfig(block_size=bs, num_blocks=nb, max_batch_tokens=max_step, prefill_chunk=128, prefill_fine_chunk=128,
                           prefix_cache=True, deterministic_decode_width=32, gamma=k, spec_max_batch=4, spec_min_acceptance=0.0,
                           max_key_len=0, batch_verify=True)
    eng = host.Engine(ec, host.StepModel.from_cuda(model, kv))
    import numpy as np
    rng = np.random.default_rng(1000)
    prompt = rng.integers(0, cfg.vocab_size, size=lo, dtype=np.int64).tolist()

    def run(n_requests, timed):
        """Generates `gen` tokens n_requests times (each request re-hits the prefix cache); returns per-step records."""
        recs, outs = [], []
        for _ in range(n_requests):
            a = eng.submit(prompt, gen)
            toks, fk, first = [], None, True
            while fk is None:
                s0 = eng.spec_stats()
                t0 = time.perf_counter()
                eng.step()
                t1 = time.perf_counter()
                s1 = eng.spec_stats()
                new, fk = eng.take_output(a)
                toks += new
                if timed and not first and new:   # the first iteration of a request is its (cached) prefill
                    recs.append({"wall_ms": (t1 - t0) * 1e3, "dev_ms": ctx.last_step_ms(), "tokens": len(new),
                                 "proposed": s1["proposed_total"] - s0["proposed_total"], "accepted": s1["accepted_total"] - s0["accepted_total"]})
                first = False
            outs.append(toks)
        return recs, outs

    _, base = run(1, False)                       # speculation off: the greedy continuation, and fills the prefix cache
    off_recs, off_outs = run(2 + warmup // 8, True)
    draft = host.DraftModel(dmodel, dkv, nb, bs)
    eng.set_drafter(draft)
    sampler = ClockSampler(0)
    sampler.start(record=False)
    run(1, False)                                  # warm-up with the drafter attached
    ctx.draft_stats(reset=True)
    sampler.arm()
    n_req = max(1, -(-args.steps * 3 // gen))      # about `steps` rounds at ~3 tokens per round
    torch.cuda.profiler.start()                     # lets `ncu --profile-from-start off` list the timed region only
    recs, outs = run(n_req, True)
    torch.cuda.profiler.stop()
    clocks = sampler.stop()
    d_ms, d_tok, d_calls = ctx.draft_stats()
    identical = all(o == base[0] for o in outs + off_outs)
    injected = injected_acceptance_run(eng, draft, prompt, gen, base[0], cfg.vocab_size, ctx, max(2, n_req // 2))
    identical = identical and injected.pop("outputs_identical")
    status = status_word(ctx)
    pk = peaks()
    tokens = sum(r["tokens"] for r in recs)
    wall = sum(r["wall_ms"] for r in recs)
    dev = sum(r["dev_ms"] for r in recs)            # device span of the verify forwards only
    off_tokens, off_wall = sum(r["tokens"] for r in off_recs), sum(r["wall_ms"] for r in off_recs)

    def qb(o, i, c):
        return o * i * c.bits / 8 + 2 * o * (i // c.group_size) * 2
    def weight_bytes(c):
        per = qb(c.num_attention_heads * c.head_dim, c.hidden_size, c) + 2 * qb(c.num_key_value_heads * c.head_dim, c.hidden_size, c) + \
            qb(c.hidden_size, c.num_attention_heads * c.head_dim, c) + 2 * qb(c.intermediate_size, c.hidden_size, c) + qb(c.hidden_size, c.intermediate_size, c)
        return c.num_hidden_layers * per + qb(c.vocab_size, c.hidden_size, c)
    floor_us = weight_bytes(dcfg) / (pk["hbm_gbs"] * 1e9) * 1e6
    draft_us = d_ms * 1e3 / max(d_tok, 1)
    verify_ms = sorted(r["dev_ms"] for r in recs)[len(recs) // 2]
    verify_floor_ms = weight_bytes(cfg) / (pk["hbm_gbs"] * 1e9) * 1e3
    launches = int(ctx.launch_count())
    gemv = stream_gemv_records(ctx, pk)
    line = {
        "metric": metric, "value": tokens / (wall * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": len(recs), "warmup": warmup,
        "ms_per_step": wall / len(recs), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": dict(config, draft=f"real draft model: first {dcfg.num_hidden_layers} layers of the target, own pool, kc_draft_chain"),
        "clocks": clocks, "device_status": status,
        "note": "batch 1: a step is latency-bound, so value is the end-to-end rate (wall clock of Engine::step: draft chain + verify + host)",
        "e2e": {"value": tokens / (wall * 1e-3), "unit": "tok/s", "ms_per_step": wall / len(recs),
                "h2d_bytes_per_step": int((k + 1) * 16 + (hi / 16 + 8) * 4 + k * 64), "d2h_bytes_per_step": int((k + 1) * 4 + 8 + k * 4)},
        "speculation_off": {"tok_s": off_tokens / (off_wall * 1e-3), "ms_per_step": off_wall / max(len(off_recs), 1)},
        "speedup_on_over_off": (tokens / wall) / (off_tokens / off_wall),
        "speedup_on_over_off_at_injected_acceptance": (injected["tok_s"] / (off_tokens / (off_wall * 1e-3))) if injected.get("tok_s") else None,
        "draft_lane": {"us_per_proposed_token": draft_us, "hbm_floor_us": floor_us, "frac_of_hbm_floor": floor_us / draft_us,
                       "proposed_tokens": d_tok, "chains": d_calls,
                       "draft_weight_bytes": weight_bytes(dcfg), "peak_source": pk["source"],
                       "lane": "kc_model_set_stream_lane: streaming kernel for the head, small-weight kernel for the layers (gated activation folded into the down projection, arg-max into the head's reduction)"},
        "injected_acceptance": injected,
        "stream_gemv": gemv,
        "verify_forward": {"p50_device_ms": verify_ms, "hbm_floor_ms": verify_floor_ms, "frac_of_hbm_floor": verify_floor_ms / verify_ms,
                           "rows": k + 1, "target_weight_bytes": weight_bytes(cfg)},
        "acceptance": {"proposed": sum(r["proposed"] for r in recs), "accepted": sum(r["accepted"] for r in recs),
                       "tokens_per_step": tokens / len(recs)},
        "spec_on_equals_off": {"sequences_checked": len(outs) + len(off_outs), "identical": bool(identical)},
        "gpu_launches": launches,
    }
    print(json.dumps(line))
    eng = None
    draft = None
    model.close(); dmodel.close(); kv.close(); dkv.close(); ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check-only", action="store_true",
                    help="run the workload once with speculation off and once with it on, to completion, and print only "
                         "whether the two outputs are identical (full-size parity property; no benchmark line)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama-3.1-8b-w4g64-verify-k5-bs32", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-record", action="store_true",
                    help="at --gpus N > 1, skip the tensor-parallel sub-record that follows the replica measurement")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)
    preset, batch, k, lo, hi, gen = WORKLOADS[args.workload][:6]
    metric = METRIC if args.workload == "llama-3.1-8b-w4g64-verify-k5-bs32" else f"verified tok/s, {args.workload}"
    config = {"workload": args.workload, "batch": batch, "k": k, "prompt_tokens": [lo, hi], "generated_tokens": gen,
              "kv_block": 16, "draft": "scripted, greedy token with p=0.7 else uniform-random id (seeded)",
              "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
              "l2": ("inputs larger than L2 (4.2 GB weights + ~5.9 GB KV per step vs 126 MB)" if args.workload == "llama-3.1-8b-w4g64-verify-k5-bs32" else "inputs larger than L2 (the weights and the KV of a step are far above 126 MB)")}

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(args.workload, None, None, args.steps, warmup)
        commit = 1 + sum(0.7 ** i for i in range(1, k + 1))
        val = commit / r["forward_s"]
        line = {"impl": "reference", "metric": metric, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": r["timed"],
                "warmup": warmup, "ms_per_step": r["mean_forward_s"] * 1e3, "p50_step_ms": r["forward_s"] * 1e3,
                "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": "tok/s", "cores": r["cores"], "threads": r["threads"], "kind": "port",
                                 "sample": r["sample"]},
                "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": ("CPU restatement of the reference's op graph (oracle/): the reference's MLX CPU path cannot be built here. "
                         f"One step = one sequence's verify forward; tokens per step = expected commit {commit:.3f} at p = 0.7. "
                         "It does not grow with --gpus: it is a host-cores baseline.")}
        print(json.dumps(line))
        return

    if len(WORKLOADS[args.workload]) > 6 and WORKLOADS[args.workload][6].get("draft_layers") and not args.check_only:
        if rank == 0:
            draft_lane_line(args, metric, config, warmup)
        return

    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        pin_rank_to_cores(local_rank, world)
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    want_cpu = rank == 0 and world == 1 and not args.no_cpu_baseline and not args.check_only
    w = Workload(args.workload, rank, local_rank, keep_cpu_sample=want_cpu, world=world, dist=dist)
    if w.tp > 1:
        config["parallelism"] = f"tp{world}"
    if args.check_only:
        t0 = time.time()
        base = w.run_off()
        off_s = time.time() - t0
        out = check_pass(w, base)
        out.update({"check_only": True, "workload": args.workload, "rank": rank, "speculation_off_s": round(off_s, 2),
                    "generated_tokens": sum(len(c) for c in base)})
        print(json.dumps(out))
        w.close()
        if dist:
            dist.destroy_process_group()
        return
    t0 = time.time()
    base = w.run_off()
    off_s = time.time() - t0
    plain_decode = w.plain_decode_pass()
    prefill = w.prefill_pass() if w.tp == 1 else None

    def barrier():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    w.ctx.sync()
    records, (checked, identical), arrivals, outs = timed_steps(w, base, args.steps, warmup, barrier, sampler)
    barrier()
    clocks = sampler.stop() if sampler else None
    dev_ms = sum(r["dev_ms"] for r in records)
    wall_ms = sum(r["wall_ms"] for r in records)
    tokens = sum(r["tokens"] for r in records)
    prof, prof_steps = roofline_pass(w, base)
    launches_per_step = sum(n for _, n in prof.values()) if prof else 0

    # finish the in-flight round so that the ON == OFF check covers full generations
    if arrivals:
        fin = w.engine.run_to_completion(arrivals)
        for a, cont in zip(arrivals, base):
            checked += 1
            identical &= (outs.get(a, []) + fin[a][0]) == cont
    device_status = status_word(w.ctx)

    from kiln_b200.replicas import combine_over_ranks
    step_ms = sorted(r["dev_ms"] for r in records)
    per_rank = None
    if dist:   # every rank's own figures, so that a slow rank or a slow host path shows in the line
        mine = torch.tensor([step_ms[len(step_ms) // 2], step_ms[-1], dev_ms / len(records), wall_ms / len(records), float(device_status)],
                            dtype=torch.float64, device=f"cuda:{local_rank}")
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        per_rank = [{"rank": i, "p50_step_ms": round(float(t[0]), 4), "max_step_ms": round(float(t[1]), 4),
                     "mean_step_ms": round(float(t[2]), 4), "mean_wall_ms": round(float(t[3]), 4), "device_status": int(t[4])}
                    for i, t in enumerate(allr)]
    if w.tp > 1 and rank != 0:
        tokens = 0   # every tensor-parallel rank verified the same tokens: count them once
    tot = combine_over_ranks(dist, f"cuda:{local_rank}", dev_ms, wall_ms, tokens, identical, world)
    dev_ms, wall_ms, tokens, identical = tot.device_ms, tot.wall_ms, tot.tokens, tot.all_identical
    tp_rec = None
    main_tp = w.tp
    cfg_main, mean_prompt, build_s = w.cfg, w.mean_prompt, w.build_s
    cpu_ctxs = [len(p) + gen // 2 for p in w.prompts]
    cpu_sample = w.cpu_sample
    w.close()
    del w
    torch.cuda.empty_cache()
    if dist and main_tp == 1 and not args.no_tp_record:
        # the configuration that shards (BASELINE config 5's layer shapes, batch, k and prompt lengths), on all N GPUs
        try:
            tp_rec = tp_record(rank, local_rank, world, dist, barrier)
        except Exception as exc:   # the replica measurement above stands; the record says what failed
            tp_rec = {"workload": TP_WORKLOAD, "ranks": world, "error": f"{type(exc).__name__}: {exc}"[:400]}
    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    pk = peaks()
    steps = len(records)
    mean_ctx = mean_prompt + gen / 2.0
    alg = algorithmic(cfg_main, batch, k, mean_ctx)
    gemm_ms, gemm_n = prof.get("gemm", (0.0, 0))
    # per-GPU rate: under tensor parallelism every rank multiplies 1 / tp of the weights
    gemm_tflops = alg["gemm_flops"] / main_tp / (gemm_ms * 1e-3) / 1e12 if gemm_ms else None
    p50 = step_ms[len(step_ms) // 2]
    value = tokens / (dev_ms * 1e-3)
    line = {
        "metric": metric, "value": value, "value_per_gpu": value / world, "unit": "tok/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": dev_ms / steps, "p50_step_ms": p50, "higher_is_better": True,
        "scaling": "strong" if main_tp > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config, "clocks": clocks, "device_status": device_status,
        "e2e": {"value": tokens / (wall_ms * 1e-3), "unit": "tok/s", "ms_per_step": wall_ms / steps,
                "h2d_bytes_per_step": int(batch * (k + 1) * 4 * 4 + batch * (mean_ctx / 16 + 2) * 4 + batch * 16 + batch * 12 + batch * (k + 1) * 8),
                "d2h_bytes_per_step": int(batch * (k + 1) * 4 + batch * 8 + 4)},
        "gpu_launches": int(launches_per_step * steps),
        "roofline": {"kernel": GEMM_KERNEL, "bound": "tensor",
                     "achieved": gemm_tflops, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": (gemm_tflops / pk["bf16_tflops_sustained"]) if gemm_tflops else None,
                     "traffic": (GEMM_DRAM_TRAFFIC_PER_WEIGHT_BYTE * alg["weight_bytes"] / main_tp / gemm_n) if gemm_n else None,
                     "traffic_unit": "bytes per launch (ncu dram read+write of one launch, scaled by weight bytes)",
                     "algorithmic_bytes_per_launch": (alg["weight_bytes"] / main_tp / gemm_n) if gemm_n else None,
                     "peak_source": pk["source"] + " (sustained: the kernel runs inside a long step)",
                     "launches_per_step": gemm_n, "ms_per_step": gemm_ms,
                     "algorithmic_flops_per_launch": alg["gemm_flops"] / main_tp / gemm_n if gemm_n else None},
        "step_roofline": {"bound": "hbm", "algorithmic_bytes_per_step": alg["bytes"], "achieved": alg["bytes"] / (p50 * 1e-3) / 1e9,
                          "peak": pk["hbm_gbs"] * main_tp, "unit": "GB/s", "frac": alg["bytes"] / (p50 * 1e-3) / 1e9 / (pk["hbm_gbs"] * main_tp),
                          "frac_of_nominal_8tbs": alg["bytes"] / (p50 * 1e-3) / 8e12, "mean_context": mean_ctx},
        "kernel_classes_ms_per_step": {k2: round(v[0], 4) for k2, v in prof.items()},
        "kernel_classes_launches_per_step": {k2: v[1] for k2, v in prof.items()},
        "acceptance": {"proposed": sum(r["proposed"] for r in records), "accepted": sum(r["accepted"] for r in records),
                       "tokens_per_step": tokens / steps / (1 if main_tp > 1 else world)},
        "spec_on_equals_off": {"sequences_checked": checked, "identical": bool(identical)},
        "setup_s": {"build_model": round(build_s, 1), "speculation_off_run": round(off_s, 1)},
        "plain_decode": plain_decode,
        "prefill": prefill,
    }
    if per_rank:
        line["per_rank"] = per_rank
    if tp_rec:
        line["tp"] = tp_rec
    if want_cpu:
        r = cpu_reference(args.workload, cpu_sample, cpu_ctxs, 6, 1, budget_s=45.0)
        per_seq_tokens = (tokens / steps) / batch
        line["cpu_baseline"] = {"value": per_seq_tokens / r["forward_s"], "unit": "tok/s", "cores": r["cores"], "threads": r["threads"],
                                "kind": "port", "sample": r["sample"], "ms_per_forward": r["forward_s"] * 1e3,
                                "ms_per_batch_round": r["forward_s"] * 1e3 * batch}
    print(json.dumps(line))
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
