#!/usr/bin/env python3
"""Benchmark: decode tokens a second of the Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

A step is one decode step of a batch of requests whose contexts stand at
``context`` tokens.  Weights are random N(0, 0.02); the caches are filled with
random keys and values (synthetic data) so that no time goes to prefilling them.
Prints ONE JSON line: ``value`` is the device-timed decode rate of the step
function, ``e2e`` the rate through the Python entry point (scheduler, sampling,
host tokens in and out; ``sampled_with_reference_defaults`` inside it: the same with the reference's default
sampling parameters instead of greedy picks), ``prefill`` a 2,048-token prompt in one step,
``roofline`` the bytes a decode step must read over its time, ``points`` the
decode rate at batch 1 and 64.  ``--workload serve`` and ``--workload long`` run
two further workloads end to end (continuous batching of 128 requests on the
Qwen3-1.7B shape; a 32,768-token prompt on the Qwen3-32B shape) and print a line
of their own.

Every decode point is the median of several repeats of ``--steps`` steps (at least 192 timed steps
together); between repeats the requests are cut back to where they began, so the contexts stay
just below ``--context``.  The bytes of the roofline are counted at the contexts that ran.  After
the timing, one step is run both from its CUDA graph and kernel by kernel and the two sets of
logits are compared, so the number belongs to a step that computes the right thing.

``--impl reference``: the reference is a Rust workspace and cannot be installed here (no cargo),
but its CUDA kernels compile unmodified for sm_100.  When ``baseline/_ref`` holds that library
(``python baseline/reference_kernels.py --build <reference checkout>``) the arm runs the same
decode step and prefill on the reference's own kernels through their C entry points, in the
order its runtime calls them, and says so in ``reference_class``; otherwise it prints why it is
unavailable.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, max_position_embeddings=40960, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False)
QWEN3_1_7B = dict(QWEN3_8B, hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  intermediate_size=6144, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600, tie_word_embeddings=False)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                        source="measured")
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, period_ms: int = 50):
        self.lines, self.proc, self.period_ms = [], None, period_ms
        self.marks = []                         # (name, first sample index, last sample index)

    def region(self, name):
        """with sampler.region("b8"): ... remembers which samples fell into the block."""
        sampler = self

        class _R:
            def __enter__(self):
                self.i0 = len(sampler.lines)

            def __exit__(self, *exc):
                sampler.marks.append((name, self.i0, len(sampler.lines)))
        return _R()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons, at = [], 0, set(), {}
        for i, l in enumerate(self.lines):
            parts = [x.strip() for x in l.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                at[i] = int(parts[0])
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        out = dict(sm_mhz=int(statistics.median(sm)) if sm else None, sm_max_mhz=mx or None,
                   reasons=sorted(reasons), samples=len(sm), period_ms=self.period_ms)
        for name, i0, i1 in self.marks:
            got = [at[i] for i in range(i0, i1) if i in at]
            out[f"sm_mhz_{name}"] = int(statistics.median(got)) if got else None
            out[f"samples_{name}"] = len(got)
        return out


def decode_bytes(cfg, n_layers, batch, context, esz=2):
    """Bytes one decode step has to read: every weight it uses once (the embedding rows
    of the batch, not the table) and the cache of the live requests."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    weights = (n_layers * per_layer + V * H) * esz + batch * H * esz
    norms = (n_layers * (2 * H + 2 * cfg.head_dim) + H) * 4
    kv = batch * context * 2 * cfg.kv_dim * esz * n_layers
    return weights + norms + kv


def prefill_flops(cfg, n_layers, T):
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    gemm = 2.0 * T * n_layers * per_layer + 2.0 * V * H
    attn = n_layers * cfg.num_attention_heads * 4.0 * cfg.head_dim * T * (T + 1) / 2
    return gemm + attn


def fill_contexts(eng, rids, context, seed=0):
    """Gives every request ``context`` tokens of random keys and values without running the model."""
    import torch
    g = torch.Generator(device=eng.device)
    g.manual_seed(seed)
    for rid in rids:
        if rid not in eng.manager.requests:
            eng.manager.add_request(rid)
        eng.manager.reserve(rid, context)
        eng.manager.commit(rid, context)
    for pool in eng.storage.paged:
        for layer in range(pool.shape[0]):
            pool[layer].copy_(torch.randn(pool[layer].shape, generator=g, device=eng.device, dtype=torch.float32)
                              .mul_(0.5).to(pool.dtype))


def repeats_for(steps: int) -> int:
    """Repeats of ``steps`` timed steps: three at least, and 192 timed steps together."""
    return max(3, -(-192 // max(steps, 1)))


def time_decode(eng, batch, context, steps, warmup, tag, check=False):
    """Device time of ``steps`` decode steps of ``batch`` requests whose contexts end just below
    ``context``: the median of ``repeats_for(steps)`` repeats, each bracketed by CUDA events; the
    requests are cut back to their first length between repeats.  Returns (ms per step, kernel
    launches of one repeat, mean context of the timed steps, ms of every repeat)."""
    import torch
    from airun_b200 import StepEntry
    from airun_b200.kernels import ops
    rids = [f"{tag}{i}" for i in range(batch)]
    start = context - steps - 1
    fill_contexts(eng, rids, start)
    V = eng.config.vocab_size
    toks = torch.randint(0, V, (steps + 1, batch), generator=torch.Generator().manual_seed(1)).tolist()
    picked = torch.zeros(batch, dtype=torch.int32, device=eng.device)

    def one(i):
        logits = eng.runner.step([StepEntry(r, [toks[i][j]], (0,)) for j, r in enumerate(rids)])
        ops.sample(logits, picked)
        return logits

    def rewind():
        for r in rids:
            eng.manager.truncate(r, start)

    for i in range(warmup):
        if i and i % steps == 0:
            rewind()
        one(i % steps)
    rewind()
    times, launches = [], 0
    for _ in range(repeats_for(steps)):
        torch.cuda.synchronize()
        l0 = ops.LAUNCHES[0] + getattr(eng.runner, "graph_launches", 0)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            one(i)
        ev1.record()
        torch.cuda.synchronize()
        launches = ops.LAUNCHES[0] + getattr(eng.runner, "graph_launches", 0) - l0
        times.append(ev0.elapsed_time(ev1) / steps)
        rewind()
    eng.runner.raise_on_device_error()
    if check:
        check_step(eng, rids, toks[0], start)
    for r in rids:
        eng.manager.free_request(r)
    # contexts of the timed steps: start + 1 .. start + steps keys
    return statistics.median(times), launches, start + (steps + 1) / 2.0, times


def check_step(eng, rids, tokens, start):
    """The step that was timed, once from its CUDA graph and once kernel by kernel: finite logits,
    the same picks, the same values up to the rounding of another split of the keys."""
    import torch
    from airun_b200 import StepEntry
    entries = [StepEntry(r, [tokens[j]], (0,)) for j, r in enumerate(rids)]
    a = eng.runner.step(entries).clone()
    for r in rids:
        eng.manager.truncate(r, start)
    graphs = eng.runner.use_graphs
    eng.runner.use_graphs = False
    try:
        b = eng.runner.step(entries).clone()
    finally:
        eng.runner.use_graphs = graphs
    for r in rids:
        eng.manager.truncate(r, start)
    torch.cuda.synchronize()
    if not (torch.isfinite(a).all() and torch.isfinite(b).all()):
        raise RuntimeError("the timed decode step gave non-finite logits")
    scale = float(b.abs().max())
    err = float((a - b).abs().max())
    if err > 0.02 * scale:
        raise RuntimeError(f"the timed decode step differs from its kernel-by-kernel run: {err:.4g} of {scale:.4g}")
    return err / max(scale, 1e-30)


def time_e2e(eng, batch, context, steps, warmup, sampled=False):
    """The same decode through the Python entry point: requests live in the scheduler, every step
    copies the step's inputs from pinned host memory and reads the sampled tokens back.  Median of
    three repeats of ``steps`` steps by the host clock.  ``sampled``: the requests sample with the
    reference's default parameters (temperature 0.8, top-k 40, top-p 0.95, min-p 0.05, repetition penalty 1.1
    over 64 tokens) instead of greedily, which brings the host's sampling chain into every step."""
    import torch
    from airun_b200 import SamplingParams
    from airun_b200.engine.scheduler import Request
    rids = [f"{'s' if sampled else 'e'}{i}" for i in range(batch)]
    reps = 3
    start = context - reps * steps - warmup - 1
    fill_contexts(eng, rids, start - 1)
    g = torch.Generator().manual_seed(2)
    reqs = []
    for rid in rids:
        prompt = torch.randint(0, eng.config.vocab_size, (start,), generator=g).tolist()
        r = Request(rid, prompt, SamplingParams(seed=len(reqs) + 1) if sampled else SamplingParams.greedy(), reps * steps + warmup + 8)
        r.num_computed = start - 1                # its cache stands one token short of the prompt
        eng.scheduler.running.append(r)
        reqs.append(r)
    for _ in range(warmup):
        eng.run_step()
    times = []
    gap0 = eng.stats.host_gap_ms
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.run_step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3 / steps)
    time_e2e.host_gap_ms = (eng.stats.host_gap_ms - gap0) / (reps * steps)
    assert all(len(r.output) == reps * steps + warmup for r in reqs), "the entry point did not decode every step"
    for r in reqs:
        eng.scheduler._finish(r, "bench")
    h2d = eng.runner.meta_host.numel() * 4 + eng._small_host.numel() * 4
    d2h = eng._picked_host.numel() * 4
    return statistics.median(times), h2d, d2h


def time_prefill(eng, T, runs=3, best=False):
    """Device time of one prompt of ``T`` tokens in one step: the median of ``runs`` runs after a first one (``best``: the
    fastest, for differences between two builds of the same step)."""
    import torch
    from airun_b200 import StepEntry
    toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
    times = []
    for i in range(runs + 1):
        rid = f"p{i}"
        eng.manager.add_request(rid)
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        eng.runner.step([StepEntry(rid, toks, (T - 1,))])
        ev1.record()
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1))
        eng.manager.free_request(rid)
    eng.runner.raise_on_device_error()
    return min(times[1:]) if best else statistics.median(times[1:])


def workload_serve(a) -> int:
    """Continuous batching: 128 requests at once, prompt lengths uniform in [64, 2048], 256 new
    tokens each, a step budget of 512 tokens (Qwen3-1.7B shape).  Runs the whole workload three times
    through the Python entry point and times the third run: a step shape is launched kernel by kernel the
    first time it is seen and captured the second time, so a shape that a run meets once is only replayed
    from its graph in the third."""
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config, SamplingParams
    d = dict(QWEN3_1_7B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    n_req, new = a.requests, a.new_tokens
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=n_req * (2048 + new + 16) + 4096, max_batch_tokens=a.budget,
        max_requests=n_req, max_context=2048 + new + 16))
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(64, 2049, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    res = {}
    for run in range(3):
        sampler = ClockSampler()
        sampler.start()
        steps0 = eng.stats.steps
        reqs = [eng.add_request(p, SamplingParams.greedy(), max_new_tokens=new) for p in prompts]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps = 0
        gap0 = eng.stats.host_gap_ms
        while eng.has_work():
            eng.run_step()
            steps += 1
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        # from reading a step's tokens to having launched the next step: the GPU may idle that long
        gap_sec = (eng.stats.host_gap_ms - gap0) / 1e3
        clocks = sampler.stop()
        gen = sum(len(r.output) for r in reqs)
        assert gen == n_req * new, "a request ended early"
        res = {"workload": "serve", "model": "Qwen3-1.7B shape, random weights", "layers": cfg.num_hidden_layers,
               "layers_full": 28, "requests": n_req, "prompt_tokens": sum(lens), "generated_tokens": gen,
               "step_budget": a.budget, "seconds": round(sec, 3), "steps": steps,
               "ms_per_step": round(sec * 1e3 / steps, 3),
               "total_tokens_per_s": round((sum(lens) + gen) / sec, 1), "decode_tokens_per_s": round(gen / sec, 1),
               "host_gap_seconds": round(gap_sec, 3), "host_share_at_most": round(gap_sec / sec, 4),
               "preemptions": eng.scheduler.stats["preemptions"], "dtype": a.dtype, "clocks": clocks}
    print(json.dumps(res))
    return 0


def workload_long(a) -> int:
    """Long context: one 32,768-token prompt in portions of 2,048, then 512 tokens decoded alone, then
    15 forks of the request (reading the same prompt pages: 16 private caches would not fit beside
    the weights; attention reads those pages once per step for all 16) and 512 tokens decoded by all
    16 (Qwen3-32B shape)."""
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config, SamplingParams
    d = dict(QWEN3_32B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    T, new, forks = a.prompt, a.new_tokens, a.forks
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=T + (forks + 2) * (2 * new + 32) + 4096,
        max_batch_tokens=2048, max_requests=forks + 1, max_context=T + 2 * new + 32))
    L = cfg.num_hidden_layers
    pk = peaks()
    esz = 2 if a.dtype == "bfloat16" else 4
    prompt = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(5)).tolist()
    # warm-up: a short request through the same kernels (prefill portion, decode graph)
    eng.generate(prompt[:4096], SamplingParams.greedy(), max_new_tokens=8)
    sampler = ClockSampler()
    sampler.start()
    parent = eng.add_request(prompt, SamplingParams.greedy(), max_new_tokens=2 * new + 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    while not parent.output:
        eng.run_step()
    torch.cuda.synchronize()
    t_pre = time.perf_counter() - t0
    t0 = time.perf_counter()
    while len(parent.output) < 1 + new:
        eng.run_step()
    torch.cuda.synchronize()
    t_b1 = time.perf_counter() - t0
    kids = [eng.fork_request(parent, max_new_tokens=new) for _ in range(forks)]
    eng.run_step()                                   # the forks' first step is not a pure decode step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_steps = 0
    while len(kids[0].output) < new:
        eng.run_step()
        n_steps += 1
    torch.cuda.synchronize()
    t_bn = time.perf_counter() - t0
    clocks = sampler.stop()
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    per_layer = (cfg.q_dim + 2 * cfg.kv_dim) * H + H * cfg.q_dim + 3 * H * I
    flops = 2.0 * T * L * per_layer + L * cfg.num_attention_heads * 4.0 * cfg.head_dim * T * (T + 1) / 2
    b1_bytes = decode_bytes(cfg, L, 1, T + new // 2, esz)
    bn_bytes = decode_bytes(cfg, L, forks + 1, T + new + new // 2, esz)
    once_bytes = decode_bytes(cfg, L, 1, T, esz) + (forks + 1) * (new + new // 2) * 2 * cfg.kv_dim * esz * L
    print(json.dumps({
        "workload": "long", "model": "Qwen3-32B shape, random weights", "layers": L, "layers_full": 64,
        "prompt_tokens": T, "portion": 2048, "dtype": a.dtype, "peaks": pk["source"],
        "prefill": {"seconds": round(t_pre, 3), "tokens_per_s": round(T / t_pre, 1),
                    "frac_of_bf16_peak": round(flops / t_pre / (pk["bf16_tflops"] * 1e12), 4)},
        "decode_b1": {"tokens": new, "tokens_per_s": round(new / t_b1, 2), "ms_per_step": round(t_b1 * 1e3 / new, 3),
                      "hbm_frac": round(b1_bytes / (t_b1 / new) / 1e9 / pk["hbm_gbs"], 4)},
        f"decode_b{forks + 1}": {"tokens": n_steps * (forks + 1), "tokens_per_s": round(n_steps * (forks + 1) / t_bn, 2),
                                 "ms_per_step": round(t_bn * 1e3 / n_steps, 3), "shared_prompt_pages": True,
                                 "hbm_frac_if_every_request_reads_the_prompt":
                                     round(bn_bytes / (t_bn / n_steps) / 1e9 / pk["hbm_gbs"], 4),
                                 "hbm_frac_prompt_read_once":
                                     round(once_bytes / (t_bn / n_steps) / 1e9 / pk["hbm_gbs"], 4)},
        "clocks": clocks}))
    return 0


REFERENCE_CLASS = "reference kernels through their C ABI; host loop restated, Rust runtime not buildable"


def workload_ablate(a) -> int:
    """What each kind of kernel adds to the decode step: the step is captured and timed again with one kind left out.

    The logits of such a step are wrong on purpose; only its time is read.  The difference to the whole step is the
    kind's marginal cost on the step's critical path, which is what a faster kernel could win back: it is smaller than
    the kernel's own duration where the next kernel's prologue overlaps it (programmatic dependent launch).
    ``rmsnorm_as_empty_kernel`` puts a kernel that does next to nothing in the norm's place: what one more
    launch boundary costs.  One JSON line per kind.
    """
    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config
    from airun_b200.kernels import fast, ops
    d = dict(QWEN3_8B)
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    L = cfg.num_hidden_layers
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype="bfloat16", page_size=16, cache_tokens=64 * a.context + 4096, max_batch_tokens=2048, max_requests=64,
        max_context=a.context))
    qkv_rows = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    kinds = {(qkv_rows, cfg.hidden_size): "product_qkv",
             (2 * cfg.intermediate_size, cfg.hidden_size): "product_gate_up",
             (cfg.hidden_size, cfg.intermediate_size): "product_down",
             (cfg.vocab_size, cfg.hidden_size): "product_head"}
    kinds.setdefault((cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim), "product_o")
    skip: set = set()
    gemm, rms, post, att = fast.gemm_tcgen05, ops.rmsnorm, ops.qkv_post, fast.attn_decode
    src, rows, dst = (torch.zeros(8, 64, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"),
                      torch.zeros(8, 64, device="cuda"))

    def gemm_or_not(x, w, *args, **kw):
        return None if kinds.get(tuple(w.shape)) in skip else gemm(x, w, *args, **kw)

    def rms_or_not(*args, **kw):
        if "rmsnorm" in skip:
            return None
        if "rmsnorm_as_empty_kernel" in skip:
            return ops.gather_rows(src, rows, dst)
        return rms(*args, **kw)

    fast.gemm_tcgen05 = gemm_or_not
    ops.rmsnorm = rms_or_not
    ops.qkv_post = lambda *args, **kw: None if "qkv_post" in skip else post(*args, **kw)
    fast.attn_decode = lambda *args, **kw: None if "attention" in skip else att(*args, **kw)
    base = {}
    try:
        for kind in [None, "rmsnorm", "rmsnorm_as_empty_kernel", "qkv_post", "attention", *sorted(set(kinds.values()))]:
            skip.clear()
            if kind:
                skip.add(kind)
            eng.runner.graphs.clear()
            eng.runner._warm_buckets.clear()
            res = {}
            for b in (8, 1, 64):
                ms, _, _, _ = time_decode(eng, b, a.context, a.steps, a.warmup, f"ab{b}_")
                res[f"b{b}"] = round(ms, 4)
                if kind is None:
                    base[b] = ms
            line = {"workload": "ablate", "left_out": kind, "layers": L, "context": a.context, "ms_per_step": res}
            if kind:
                per = 1 if kind == "product_head" else L
                line["marginal_us_each" if kind == "product_head" else "marginal_us_per_layer"] = {
                    f"b{b}": round((base[b] - res[f"b{b}"]) * 1e3 / per, 2) for b in (8, 1, 64)}
            print(json.dumps(line), flush=True)
    finally:
        fast.gemm_tcgen05, ops.rmsnorm, ops.qkv_post, fast.attn_decode = gemm, rms, post, att
    return 0


# ---------------------------------------------------------------------------------------------------------
# The Vedizen design beside the dense Qwen3 decoder at equal size (--workload vedizen)
VEDIZEN_SIZES = {
    # width, feed-forward, heads, KV heads: the layer sizes of the Qwen3-1.7B and Qwen3-8B shapes
    "2048": dict(width=2048, ff=6144, heads=16, kv_heads=8),
    "4096": dict(width=4096, ff=12288, heads=32, kv_heads=8),
}
VEDIZEN_VOCAB, VEDIZEN_RUNS = 32768, 6


def vedizen_pair(size: dict):
    """(Vedizen configuration, Qwen3 configuration) with the same width, feed-forward size, head counts, vocabulary
    and six layer runs a token: four Vedizen layers (gated linear attention, two differential attention layers with
    chunks of 2,048 positions, gated linear attention) of which the first two run twice, against six Qwen3 layers.
    A differential attention layer has exactly the weights of a Qwen3 layer (two query/key maps of 64 where Qwen3 has
    one of 128); a gated linear attention layer has a third more in its mixer."""
    from airun_b200 import Qwen3Config, VedizenConfig
    W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
    mlp = dict(kind="dense", ff=F, limit=7.0)
    gla = dict(type="gla", mixer=dict(heads=H, dim=64, vdim=128, tau=16.0), mlp=mlp)
    att = dict(type="attention", mixer=dict(heads=H, kv_heads=G, dim=64, vdim=128, scale=0.125, softcap=50.0, diff=0.5,
                                            mask=dict(size=2048)), mlp=mlp)
    ved = VedizenConfig.from_dict(dict(architecture="Vedizen", vocab=VEDIZEN_VOCAB, width=W, embedding=dict(scale=1.0),
                                       norm=dict(eps=1e-5), layers=[gla, att, att, gla], loop=dict(start=0, stop=2, times=2)))
    qw = Qwen3Config.from_dict(dict(QWEN3_8B, vocab_size=VEDIZEN_VOCAB, hidden_size=W, num_hidden_layers=VEDIZEN_RUNS,
                                    num_attention_heads=H, num_key_value_heads=G, head_dim=128, intermediate_size=F))
    return ved, qw


def fill_states(eng, seed=1):
    import torch
    g = torch.Generator(device=eng.device)
    g.manual_seed(seed)
    for st in eng.storage.state:
        st.copy_(torch.randn(st.shape, generator=g, device=eng.device, dtype=torch.float32).mul_(0.1))


def time_decode_onward(eng, batch, context, steps, warmup, tag):
    """Device time of a decode step of ``batch`` requests whose contexts begin at ``context`` and grow as they
    decode (requests with a recurrent state cannot be cut back between repeats): median of three repeats."""
    import torch
    from airun_b200 import StepEntry
    from airun_b200.kernels import ops
    rids = [f"{tag}{i}" for i in range(batch)]
    fill_contexts(eng, rids, context)
    fill_states(eng)
    toks = torch.randint(0, eng.config.vocab_size, (batch,), generator=torch.Generator().manual_seed(1)).tolist()
    picked = torch.zeros(batch, dtype=torch.int32, device=eng.device)
    entries = [StepEntry(r, [toks[j]], (0,)) for j, r in enumerate(rids)]

    def one():
        ops.sample(eng.runner.step(entries), picked)

    for _ in range(warmup):
        one()
    times = []
    for _ in range(3):
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            one()
        ev1.record()
        torch.cuda.synchronize()
        times.append(ev0.elapsed_time(ev1) / steps)
    eng.runner.raise_on_device_error()
    for r in rids:
        eng.manager.free_request(r)
    return statistics.median(times)


def workload_vedizen(a) -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 and 64 at a context of 1,024) of the Vedizen design and of
    the Qwen3 decoder at equal size, through the step function and its CUDA graphs, and how long each kind of kernel of
    the two runs inside the prefill step and the batch-64 decode step (CUDA events around every call of the kind, the
    step launched kernel by kernel), with the fraction of the measured peak that its bytes or FLOPs over that time come
    to.  One JSON line per size."""
    import torch
    from airun_b200 import Engine, EngineOptions
    from airun_b200.kernels import fast, ops
    pk = peaks()
    T, ctx_len, steps = 2048, 1024, max(8, min(a.steps, 32))
    fp32_peak = 148 * 128 * 2 * 1.965e9          # FMA lanes x 2 x the highest SM clock: nominal, no measured figure
    for name in (a.sizes.split(",") if a.sizes else list(VEDIZEN_SIZES)):
        size = VEDIZEN_SIZES[name]
        W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
        line = {"workload": "vedizen", "size": size, "layer_runs": VEDIZEN_RUNS, "vocab": VEDIZEN_VOCAB, "dtype": "bf16",
                "data": "synthetic, random weights", "prompt": T, "decode_context": ctx_len, "peaks": pk["source"], "models": {}}
        for model, cfg in zip(("vedizen", "qwen3"), vedizen_pair(size)):
            eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
                dtype="bfloat16", page_size=16, cache_tokens=64 * (ctx_len + 4 * steps + 64) + 4096, max_batch_tokens=T,
                max_requests=64, max_context=max(T, ctx_len + 4 * steps + 64)))
            kinds = {}                       # kind -> (module, function name, bytes or FLOPs at prefill, at batch 64, bound)
            if model == "vedizen":
                n_att, n_gla = 3, 3          # runs of each mixer among the six
                kinds["norm (dynamic tanh)"] = (ops, "dyt_norm", lambda t: 7 * t * W * 14.0, "hbm")
                kinds["q/k/v bias + cache write"] = (ops, "qkv_bias_store", lambda t: n_att * t * ((H + G) * 128 + G * 128) * 6.0, "hbm")
                kinds["differential attention"] = (fast, "diff_attention_bf16", None, "mixed")
                kinds["linear attention: decay"] = (ops, "gla_decay", lambda t: n_gla * t * H * 64 * 4.0, "hbm")
                kinds["linear attention: recurrence"] = (ops, "gla_recurrent", None, "mixed")
                kinds["linear attention: norm and gate"] = (ops, "gla_out_gate", lambda t: n_gla * t * H * 128 * 10.0, "hbm")
                kinds["gate/up product + gated unit"] = (fast, "linear_glu_clamped_bf16", lambda t: 6 * 2.0 * t * W * 2 * F, "tensor")
                att_flops = n_att * H * 2 * (2 * 64 + 2 * 128) * T * (T + 1) / 2
                att_bytes = lambda b, c: n_att * b * c * G * (128 + 128) * 2.0
                rec_flops = n_gla * T * H * 64 * 128 * 5.0
                rec_bytes = lambda b: n_gla * b * H * 64 * 128 * 4.0 * 2
            else:
                kinds["norm (rms)"] = (ops, "rmsnorm", lambda t: 13 * t * W * 14.0, "hbm")
                kinds["q/k norm + rotary + cache write"] = (ops, "qkv_post", lambda t: 6 * t * (H + 2 * G) * 128 * 6.0, "hbm")
                kinds["attention"] = (fast, "attention_bf16", None, "mixed")
                kinds["gate/up product + gated unit"] = (fast, "linear_swiglu_bf16", lambda t: 6 * 2.0 * t * W * 2 * F, "tensor")
                att_flops = 6 * H * 4 * 128 * T * (T + 1) / 2
                att_bytes = lambda b, c: 6 * b * c * G * 256 * 2.0
            res = {}
            pre_ms = time_prefill(eng, T, runs=5)
            b64 = time_decode_onward(eng, 64, ctx_len, steps, a.warmup, "v")
            b8 = time_decode_onward(eng, 8, ctx_len, steps, a.warmup, "w")
            res["prefill"] = {"ms": round(pre_ms, 3), "tokens_per_s": round(T / pre_ms * 1e3, 1)}
            res["decode_b8"] = {"ms_per_step": round(b8, 4), "tokens_per_s": round(8 / b8 * 1e3, 1)}
            res["decode_b64"] = {"ms_per_step": round(b64, 4), "tokens_per_s": round(64 / b64 * 1e3, 1)}
            # every kind of kernel timed where it runs: the same two steps kernel by kernel (no graph), CUDA events
            # around each call of the kind, summed over the step; the fastest of four such steps
            spans = {k: [] for k in kinds}
            real = {k: getattr(mod, fn) for k, (mod, fn, _, _) in kinds.items()}

            def timed(kind):
                def call(*x, **kw):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = real[kind](*x, **kw)
                    e1.record()
                    spans[kind].append((e0, e1))
                    return out
                return call

            def step_times(run):
                best = {}
                for _ in range(4):
                    for k in spans:
                        spans[k].clear()
                    run()
                    torch.cuda.synchronize()
                    for k, evs in spans.items():
                        us = sum(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3
                        best[k] = min(best.get(k, us), us)
                return best

            from airun_b200 import StepEntry
            toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
            rids = [f"k{i}" for i in range(64)]
            count = [0]

            def run_prefill():
                count[0] += 1
                eng.manager.add_request(f"kp{count[0]}")
                eng.runner.step([StepEntry(f"kp{count[0]}", toks, (T - 1,))])
                eng.manager.free_request(f"kp{count[0]}")

            def run_decode():
                eng.runner.step([StepEntry(r, [toks[j]], (0,)) for j, r in enumerate(rids)])

            graphs, eng.runner.use_graphs = eng.runner.use_graphs, False
            for k, (mod, fn, _, _) in kinds.items():
                setattr(mod, fn, timed(k))
            try:
                pre_t = step_times(run_prefill)
                fill_contexts(eng, rids, ctx_len)
                fill_states(eng)
                dec_t = step_times(run_decode)
            finally:
                for k, (mod, fn, _, _) in kinds.items():
                    setattr(mod, fn, real[k])
                eng.runner.use_graphs = graphs
            for r in rids:
                eng.manager.free_request(r)
            res["kernels"] = {}
            for kind, (mod, fn, work, bound) in kinds.items():
                pre_us, dec_us = pre_t[kind], dec_t[kind]
                row = {"prefill_us": round(pre_us, 1), "decode_b64_us": round(dec_us, 1)}
                if kind in ("differential attention", "attention"):
                    row["prefill_frac_of_bf16_peak"] = round(att_flops / max(pre_us, 1e-3) / 1e6 / (pk["bf16_tflops"] * 1e12) * 1e12, 4)
                    row["decode_b64_frac_of_hbm"] = round(att_bytes(64, ctx_len) / max(dec_us, 1e-3) / 1e3 / pk["hbm_gbs"], 4)
                elif kind == "linear attention: recurrence":
                    row["prefill_frac_of_nominal_fp32"] = round(rec_flops / max(pre_us, 1e-3) * 1e6 / fp32_peak, 4)
                    row["decode_b64_frac_of_hbm"] = round(rec_bytes(64) / max(dec_us, 1e-3) / 1e3 / pk["hbm_gbs"], 4)
                elif bound == "hbm":
                    row["prefill_frac_of_hbm"] = round(work(T) / max(pre_us, 1e-3) / 1e3 / pk["hbm_gbs"], 4)
                    row["decode_b64_frac_of_hbm"] = round(work(64) / max(dec_us, 1e-3) / 1e3 / pk["hbm_gbs"], 4)
                else:
                    row["prefill_frac_of_bf16_peak"] = round(work(T) / max(pre_us, 1e-3) * 1e6 / (pk["bf16_tflops"] * 1e12), 4)
                    row["decode_b64_frac_of_hbm"] = round(6 * 2.0 * W * 2 * F / max(dec_us, 1e-3) / 1e3 / pk["hbm_gbs"], 4)
                res["kernels"][kind] = row
            line["models"][model] = res
            del eng
            torch.cuda.empty_cache()
        print(json.dumps(line), flush=True)
    return 0



# ---------------------------------------------------------------------------------------------------------
# The Pogarax design beside the Vedizen design at equal size (--workload pogarax)
def pogarax_pair(size: dict):
    """(Pogarax configuration, Vedizen configuration) with the same width, head counts, vocabulary and six layer runs a
    token.  Pogarax: gated delta rule (heads x 64 x 128, q/k heads halved, 4 taps) with a dense feed-forward, latent
    attention (heads x (128 + 64), values of 128, latent 512, queries through a latent of width/2, window 2,048) with 16
    experts of half the feed-forward size of which a token uses two (the dense layer's FLOPs), the same pair again with the
    attention on the first one's cached rows, a third delta layer, and a time mix (width/64 heads of 64) with experts.
    Vedizen: as in its own workload (gated linear attention heads x 64 x 128, differential attention in chunks of 2,048)."""
    from airun_b200.config import PogaraxConfig
    W, F, H = size["width"], size["ff"], size["heads"]
    dense = dict(kind="dense", ff=F)
    moe = dict(kind="moe", expert=dict(ff=F // 2), router=dict(experts=16, top=2))
    delta = dict(type="channel_delta", mixer=dict(heads=H, kv_heads=H // 2, dim=64, vdim=128, conv=4), mlp=dense)
    lat = dict(heads=H, dim=128, rot_dim=64, vdim=128, q_rank=W // 2, kv_rank=512, scale=192 ** -0.5, mask=dict(size=2048),
               rot=dict(dims=64, base=1e6, scaling=dict(factor=4.0, original=4096, fast=32.0, slow=1.0)))
    layers = [delta, dict(type="latent_attention", mixer=dict(lat), mlp=moe), delta,
              dict(type="latent_attention", mixer=dict(lat, kv_from=1), mlp=moe), delta,
              dict(type="wkv", mixer=dict(heads=W // 64, dim=64), mlp=moe)]
    pog = PogaraxConfig.from_dict(dict(architecture="Pogarax", vocab=VEDIZEN_VOCAB, width=W, norm=dict(eps=1e-5),
                                       residual_mult=0.7, layers=layers))
    return pog, vedizen_pair(size)[0]


def workload_pogarax(a) -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 and 64 at a context of 1,024) of the Pogarax design and of
    the Vedizen design at equal size, through the step function and its CUDA graphs, and how long each kind of kernel
    runs inside the prefill step and the batch-64 decode step (CUDA events around every call of the kind, the step
    launched kernel by kernel), with the fraction of the measured peak its bytes or FLOPs over that time come to.  One
    JSON line per size."""
    import torch
    from airun_b200 import Engine, EngineOptions, StepEntry
    from airun_b200.kernels import fast, ops
    from airun_b200.parts import latent_attention as latent_part
    pk = peaks()
    T, ctx_len, steps = 2048, 1024, max(8, min(a.steps, 32))
    fp32_peak = 148 * 128 * 2 * 1.965e9          # FMA lanes x 2 x the highest SM clock: nominal, no measured figure
    for name in (a.sizes.split(",") if a.sizes else list(VEDIZEN_SIZES)):
        size = VEDIZEN_SIZES[name]
        W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
        line = {"workload": "pogarax", "size": size, "layer_runs": 6, "vocab": VEDIZEN_VOCAB, "dtype": "bf16",
                "data": "synthetic, random weights", "prompt": T, "decode_context": ctx_len, "peaks": pk["source"], "models": {}}
        for model, cfg in zip(("pogarax", "vedizen"), pogarax_pair(size)):
            eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
                dtype="bfloat16", page_size=16, cache_tokens=64 * (ctx_len + 4 * steps + 64) + 4096, max_batch_tokens=T,
                max_requests=64, max_context=max(T, ctx_len + 4 * steps + 64)))
            win = lambda t: sum(min(i + 1, 2048) for i in range(t))      # keys all tokens of a t-token prompt see together
            # kind -> (module, function, work at t tokens of one prompt or None, work at a batch of b single tokens, bound)
            if model == "pogarax":
                R, rd, D, Dv, qr, Fe, E, top, Hw = 512, 64, 128, 128, W // 2, F // 2, 16, 2, W // 64
                kinds = {
                    "norm on the output + add (rms)": (ops, "postnorm_add", lambda t: 12 * t * W * 14.0, lambda b: 12 * b * W * 14.0, "hbm"),
                    "latent: norms, rotation, cache write": (ops, "latent_prepare", lambda t: 2 * t * ((qr + R + rd) * 4.0 + qr * 2 + (R + rd)),
                                                             lambda b: 2 * b * ((qr + R + rd) * 4.0 + qr * 2 + (R + rd)), "hbm"),
                    "latent: query parts and rotation": (ops, "latent_query", lambda t: 2 * t * H * ((D + rd) * 4.0 + (D + rd) * 2),
                                                         lambda b: 2 * b * H * ((D + rd) * 4.0 + (D + rd) * 2), "hbm"),
                    "latent attention": (fast, "latent_attention_bf16", lambda t: 2 * H * 2.0 * (2 * R + rd) * win(t),
                                         lambda b: 2 * b * min(ctx_len, 2048) * (R + rd) * 2.0, "mixed"),
                    "products per head (Wuk, Wuv)": (latent_part, "head_linear", lambda t: 2 * t * H * 2.0 * (D * R + R * Dv),
                                                     lambda b: 2 * H * (D * R + R * Dv) * 2.0, "tensor"),
                    "delta rule: convolution": (ops, "short_conv", lambda t: 3 * t * (H * 64 + H * 128) * 8.0, lambda b: 3 * b * (H * 64 + H * 128) * 8.0, "hbm"),
                    "low-rank second halves (decays, gate)": (ops, "lowrank_act", lambda t: t * (3 * (H * 64 + H * 128) + W) * 4.0,
                                                              lambda b: b * (3 * (H * 64 + H * 128) + W) * 4.0, "hbm"),
                    "recurrence (delta rule, time mix)": (ops, "recurrent_state", lambda t: t * (3 * H * 64 * 128 * 9.0 + Hw * 64 * 64 * 6.0),
                                                          lambda b: b * (3 * H * 64 * 128 + Hw * 64 * 64) * 8.0, "fp32"),
                    "norm and gate of the heads": (ops, "gla_out_gate", lambda t: t * (3 * H * 128 + W) * 10.0, lambda b: b * (3 * H * 128 + W) * 10.0, "hbm"),
                    "token shift": (ops, "token_shift", lambda t: t * W * 14.0, lambda b: b * W * 14.0, "hbm"),
                    "gate/up product + gated unit (dense)": (fast, "linear_swiglu_bf16", lambda t: 3 * 2.0 * t * W * 2 * F, lambda b: 3 * W * 2 * F * 2.0, "tensor"),
                    "expert products (gate/up + unit, down)": (fast, "grouped_linear_bf16", lambda t: 3 * t * top * 6.0 * W * Fe,
                                                               lambda b: 3 * min(E, b * top) * 3 * W * Fe * 2.0, "tensor"),
                    "router": (ops, "moe_route", lambda t: 3 * t * W * 2.0, lambda b: 3 * (b * W + E * W) * 2.0, "hbm"),
                    "rows to experts and back": (ops, "moe_scatter", lambda t: 3 * t * (W * 2 + top * W * 2.0), lambda b: 3 * b * (W * 2 + top * W * 2.0), "hbm"),
                    "sum of a token's experts": (ops, "moe_combine", lambda t: 3 * t * (top + 1) * W * 4.0, lambda b: 3 * b * (top + 1) * W * 4.0, "hbm"),
                }
            else:
                n_att, n_gla = 3, 3
                kinds = {
                    "norm (dynamic tanh)": (ops, "dyt_norm", lambda t: 7 * t * W * 14.0, lambda b: 7 * b * W * 14.0, "hbm"),
                    "q/k/v bias + cache write": (ops, "qkv_bias_store", lambda t: n_att * t * ((H + G) * 128 + G * 128) * 6.0,
                                                 lambda b: n_att * b * ((H + G) * 128 + G * 128) * 6.0, "hbm"),
                    "differential attention": (fast, "diff_attention_bf16", lambda t: n_att * H * 2.0 * (2 * 64 + 2 * 128) * t * (t + 1) / 2,
                                               lambda b: n_att * b * ctx_len * G * 256 * 2.0, "mixed"),
                    "linear attention: decay": (ops, "gla_decay", lambda t: n_gla * t * H * 64 * 4.0, lambda b: n_gla * b * H * 64 * 4.0, "hbm"),
                    "linear attention: recurrence": (ops, "gla_recurrent", lambda t: n_gla * t * H * 64 * 128 * 5.0,
                                                     lambda b: n_gla * b * H * 64 * 128 * 8.0, "fp32"),
                    "linear attention: norm and gate": (ops, "gla_out_gate", lambda t: n_gla * t * H * 128 * 10.0, lambda b: n_gla * b * H * 128 * 10.0, "hbm"),
                    "gate/up product + gated unit": (fast, "linear_glu_clamped_bf16", lambda t: 6 * 2.0 * t * W * 2 * F, lambda b: 6 * W * 2 * F * 2.0, "tensor"),
                }
            res = {}
            pre_ms = time_prefill(eng, T, runs=5)
            b64 = time_decode_onward(eng, 64, ctx_len, steps, a.warmup, "v")
            b8 = time_decode_onward(eng, 8, ctx_len, steps, a.warmup, "w")
            res["prefill"] = {"ms": round(pre_ms, 3), "tokens_per_s": round(T / pre_ms * 1e3, 1)}
            res["decode_b8"] = {"ms_per_step": round(b8, 4), "tokens_per_s": round(8 / b8 * 1e3, 1)}
            res["decode_b64"] = {"ms_per_step": round(b64, 4), "tokens_per_s": round(64 / b64 * 1e3, 1)}
            spans = {k: [] for k in kinds}
            real = {k: getattr(v[0], v[1]) for k, v in kinds.items()}

            def timed(kind):
                def call(*x, **kw):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = real[kind](*x, **kw)
                    e1.record()
                    spans[kind].append((e0, e1))
                    return out
                return call

            def step_times(run):
                best = {}
                for _ in range(4):
                    for k in spans:
                        spans[k].clear()
                    run()
                    torch.cuda.synchronize()
                    for k, evs in spans.items():
                        us = sum(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3
                        best[k] = min(best.get(k, us), us)
                return best

            toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
            rids = [f"k{i}" for i in range(64)]
            count = [0]

            def run_prefill():
                count[0] += 1
                eng.manager.add_request(f"kp{count[0]}")
                eng.runner.step([StepEntry(f"kp{count[0]}", toks, (T - 1,))])
                eng.manager.free_request(f"kp{count[0]}")

            def run_decode():
                eng.runner.step([StepEntry(r, [toks[j]], (0,)) for j, r in enumerate(rids)])

            graphs, eng.runner.use_graphs = eng.runner.use_graphs, False
            for k, v in kinds.items():
                setattr(v[0], v[1], timed(k))
            try:
                pre_t = step_times(run_prefill)
                fill_contexts(eng, rids, ctx_len)
                fill_states(eng)
                dec_t = step_times(run_decode)
            finally:
                for k, v in kinds.items():
                    setattr(v[0], v[1], real[k])
                eng.runner.use_graphs = graphs
            for r in rids:
                eng.manager.free_request(r)
            res["kernels"] = {}
            for kind, (_, _, work_p, work_d, bound) in kinds.items():
                pre_us, dec_us = max(pre_t[kind], 1e-3), max(dec_t[kind], 1e-3)
                row = {"prefill_us": round(pre_us, 1), "decode_b64_us": round(dec_us, 1)}
                if bound == "hbm":
                    row["prefill_frac_of_hbm"] = round(work_p(T) / pre_us / 1e3 / pk["hbm_gbs"], 4)
                elif bound == "fp32":
                    row["prefill_frac_of_nominal_fp32"] = round(work_p(T) / pre_us * 1e6 / fp32_peak, 4)
                else:
                    row["prefill_frac_of_bf16_peak"] = round(work_p(T) / pre_us * 1e6 / (pk["bf16_tflops"] * 1e12), 4)
                row["decode_b64_frac_of_hbm"] = round(work_d(64) / dec_us / 1e3 / pk["hbm_gbs"], 4)
                res["kernels"][kind] = row
            line["models"][model] = res
            del eng
            torch.cuda.empty_cache()
        print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------------------
# The Gamanex design beside the dense Qwen3 decoder at equal size (--workload gamanex)
def gamanex_pair(size: dict):
    """(Gamanex configuration, Qwen3 configuration) with the same width, head counts (heads of 128), vocabulary and six
    layers.  Gamanex: attention without softmax in every layer, the second and fourth on the keys and values of the layer
    before them; feed-forwards in turn dense (relu squared, 3/2 of the size: two matrices where the gated unit has
    three) and 16 experts of half the size of which a token uses two (the dense layer's FLOPs); a gate matrix of
    width x width on each sub-layer."""
    from airun_b200 import Qwen3Config
    from airun_b200.config import GamanexConfig
    W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
    dense = dict(kind="dense", ff=3 * F // 2)
    moe = dict(kind="moe", expert=dict(ff=F // 2), router=dict(experts=16, top=2))
    mix = dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, q_temp=dict(coef=0.3, every=512))
    layers = [dict(type="attention", mixer=dict(mix), mlp=dense), dict(type="attention", mixer=dict(mix, kv_from=0), mlp=moe),
              dict(type="attention", mixer=dict(mix), mlp=dense), dict(type="attention", mixer=dict(mix, kv_from=2), mlp=moe),
              dict(type="attention", mixer=dict(mix), mlp=dense), dict(type="attention", mixer=dict(mix), mlp=moe)]
    gam = GamanexConfig.from_dict(dict(architecture="Gamanex", vocab=VEDIZEN_VOCAB, width=W, norm=dict(eps=1e-5),
                                       logit_scale=0.5, layers=layers))
    return gam, vedizen_pair(size)[1]


def workload_gamanex(a) -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 and 64 at a context of 1,024) of the Gamanex design and of
    the Qwen3 decoder at equal size, through the step function and its CUDA graphs, and how long each kind of kernel
    runs inside the prefill step and the batch-64 decode step (CUDA events around every call of the kind, the step
    launched kernel by kernel), with the fraction of the measured peak its bytes or FLOPs over that time come to.  One
    JSON line per size."""
    import torch
    from airun_b200 import Engine, EngineOptions, StepEntry
    from airun_b200.kernels import fast, ops
    pk = peaks()
    T, ctx_len, steps = 2048, 1024, max(8, min(a.steps, 32))
    for name in (a.sizes.split(",") if a.sizes else list(VEDIZEN_SIZES)):
        size = VEDIZEN_SIZES[name]
        W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
        line = {"workload": "gamanex", "size": size, "layer_runs": 6, "vocab": VEDIZEN_VOCAB, "dtype": "bf16",
                "data": "synthetic, random weights", "prompt": T, "decode_context": ctx_len, "peaks": pk["source"], "models": {}}
        for model, cfg in zip(("gamanex", "qwen3"), gamanex_pair(size)):
            eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
                dtype="bfloat16", page_size=16, cache_tokens=64 * (ctx_len + 4 * steps + 64) + 4096, max_batch_tokens=T,
                max_requests=64, max_context=max(T, ctx_len + 4 * steps + 64)))
            tri = lambda t: t * (t + 1) / 2                                   # keys all tokens of a t-token prompt see together
            # kind -> (module, function, work at t tokens of one prompt, work at a batch of b single tokens, bound)
            if model == "gamanex":
                Fd, Fe, E, top = 3 * F // 2, F // 2, 16, 2
                kinds = {
                    "two norms in one pass (rms) + add": (ops, "rmsnorm_pair", lambda t: 6 * t * W * 16.0, lambda b: 6 * b * W * 16.0, "hbm"),
                    "q/k norm, temperature, cache write": (ops, "qk_rownorm_store", lambda t: t * (4 * (H + 2 * G) + 2 * H) * 128 * 6.0,
                                                           lambda b: b * (4 * (H + 2 * G) + 2 * H) * 128 * 6.0, "hbm"),
                    "attention without softmax": (fast, "sigmoid_attention_bf16", lambda t: 6 * H * 4.0 * 128 * tri(t),
                                                  lambda b: 6 * b * ctx_len * G * 256 * 2.0, "mixed"),
                    "gates, scales and sum of the sub-layers": (ops, "gated_sum", lambda t: 6 * t * W * 20.0, lambda b: 6 * b * W * 20.0, "hbm"),
                    "up product + relu squared (dense)": (fast, "linear_act_bf16", lambda t: 3 * 2.0 * t * W * Fd, lambda b: 3 * W * Fd * 2.0, "tensor"),
                    "expert products (gate/up + unit, down)": (fast, "grouped_linear_bf16", lambda t: 3 * t * top * 6.0 * W * Fe,
                                                               lambda b: 3 * min(E, b * top) * 3 * W * Fe * 2.0, "tensor"),
                    "router": (ops, "moe_route", lambda t: 3 * t * (E + 3 * top) * 4.0, lambda b: 3 * b * (E + 3 * top) * 4.0, "hbm"),
                    "rows to experts and back": (ops, "moe_scatter", lambda t: 3 * t * (W * 2 + top * W * 2.0), lambda b: 3 * b * (W * 2 + top * W * 2.0), "hbm"),
                    "sum of a token's experts": (ops, "moe_combine", lambda t: 3 * t * (top + 1) * W * 4.0, lambda b: 3 * b * (top + 1) * W * 4.0, "hbm"),
                }
            else:
                kinds = {
                    "norm (rms)": (ops, "rmsnorm", lambda t: 13 * t * W * 14.0, lambda b: 13 * b * W * 14.0, "hbm"),
                    "q/k norm + rotary + cache write": (ops, "qkv_post", lambda t: 6 * t * (H + 2 * G) * 128 * 6.0,
                                                        lambda b: 6 * b * (H + 2 * G) * 128 * 6.0, "hbm"),
                    "attention": (fast, "attention_bf16", lambda t: 6 * H * 4.0 * 128 * tri(t), lambda b: 6 * b * ctx_len * G * 256 * 2.0, "mixed"),
                    "gate/up product + gated unit": (fast, "linear_swiglu_bf16", lambda t: 6 * 2.0 * t * W * 2 * F, lambda b: 6 * W * 2 * F * 2.0, "tensor"),
                }
            kinds = {k: v for k, v in kinds.items() if hasattr(v[0], v[1])}
            res = {}
            pre_ms = time_prefill(eng, T, runs=5)
            b64 = time_decode_onward(eng, 64, ctx_len, steps, a.warmup, "v")
            b8 = time_decode_onward(eng, 8, ctx_len, steps, a.warmup, "w")
            res["prefill"] = {"ms": round(pre_ms, 3), "tokens_per_s": round(T / pre_ms * 1e3, 1)}
            res["decode_b8"] = {"ms_per_step": round(b8, 4), "tokens_per_s": round(8 / b8 * 1e3, 1)}
            res["decode_b64"] = {"ms_per_step": round(b64, 4), "tokens_per_s": round(64 / b64 * 1e3, 1)}
            spans = {k: [] for k in kinds}
            real = {k: getattr(v[0], v[1]) for k, v in kinds.items()}

            def timed(kind):
                def call(*x, **kw):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = real[kind](*x, **kw)
                    e1.record()
                    spans[kind].append((e0, e1))
                    return out
                return call

            def step_times(run):
                best = {}
                for _ in range(4):
                    for k in spans:
                        spans[k].clear()
                    run()
                    torch.cuda.synchronize()
                    for k, evs in spans.items():
                        us = sum(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3
                        best[k] = min(best.get(k, us), us)
                return best

            toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
            rids = [f"k{i}" for i in range(64)]
            count = [0]

            def run_prefill():
                count[0] += 1
                eng.manager.add_request(f"kp{count[0]}")
                eng.runner.step([StepEntry(f"kp{count[0]}", toks, (T - 1,))])
                eng.manager.free_request(f"kp{count[0]}")

            def run_decode():
                eng.runner.step([StepEntry(r, [toks[j]], (0,)) for j, r in enumerate(rids)])

            graphs, eng.runner.use_graphs = eng.runner.use_graphs, False
            for k, v in kinds.items():
                setattr(v[0], v[1], timed(k))
            try:
                pre_t = step_times(run_prefill)
                fill_contexts(eng, rids, ctx_len)
                dec_t = step_times(run_decode)
            finally:
                for k, v in kinds.items():
                    setattr(v[0], v[1], real[k])
                eng.runner.use_graphs = graphs
            for r in rids:
                eng.manager.free_request(r)
            res["kernels"] = {}
            for kind, (_, _, work_p, work_d, bound) in kinds.items():
                pre_us, dec_us = max(pre_t[kind], 1e-3), max(dec_t[kind], 1e-3)
                row = {"prefill_us": round(pre_us, 1), "decode_b64_us": round(dec_us, 1)}
                if bound == "hbm":
                    row["prefill_frac_of_hbm"] = round(work_p(T) / pre_us / 1e3 / pk["hbm_gbs"], 4)
                else:
                    row["prefill_frac_of_bf16_peak"] = round(work_p(T) / pre_us * 1e6 / (pk["bf16_tflops"] * 1e12), 4)
                row["decode_b64_frac_of_hbm"] = round(work_d(64) / dec_us / 1e3 / pk["hbm_gbs"], 4)
                res["kernels"][kind] = row
            line["models"][model] = res
            del eng
            torch.cuda.empty_cache()
        print(json.dumps(line), flush=True)
    return 0


# The Tagulix design beside the dense Qwen3 decoder at equal size (--workload tagulix)
def tagulix_pair(size: dict):
    """(Tagulix configuration, Qwen3 configuration) with the same width, head counts (heads of 128), vocabulary and six
    layer runs.  Tagulix: four residual streams; a windowed softmax attention (window 1,024, half of each head rotated)
    and a pair of mixers side by side (causal softmax attention with a distance table, a sink and a query temperature,
    beside a decayed linear attention of half as many heads, 64 x 128) in turn; the third and fifth run use the first
    layer's tensors and the sixth the second's; every layer routes a token to 4 of 16 + 4 router outputs (four groups of
    which two are kept; the last four return their input) with experts of a quarter of the dense feed-forward size,
    without a gate: at most 2 W F multiply-adds where Qwen3 has 3."""
    from airun_b200.config import TagulixConfig
    W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
    moe = dict(kind="moe", expert=dict(ff=F // 4), router=dict(experts=16, top=4, identity=4, scale=1.5, groups=dict(count=4, keep=2)))
    att = dict(type="attention", mixer=dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=0.1, mask=dict(size=1024),
                                            rot=dict(dims=64, base=10000.0)), mlp=moe)
    par = dict(type="parallel", mixer=dict(
        left=dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, bias_max=2048, q_temp=dict(coef=0.3, every=512)),
        right=dict(heads=H // 2, dim=64, vdim=128, decay=[1.0 - 2.0 ** -(3 + i % 6) for i in range(H // 2)]),
        left_scale=1.0, right_scale=1.0), mlp=moe)
    layers = [att, par, dict(att, weights_of=0), par, dict(att, weights_of=0), dict(par, weights_of=1)]
    tag = TagulixConfig.from_dict(dict(architecture="Tagulix", vocab=VEDIZEN_VOCAB, width=W, norm=dict(eps=1e-5), residual_mult=0.6,
                                       streams=4, layers=layers))
    return tag, vedizen_pair(size)[1]


def workload_tagulix(a) -> int:
    """Prefill (one 2,048-token prompt) and decode (batch 8 and 64 at a context of 1,024) of the Tagulix design and of
    the Qwen3 decoder at equal size, through the step function and its CUDA graphs, and how long each kind of kernel
    runs inside the prefill step and the batch-64 decode step (CUDA events around every call of the kind, the step
    launched kernel by kernel), with the fraction of the measured peak its bytes or FLOPs over that time come to.  One
    JSON line per size."""
    import torch
    from airun_b200 import Engine, EngineOptions, StepEntry
    from airun_b200.kernels import fast, ops
    pk = peaks()
    T, ctx_len, steps = 2048, 1024, max(8, min(a.steps, 32))
    for name in (a.sizes.split(",") if a.sizes else list(VEDIZEN_SIZES)):
        size = VEDIZEN_SIZES[name]
        W, F, H, G = size["width"], size["ff"], size["heads"], size["kv_heads"]
        line = {"workload": "tagulix", "size": size, "layer_runs": 6, "vocab": VEDIZEN_VOCAB, "dtype": "bf16",
                "data": "synthetic, random weights", "prompt": T, "decode_context": ctx_len, "peaks": pk["source"], "models": {}}
        for model, cfg in zip(("tagulix", "qwen3"), tagulix_pair(size)):
            eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
                dtype="bfloat16", page_size=16, cache_tokens=64 * (ctx_len + 4 * steps + 64) + 4096, max_batch_tokens=T,
                max_requests=64, max_context=max(T, ctx_len + 4 * steps + 64)))
            tri = lambda t: t * (t + 1) / 2                                   # keys all tokens of a t-token prompt see together
            win = lambda t: tri(min(t, 1024)) + max(0, t - 1024) * 1024.0     # the same under a window of 1,024
            # kind -> (module, function, work at t tokens of one prompt, work at a batch of b single tokens, bound)
            if model == "tagulix":
                S, Fe, E, top, Hl = 4, F // 4, 16, 4, H // 2
                lin_in, lin_out = Hl * (64 * 2 + 128 * 2) * 4.0, Hl * 128 * 4.0
                kinds = {
                    "streams: write, read and norm in one pass": (ops, "stream_step", lambda t: 13 * t * W * (8.0 * S + 6), lambda b: 13 * b * W * (8.0 * S + 6), "hbm"),
                    "q/k norm, rotation, temperature, cache write": (ops, "qkv_prepare", lambda t: 6 * t * (H + 2 * G) * 128 * 6.0,
                                                                     lambda b: 6 * b * (H + 2 * G) * 128 * 6.0, "hbm"),
                    "softmax attention (window; table and sink)": (fast, "softmax_attention_bf16", lambda t: 3 * H * 4.0 * 128 * (tri(t) + win(t)),
                                                                   lambda b: 6 * b * ctx_len * G * 256 * 2.0, "mixed"),
                    "decayed linear attention: recurrence": (ops, "decay_recurrent", lambda t: 3 * t * (lin_in - Hl * 128 * 4.0 + lin_out),
                                                             lambda b: 3 * b * (Hl * 64 * 128 * 8.0), "hbm"),
                    "norm over all heads and gate": (ops, "rownorm_gate", lambda t: 3 * t * Hl * 128 * 10.0, lambda b: 3 * b * Hl * 128 * 10.0, "hbm"),
                    # a random router sends top * E / (E + 4) of a token's choices to experts with matrices
                    "expert products (up + GELU, down)": (fast, "grouped_linear_bf16", lambda t: 6 * t * (top * E / (E + 4.0)) * 4.0 * W * Fe,
                                                          lambda b: 6 * min(E, b * top) * 2 * W * Fe * 2.0, "tensor"),
                    "router with groups": (ops, "moe_route_grouped", lambda t: 6 * t * (E + 4 + 3 * top) * 4.0, lambda b: 6 * b * (E + 4 + 3 * top) * 4.0, "hbm"),
                    "rows to experts and back": (ops, "moe_scatter", lambda t: 6 * t * (W * 2 + top * W * 2.0), lambda b: 6 * b * (W * 2 + top * W * 2.0), "hbm"),
                    "sum of a token's experts": (ops, "moe_combine", lambda t: 6 * t * (top + 1) * W * 4.0, lambda b: 6 * b * (top + 1) * W * 4.0, "hbm"),
                }
            else:
                kinds = {
                    "norm (rms)": (ops, "rmsnorm", lambda t: 13 * t * W * 14.0, lambda b: 13 * b * W * 14.0, "hbm"),
                    "q/k norm + rotary + cache write": (ops, "qkv_post", lambda t: 6 * t * (H + 2 * G) * 128 * 6.0,
                                                        lambda b: 6 * b * (H + 2 * G) * 128 * 6.0, "hbm"),
                    "attention": (fast, "attention_bf16", lambda t: 6 * H * 4.0 * 128 * tri(t), lambda b: 6 * b * ctx_len * G * 256 * 2.0, "mixed"),
                    "gate/up product + gated unit": (fast, "linear_swiglu_bf16", lambda t: 6 * 2.0 * t * W * 2 * F, lambda b: 6 * W * 2 * F * 2.0, "tensor"),
                }
            kinds = {k: v for k, v in kinds.items() if hasattr(v[0], v[1])}
            res = {}
            pre_ms = time_prefill(eng, T, runs=5)
            b64 = time_decode_onward(eng, 64, ctx_len, steps, a.warmup, "v")
            b8 = time_decode_onward(eng, 8, ctx_len, steps, a.warmup, "w")
            res["prefill"] = {"ms": round(pre_ms, 3), "tokens_per_s": round(T / pre_ms * 1e3, 1)}
            res["decode_b8"] = {"ms_per_step": round(b8, 4), "tokens_per_s": round(8 / b8 * 1e3, 1)}
            res["decode_b64"] = {"ms_per_step": round(b64, 4), "tokens_per_s": round(64 / b64 * 1e3, 1)}
            spans = {k: [] for k in kinds}
            real = {k: getattr(v[0], v[1]) for k, v in kinds.items()}

            def timed(kind):
                def call(*x, **kw):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = real[kind](*x, **kw)
                    e1.record()
                    spans[kind].append((e0, e1))
                    return out
                return call

            def step_times(run):
                best = {}
                for _ in range(4):
                    for k in spans:
                        spans[k].clear()
                    run()
                    torch.cuda.synchronize()
                    for k, evs in spans.items():
                        us = sum(e0.elapsed_time(e1) for e0, e1 in evs) * 1e3
                        best[k] = min(best.get(k, us), us)
                return best

            toks = torch.randint(0, eng.config.vocab_size, (T,), generator=torch.Generator().manual_seed(3)).tolist()
            rids = [f"k{i}" for i in range(64)]
            count = [0]

            def run_prefill():
                count[0] += 1
                eng.manager.add_request(f"kp{count[0]}")
                eng.runner.step([StepEntry(f"kp{count[0]}", toks, (T - 1,))])
                eng.manager.free_request(f"kp{count[0]}")

            def run_decode():
                eng.runner.step([StepEntry(r, [toks[j]], (0,)) for j, r in enumerate(rids)])

            graphs, eng.runner.use_graphs = eng.runner.use_graphs, False
            for k, v in kinds.items():
                setattr(v[0], v[1], timed(k))
            try:
                pre_t = step_times(run_prefill)
                fill_contexts(eng, rids, ctx_len)
                dec_t = step_times(run_decode)
            finally:
                for k, v in kinds.items():
                    setattr(v[0], v[1], real[k])
                eng.runner.use_graphs = graphs
            for r in rids:
                eng.manager.free_request(r)
            res["kernels"] = {}
            for kind, (_, _, work_p, work_d, bound) in kinds.items():
                pre_us, dec_us = max(pre_t[kind], 1e-3), max(dec_t[kind], 1e-3)
                row = {"prefill_us": round(pre_us, 1), "decode_b64_us": round(dec_us, 1)}
                if bound == "hbm":
                    row["prefill_frac_of_hbm"] = round(work_p(T) / pre_us / 1e3 / pk["hbm_gbs"], 4)
                else:
                    row["prefill_frac_of_bf16_peak"] = round(work_p(T) / pre_us * 1e6 / (pk["bf16_tflops"] * 1e12), 4)
                row["decode_b64_frac_of_hbm"] = round(work_d(64) / dec_us / 1e3 / pk["hbm_gbs"], 4)
                res["kernels"][kind] = row
            line["models"][model] = res
            del eng
            torch.cuda.empty_cache()
        print(json.dumps(line), flush=True)
    return 0


def reference_arm(a) -> int:
    """The same metric on the reference's own CUDA kernels (compiled unmodified for sm_100), called
    through their C entry points in the order the reference's runtime calls them
    (baseline/reference_kernels.py).  The decode step is captured into a CUDA graph as the reference
    captures its own; no scheduler, sampler or host transfer of the reference runs, so there is no
    end-to-end figure."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_kernels as rk
        if not rk.available():
            raise FileNotFoundError("baseline/_ref/libairun_ref_kernels.so has not been built")
        rk.load()
    except (OSError, ImportError) as e:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (pip: 'not installable', no cargo or rustc in this image) "
                          f"and its CUDA kernels are not built here: {e}"}))
        return 0
    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm here drives one GPU"}))
        return 0
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no GPU is visible to this process"}))
        return 0
    a.warmup = max(a.warmup, 3)
    cfg = dict(QWEN3_8B)
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    L, H, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["vocab_size"]
    nh, nkv, hd, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def mat(r, c):
        return (0.02 * torch.randn(r, c, generator=g, device=dev, dtype=torch.float32)).to(torch.bfloat16)

    def vec(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g, device=dev, dtype=torch.float32)

    W = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": vec(H), "lm_head.weight": mat(V, H)}
    for l in range(L):
        p = f"model.layers.{l}"
        W.update({f"{p}.input_layernorm.weight": vec(H), f"{p}.post_attention_layernorm.weight": vec(H),
                  f"{p}.self_attn.q_proj.weight": mat(nh * hd, H), f"{p}.self_attn.k_proj.weight": mat(nkv * hd, H),
                  f"{p}.self_attn.v_proj.weight": mat(nkv * hd, H), f"{p}.self_attn.o_proj.weight": mat(H, nh * hd),
                  f"{p}.self_attn.q_norm.weight": vec(hd), f"{p}.self_attn.k_norm.weight": vec(hd),
                  f"{p}.mlp.gate_proj.weight": mat(I, H), f"{p}.mlp.up_proj.weight": mat(I, H),
                  f"{p}.mlp.down_proj.weight": mat(H, I)})
    slots = max(64, a.batch) if not a.skip_points else a.batch
    dec = rk.ReferenceDecoder(cfg, W, ctx=a.context, slots=slots, max_batch=512, logit_rows=max(64, a.batch))
    for s_ in range(slots):                          # random keys and values, as in the other arm
        dec.kc[s_].normal_(0.0, 0.5, generator=g)
        dec.vc[s_].normal_(0.0, 0.5, generator=g)
    pk = peaks()
    sampler = ClockSampler()
    sampler.start()

    def time_rows(batch, steps):
        start = a.context - steps - 1
        rows = list(range(batch))
        dec.prepare_rows(rows)
        toks = torch.randint(0, V, (steps + 1, batch), generator=torch.Generator().manual_seed(1)).to(dev, torch.int32)
        pos = torch.zeros(batch, dtype=torch.int32, device=dev)
        graph = None

        def one(i):
            dec.tokens[:batch].copy_(toks[i])
            dec.positions[:batch].copy_(pos)
            pos.add_(1)
            if graph is None:
                dec.launch_rows()
            else:
                graph.replay()

        pos.fill_(start)
        one(0)                                          # loads and configures every kernel
        torch.cuda.synchronize()
        try:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                dec.launch_rows()
            graph = gr
        except Exception as e:                          # the reference falls back the same way (runtime.rs:3096-3103)
            print(f"note: the reference arm's decode runs without a CUDA graph: {e}", file=sys.stderr)
            torch.cuda.synchronize()
        for i in range(a.warmup):
            pos.fill_(start + (i % steps))
            one(i % steps)
        times = []
        for _ in range(repeats_for(steps)):
            pos.fill_(start)
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for i in range(steps):
                one(i)
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1) / steps)
        if not torch.isfinite(dec.logits[:batch]).all():
            raise RuntimeError("the reference arm's decode step gave non-finite logits")
        return statistics.median(times), start + (steps + 1) / 2.0, graph is not None

    esz = 2
    cfgo = QwenShape(cfg)
    with sampler.region("b%d" % a.batch):
        ms, mean_ctx, graphed = time_rows(a.batch, a.steps)
    value = a.batch / (ms / 1e3)
    gbs = decode_bytes(cfgo, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9
    points, detail = {}, {}
    if not a.skip_points:
        for b in (1, 64):
            with sampler.region(f"b{b}"):
                pms, pctx, _ = time_rows(b, max(4, a.steps // 2))
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            detail[f"decode_b{b}"] = {"tok_s": round(b / (pms / 1e3), 2), "ms_per_step": round(pms, 4), "hbm_frac": round(
                decode_bytes(cfgo, L, b, pctx, esz) / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    T = 2048
    ptoks = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(3)).tolist()
    ptimes = []
    with sampler.region("prefill"):
        for i in range(3):
            dec.n_past[0] = 0
            torch.cuda.synchronize()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            dec.forward(0, ptoks)                         # portions of 512 tokens, the reference's default batch
            ev1.record()
            torch.cuda.synchronize()
            ptimes.append(ev0.elapsed_time(ev1))
    pre_ms = statistics.median(ptimes[1:])
    clocks = sampler.stop()
    flops = prefill_flops(cfgo, L, T)
    out = {
        "metric": "Qwen3-8B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tok; % roofline",
        "value": round(value, 2), "unit": "tokens/s", "value_of": f"decode tok/s at batch {a.batch}, context {a.context}",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "repeats": repeats_for(a.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference", "reference_class": REFERENCE_CLASS,
        "config": {"model": "Qwen3-8B shape, random weights", "layers": L, "layers_full": QWEN3_8B["num_hidden_layers"],
                   "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
                   "global_batch": a.batch, "seq_len": a.context, "kv_cache": "float16, contiguous per slot",
                   "activations": "float32", "decode_graph": graphed, "prefill_portion": 512,
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (weights and cache are read once per step)",
                   "peaks": pk["source"]},
        "e2e": None, "gpu_launches": 0,
        "prefill": {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "mean_context": round(mean_ctx, 1)},
        "points": points, "points_detail": detail, "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


class QwenShape:
    """The sizes ``decode_bytes`` and ``prefill_flops`` read, from a config dictionary."""

    def __init__(self, d):
        self.hidden_size, self.intermediate_size, self.vocab_size = d["hidden_size"], d["intermediate_size"], d["vocab_size"]
        self.num_attention_heads, self.head_dim = d["num_attention_heads"], d["head_dim"]
        self.q_dim = d["num_attention_heads"] * d["head_dim"]
        self.kv_dim = d["num_key_value_heads"] * d["head_dim"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="layers to build (default: all 36)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--decode-only", action="store_true", help="time the decode step only (for profiling runs)")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prompt only (for profiling runs)")
    ap.add_argument("--workload", default="decode", choices=("decode", "serve", "long", "ablate", "vedizen", "pogarax", "gamanex", "tagulix"),
                    help="decode: the headline line; serve: 128 requests continuously batched (Qwen3-1.7B shape); "
                         "long: a 32,768-token prompt, then decoding alone and as 16 forks (Qwen3-32B shape); "
                         "ablate: the decode step timed with one kind of kernel left out at a time; "
                         "vedizen: prefill and decode of the Vedizen design beside the Qwen3 decoder at equal size; "
                         "pogarax: the same for the Pogarax design beside the Vedizen design; "
                         "gamanex: the same for the Gamanex design beside the Qwen3 decoder; "
                         "tagulix: the same for the Tagulix design beside the Qwen3 decoder")
    ap.add_argument("--sizes", default="", help="vedizen / pogarax / gamanex / tagulix: widths to run, comma separated (default: 2048,4096)")
    ap.add_argument("--requests", type=int, default=128, help="serve: requests")
    ap.add_argument("--new-tokens", type=int, default=None, help="serve / long: tokens decoded per request")
    ap.add_argument("--budget", type=int, default=512, help="serve: tokens per step")
    ap.add_argument("--prompt", type=int, default=32768, help="long: prompt length")
    ap.add_argument("--forks", type=int, default=15, help="long: forks of the request for the batched decode")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not supported (the engine is single-GPU)")
        return 2
    a.warmup = max(a.warmup, 3)
    if a.workload == "serve":
        a.new_tokens = a.new_tokens or 256
        return workload_serve(a)
    if a.workload == "long":
        a.new_tokens = a.new_tokens or 512
        return workload_long(a)
    if a.workload == "ablate":
        return workload_ablate(a)
    if a.workload == "vedizen":
        return workload_vedizen(a)
    if a.workload == "pogarax":
        return workload_pogarax(a)
    if a.workload == "gamanex":
        return workload_gamanex(a)
    if a.workload == "tagulix":
        return workload_tagulix(a)

    import torch
    from airun_b200 import Engine, EngineOptions, Qwen3Config
    d = dict(QWEN3_8B)
    full_layers = d["num_hidden_layers"]
    if a.layers:
        d["num_hidden_layers"] = a.layers
    cfg = Qwen3Config.from_dict(d)
    L = cfg.num_hidden_layers
    pk = peaks()
    max_batch = a.batch if (a.decode_only or a.skip_points or a.prefill_only) else max(64, a.batch)
    cache_tokens = max_batch * a.context + 4096
    cache_gb = cache_tokens * full_layers * 2 * cfg.num_key_value_heads * cfg.head_dim * (2 if a.dtype == "bfloat16" else 4) / 1e9
    if cache_gb > 140.0:
        print(f"bench.py: a cache of {cache_tokens} tokens ({cache_gb:.0f} GB) does not fit beside the weights; "
              f"lower --batch or --context" + ("" if max_batch == a.batch else " or pass --skip-points"))
        return 2
    eng = Engine.from_config(cfg, seed=0, options=EngineOptions(
        dtype=a.dtype, page_size=16, cache_tokens=cache_tokens, max_batch_tokens=2048,
        max_requests=max_batch, max_context=a.context))
    esz = 2 if a.dtype == "bfloat16" else 4

    if a.prefill_only:
        pre_ms = time_prefill(eng, 2048)
        print(json.dumps({"prefill_only": True, "tokens": 2048, "ms": round(pre_ms, 3),
                          "value": round(2048 / (pre_ms / 1e3), 1), "layers": L}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    with sampler.region(f"b{a.batch}"):
        ms, launches, mean_ctx, reps = time_decode(eng, a.batch, a.context, a.steps, a.warmup, "d", check=True)
    value = a.batch / (ms / 1e3)

    if a.decode_only:
        sampler.stop()
        print(json.dumps({"decode_only": True, "ms_per_step": round(ms, 4), "value": round(value, 2),
                          "layers": L, "batch": a.batch, "context": a.context, "mean_context": round(mean_ctx, 1),
                          "hbm_frac": round(decode_bytes(cfg, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}))
        return 0
    with sampler.region("e2e"):
        e2e_ms, h2d, d2h = time_e2e(eng, a.batch, a.context, a.steps, a.warmup)
        e2e_gap = getattr(time_e2e, "host_gap_ms", 0.0)
        e2e_sampled_ms, _, _ = time_e2e(eng, a.batch, a.context, a.steps, a.warmup, sampled=True)
    points, detail = {}, {}
    if not a.skip_points:
        for b in (1, 64):
            with sampler.region(f"b{b}"):
                pms, _, pctx, _ = time_decode(eng, b, a.context, a.steps, a.warmup, f"b{b}_", check=True)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 2)
            detail[f"decode_b{b}"] = {"tok_s": round(b / (pms / 1e3), 2), "ms_per_step": round(pms, 4), "hbm_frac": round(
                decode_bytes(cfg, L, b, pctx, esz) / (pms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    T = 2048
    with sampler.region("prefill"):
        pre_ms = time_prefill(eng, T)
    clocks = sampler.stop()
    flops = prefill_flops(cfg, L, T)
    pre = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3), "frac": None}
    if a.dtype == "bfloat16":
        pre["frac"] = pre["frac_burst"] = round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
        pre["frac_sustained"] = round(flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    gbs = decode_bytes(cfg, L, a.batch, mean_ctx, esz) / (ms / 1e3) / 1e9
    out = {
        "metric": "Qwen3-8B decode tok/s @ batch 1/8/64; prefill tok/s @ 2048 tok; % roofline",
        "value": round(value, 2), "unit": "tokens/s", "value_of": f"decode tok/s at batch {a.batch}, context {a.context}",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "repeats": len(reps), "ms_per_step_repeats": [round(t, 4) for t in reps],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if a.dtype == "bfloat16" else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "Qwen3-8B shape, random weights", "layers": L, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": a.batch, "seq_len": a.context, "page_size": 16, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights and cache are read once per step)",
                   "peaks": pk["source"]},
        "e2e": {"value": round(a.batch / (e2e_ms / 1e3), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "host_gap_ms_per_step": round(e2e_gap, 4),
                "sampled_with_reference_defaults": {"value": round(a.batch / (e2e_sampled_ms / 1e3), 2),
                                                    "ms_per_step": round(e2e_sampled_ms, 4)}},
        "gpu_launches": launches,
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(gbs / pk["hbm_gbs"], 4), "mean_context": round(mean_ctx, 1)},
        "points": points, "points_detail": detail,
        "checked": "each timed decode step: finite logits, graph replay against a kernel-by-kernel run",
        "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
