#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and prefill) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config configs/qwen3-0.6b.json] [--layers N] [--batch 8] [--context 4096]

Default workload: the layer sizes of Qwen3-0.6B (configs/qwen3-0.6b.json) with random weights
drawn on the device, bfloat16, 8 requests decoding at a context of 4,096 tokens, pages of 16
tokens.  ``--config`` names another configuration of the architecture (configs/qwen3-8b.json,
configs/qwen3-32b.json); ``--layers`` runs fewer layers than it has (``config`` in the output names
both numbers).  One "step" is one decode step: every live request advances by one token (step
function, then the sampling kernel).  One JSON line is printed:

* ``value``: decoded tokens a second over exactly K steps, timed with CUDA events on the
  launching stream, after W warm-up steps, with a synchronize on both sides; ``samples``: the
  smallest, mean and median step time from an event after every step (the reference's
  ``timing_summary``, benchmarks/common.py:44-53);
* ``e2e``: the same through the public ``Engine`` API: every step copies the step's token
  ids and tables from pinned host memory to the device and reads the sampled token ids back;
* ``prefill``: one prompt of 2,048 tokens in one step: tokens a second, milliseconds, and the
  fraction of the tensor-core peak that the step's flops amount to;
* ``roofline``: bytes a decode step has to read (every weight it uses once, and the keys and
  values of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens a second at batch 1 and 64 (same context), and ``gen_b1/8/64``: the
  reference's closed loop (benchmarks/benchmark_decode.py:24-33, tools/run_infurnace_model.py:19-44):
  prompts of 128 tokens prefilled through the engine, then 256 tokens generated greedily through
  ``Engine.step()``, tokens a second over the decode steps; ``points_detail`` gives each point's
  microseconds per step (min / mean / median) and its fraction of the HBM bound;
* ``kernels``: where a decode step's and the prefill's time goes by class of kernel (attention,
  products, LM head, the rest), from an eager pass with CUDA events around every launch
  (launches then do not overlap their neighbours, so the classes add up to more than the
  graph-replayed step: compare shares), with each class's achieved GB/s or TFLOP/s;
* ``clocks``: SM clock and throttle reasons sampled with nvidia-smi during the timed region.

The contexts of the device-timed decode steps are synthetic: the pages of each request are filled
with random keys and values instead of being computed by a prefill, which changes nothing of what
a decode step reads or computes.  Inputs are larger than the L2 cache (weights 1.2 GB and more, keys
and values 3.8 GB and more at the default), so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0          # copy bandwidth of a B200, used when no measured figure is at hand
FALLBACK_BF16_TFLOPS = 1590.0      # library bf16 matrix-product burst of a B200, likewise
PREFILL_TOKENS = 2048
GEN_PROMPT, GEN_TOKENS = 128, 256


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        got_hbm, got_tf = d.get("hbm_gbs"), d.get("bf16_tflops")
        if isinstance(got_hbm, (int, float)) and got_hbm > 0 and isinstance(got_tf, (int, float)) and got_tf > 0:
            hbm, tf, src = float(got_hbm), float(got_tf), "measured"
    except (OSError, ValueError, TypeError, AttributeError):
        pass
    return hbm, tf, src


class ClockSampler:
    """nvidia-smi in the background, every 50 ms, while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def summary(ms):
    """min / mean / median of a list of times in milliseconds."""
    return {"min_ms": min(ms), "mean_ms": statistics.fmean(ms), "median_ms": statistics.median(ms), "n": len(ms)}


def fill_contexts(runner, batch, context, prefix="c"):
    """``batch`` live requests that hold ``context`` tokens of (random) keys and values."""
    cache = runner.cache
    rids = []
    for i in range(batch):
        rid = f"{prefix}{i}"
        cache.add_request(rid)
        cache.allocate(rid, context)
        cache.commit(rid, context)
        rids.append(rid)
    return rids


def randomize_pages(runner, seed=0):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    for grp in runner.cache.kv_groups:
        tensors = [t for t in grp.tensors.values() if t is not None]
        tensors += [x for cid, t in grp.tensors.items() if t is None for x in grp.streams[cid].values()]
        for t in tensors:
            flat = t.view(-1)
            step = 1 << 26
            for s in range(0, flat.numel(), step):
                chunk = flat[s:s + step]
                chunk.copy_(torch.randn(chunk.numel(), generator=g, device="cuda", dtype=torch.float32).mul_(0.5))


def release(runner, rids):
    for rid in rids:
        runner.cache.free_request(rid)


def weight_bytes(plan, esize):
    """Bytes of every tensor a decode step reads once (an untied embedding is only gathered from)."""
    skip = set() if plan.lm_head.tied else {plan.embedding.weight}
    total = 0
    for name, spec in plan.tensors().items():
        if name in skip:
            continue
        n = 1
        for s in spec.shape:
            n *= s
        total += n * esize
    return total


def decode_bytes(plan, runner, contexts, esize):
    """Bytes one decode step must read: each weight it uses once and the live keys and values."""
    return weight_bytes(plan, esize), sum(contexts) * runner.cache.bytes_per_token()


def prefill_flops(plan, tokens):
    """Flops of one prompt of ``tokens`` tokens in one step, from the plan: two per weight element and
    token for every matrix of every layer call, causal attention scores and values (window honoured),
    and the head on the one wanted row."""
    linear = attn = 0
    for call in plan.resolved_schedule():
        layer = plan.layers[call.layer]
        for spec in layer.tensors().values():
            if len(spec.shape) == 2:
                linear += 2 * spec.shape[0] * spec.shape[1] * tokens
        mixer = getattr(layer, "mixer", None)
        heads, hd = getattr(mixer, "num_heads", None), getattr(mixer, "head_dim", None)
        if heads and hd:
            w = getattr(mixer, "window", None)
            pairs = tokens * (tokens + 1) // 2 if not w or w >= tokens else w * (w + 1) // 2 + (tokens - w) * w
            attn += 4 * heads * hd * pairs
    head = 2 * plan.hidden_size * plan.vocab_size
    return linear + attn + head


def hold_the_device(ms=12.0):
    """Keep the device busy for about ``ms`` so that the launches that follow queue up behind it: the events
    around them then measure the kernels, not the host's time between launches."""
    import torch
    torch.cuda._sleep(int(ms * 1.9e6))


class KernelClassTimer:
    """CUDA events around every launch of the kernel set, by class.  With events between them, launches do
    not overlap their neighbours (no programmatic dependent launch), so times are those of kernels alone
    on a warm device; the caller queues the launches behind ``hold_the_device`` so that the host's pace
    does not show."""
    METHODS = ("embed", "rmsnorm", "linear", "linear_residual_norm", "rope_table", "qk_norm_rope_store",
               "paged_attention", "sample")

    def __init__(self, kernels, vocab):
        self.k, self.vocab = kernels, vocab
        self.records = []          # (class, start event, end event, bytes, flops)
        self.kv_bytes_per_call = 0
        self.attn_flops_per_call = 0
        self._saved = {}

    def __enter__(self):
        import torch
        for name in self.METHODS:
            inner = getattr(self.k, name)
            self._saved[name] = inner

            def wrapped(*a, _inner=inner, _name=name, **kw):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = _inner(*a, **kw)
                e.record()
                self.records.append((*self._classify(_name, a, kw), s, e))
                return out
            setattr(self.k, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, inner in self._saved.items():
            setattr(self.k, name, inner)
        return False

    def _classify(self, name, a, kw):
        if name == "paged_attention":
            return "attention", self.kv_bytes_per_call, self.attn_flops_per_call
        if name in ("linear", "linear_residual_norm"):
            x, w = a[0], a[1]
            cls = "lm_head" if w.shape[0] == self.vocab else "products"
            return cls, w.numel() * w.element_size(), 2 * x.shape[0] * w.numel()
        return "rest", 0, 0

    def report(self, steps):
        import torch
        torch.cuda.synchronize()
        out = {}
        for cls, nbytes, flops, s, e in self.records:
            d = out.setdefault(cls, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
            d["ms"] += s.elapsed_time(e)
            d["bytes"] += nbytes
            d["flops"] += flops
            d["launches"] += 1
        total = sum(d["ms"] for d in out.values()) or 1.0
        rep = {}
        for cls, d in out.items():
            r = {"ms_per_step": d["ms"] / steps, "share": d["ms"] / total, "launches_per_step": d["launches"] // steps}
            if d["bytes"]:
                r["gbs"] = d["bytes"] / (d["ms"] / 1000.0) / 1e9
            if d["flops"]:
                r["tflops"] = d["flops"] / (d["ms"] / 1000.0) / 1e12
            rep[cls] = r
        return rep


def time_decode(runner, rids, vocab, steps, warmup, seed=1):
    """Device time of ``steps`` decode steps (ms), each step: step function + sampling kernel; and the
    time of each step from an event recorded after it."""
    import torch
    from infurnace_b200.engine.runner import StepEntry
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (warmup + steps, len(rids)), generator=g).tolist()
    zeros = [0.0] * len(rids)

    def one(k):
        # the step function with the sampling kernel behind it; decode-only steps replay a CUDA graph
        runner.step_and_sample([StepEntry(rid, [ids[k][j]], [0]) for j, rid in enumerate(rids)], zeros, zeros)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    launches0 = runner.rt.kernels.launches
    replays0 = runner.graph_replays
    marks[0].record()
    for k in range(steps):
        one(warmup + k)
        marks[k + 1].record()
    torch.cuda.synchronize()
    launches = runner.rt.kernels.launches - launches0
    replays = runner.graph_replays - replays0
    if replays:          # a replayed step launches what one recorded step launched
        launches += replays * runner.launches_per_graph_step
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    return marks[0].elapsed_time(marks[steps]), launches, per_step


def time_prefill(runner, vocab, reps, warm=2):
    import torch
    from infurnace_b200.engine.runner import StepEntry
    toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(2)).tolist()
    times = []
    for rep in range(warm + reps):
        runner.cache.add_request("p")
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.cache.free_request("p")
        if rep >= warm:
            times.append(s.elapsed_time(e))
    return times


def profile_classes(runner, plan, cfg_sizes, batch, context, vocab, esize):
    """The eager pass: kernel classes of a decode step at (batch, context) and of the 2,048-token prefill."""
    import torch
    from infurnace_b200.engine.runner import StepEntry
    K = runner.rt.kernels
    graphs = runner.use_graphs
    runner.use_graphs = False
    out = {}
    try:
        steps = 3
        rids = fill_contexts(runner, batch, context - steps - 2, prefix="k")
        zeros = [0.0] * batch
        step = lambda: runner.step_and_sample([StepEntry(r, [1], [0]) for r in rids], zeros, zeros)      # noqa: E731
        step(); step()
        with KernelClassTimer(K, vocab) as t:
            t.kv_bytes_per_call = batch * context * cfg_sizes["kv_bytes_per_token_per_layer"]
            for _ in range(steps):
                torch.cuda.synchronize()
                hold_the_device()
                step()
            out["decode"] = t.report(steps)
        release(runner, rids)
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(2)).tolist()
        for rep in range(2):
            runner.cache.add_request("kp")
            if rep == 1:
                with KernelClassTimer(K, vocab) as t:
                    t.attn_flops_per_call = cfg_sizes["attn_flops_per_layer_prefill"]
                    torch.cuda.synchronize()
                    hold_the_device(20.0)
                    runner.step([StepEntry("kp", toks, [PREFILL_TOKENS - 1])])
                    out["prefill"] = t.report(1)
            else:
                runner.step([StepEntry("kp", toks, [PREFILL_TOKENS - 1])])
            runner.cache.free_request("kp")
    finally:
        runner.use_graphs = graphs
    for phase in out.values():
        for cls, r in phase.items():
            for key in list(r):
                if isinstance(r[key], float):
                    r[key] = round(r[key], 4)
    return out


def time_generation(engine, plan, vocab, batch, hbm_peak, esize, seed=5):
    """The reference's closed loop: ``batch`` prompts of 128 tokens prefilled through the engine, then 256
    tokens each generated greedily through ``Engine.step()`` (no end-of-sequence id: every request runs to
    its count).  Timed: the decode steps from the moment every request decodes, host clock around each
    ``step()`` (plan, staging copy, kernels, read-back of the tokens)."""
    import torch
    from infurnace_b200.engine import Request, RequestState, SamplingParams
    prompts = torch.randint(0, vocab, (batch, GEN_PROMPT), generator=torch.Generator().manual_seed(seed)).tolist()
    reqs = [Request(f"g{batch}-{j}", prompts[j], SamplingParams(max_tokens=GEN_TOKENS)) for j in range(batch)]
    for r in reqs:
        engine.add_request(r)
    guard = 0
    while any(r.state is not RequestState.DECODING for r in reqs):
        engine.step()
        guard += 1
        if guard > 1000 or any(r.is_terminal() for r in reqs):
            raise RuntimeError("prefill for the generation measurement did not complete")
    for _ in range(3):
        engine.step()
    torch.cuda.synchronize()
    left = min(r.sampling_params.max_tokens - len(r.output_token_ids) for r in reqs) - 2
    times, tokens = [], 0
    start_ctx = statistics.fmean(r.num_tokens for r in reqs)
    t_all = time.perf_counter()
    for _ in range(left):
        t0 = time.perf_counter()
        tokens += engine.step().num_decode_tokens
        times.append((time.perf_counter() - t0) * 1000.0)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t_all
    end_ctx = statistics.fmean(r.num_tokens for r in reqs)
    while not engine.is_done():
        engine.step()
    w = weight_bytes(plan, esize)
    kv = batch * (start_ctx + end_ctx) / 2 * engine.runner.cache.bytes_per_token()
    bound_us = (w + kv) / (hbm_peak * 1e9) * 1e6
    s = summary(times)
    return {"tokens_per_s": tokens / wall, "steps": left, "us_per_step_min": s["min_ms"] * 1000, "us_per_step_mean": wall / left * 1e6,
            "us_per_step_median": s["median_ms"] * 1000, "bound_us": bound_us, "frac": bound_us / (wall / left * 1e6),
            "mean_context": (start_ctx + end_ctx) / 2}


def time_e2e(engine, vocab, batch, context, steps, warmup):
    """Decode through Engine.step(): scheduler, pinned host staging, H2D copy, kernels, sampling,
    and the read-back of the sampled ids, every step.  The contexts are real here: the prompts
    are prefilled through the same engine first (not timed)."""
    import torch
    from infurnace_b200.engine import Request, RequestState, SamplingParams
    # requests that finish their prompt early decode while the others still prefill: leave room for that
    prefill_steps = -(-batch * context // engine.runner.max_tokens) + 2
    budget = warmup + steps + 2 + prefill_steps
    prompts = torch.randint(0, vocab, (batch, context - budget), generator=torch.Generator().manual_seed(3)).tolist()
    reqs = [Request(f"e{j}", prompts[j], SamplingParams(max_tokens=budget)) for j in range(batch)]
    for r in reqs:
        engine.add_request(r)
    guard = 0
    while any(r.state is not RequestState.DECODING for r in reqs):
        engine.step()
        guard += 1
        if guard > 10000 or any(r.is_terminal() for r in reqs):
            raise RuntimeError("prefill for the end-to-end measurement did not complete")
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    s.record()
    n = 0
    for _ in range(steps):
        n += engine.step().num_decode_tokens
    e.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    for r in reqs:
        engine.cancel(r.request_id)
    while not engine.is_done():
        engine.step()
    run = engine.runner
    h2d = run._small_len * 4 + batch * run.max_pages * 4 * max(1, len(run.cache.kv_groups))
    return {"value": n / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": batch * 4,
            "ms_per_step": wall * 1000 / steps, "device_ms_per_step": s.elapsed_time(e) / steps}


def run_ours(args):
    import dataclasses
    import torch
    from infurnace_b200.engine import Engine, EngineOptions
    from infurnace_b200.engine.runner import StepEntry
    from infurnace_b200.models import read_config

    hbm_peak, tf_peak, peak_src = read_peaks()
    cfg = read_config(args.config)
    layers_full = cfg.num_hidden_layers
    if args.layers and args.layers < layers_full:
        fields = {"num_hidden_layers": args.layers}
        if getattr(cfg, "layer_types", None) is not None:
            fields["layer_types"] = tuple(cfg.layer_types[:args.layers])
        cfg = dataclasses.replace(cfg, **fields)
    layers_run = cfg.num_hidden_layers
    name = os.path.splitext(os.path.basename(args.config))[0]
    batch, steps, warmup, context = args.batch, args.steps, args.warmup, args.context
    page = args.page_size
    big = max(batch, 64) if args.mode == "all" else batch          # the largest batch of the run
    pool_tokens = big * context + PREFILL_TOKENS + 64
    opts = EngineOptions(dtype="bfloat16", page_size=page, num_pages=pool_tokens // page, max_num_seqs=big,
                         max_num_batched_tokens=PREFILL_TOKENS, max_model_len=context)
    engine = Engine.from_random(cfg, 0, opts)
    runner, plan = engine.runner, engine.plan
    vocab, esize = plan.vocab_size, 2
    if args.eager:
        runner.use_graphs = False
    if args.mode == "prefill":
        times = time_prefill(runner, vocab, max(1, steps), warm=1)
        print(json.dumps({"mode": "prefill", "tokens": PREFILL_TOKENS, "steps": max(1, steps),
                          "ms_median": statistics.median(times), "ms_min": min(times)}))
        return 0
    if args.mode == "generate":
        out = {f"gen_b{b}": time_generation(engine, plan, vocab, b, hbm_peak, esize) for b in sorted({1, batch})}
        print(json.dumps({"mode": "generate", **out}))
        return 0
    randomize_pages(runner)
    torch.cuda.synchronize()
    start_ctx = context - warmup - steps

    # ---- decode, device timed
    clocks = ClockSampler()
    rids = fill_contexts(runner, batch, start_ctx)
    clocks.start()
    ms, launches, per_step = time_decode(runner, rids, vocab, steps, warmup)
    clock_report = clocks.stop()
    release(runner, rids)
    ms_per_step = ms / steps
    value = batch * steps / (ms / 1000.0)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "batch": batch, "context": context, "steps": steps, "ms_per_step": ms_per_step,
                          "tokens_per_s": value, "graphs": runner.use_graphs, "launches": launches, "samples": summary(per_step)}))
        return 0
    mean_ctx = context - steps / 2
    w_bytes, kv_bytes = decode_bytes(plan, runner, [mean_ctx] * batch, esize)
    achieved = (w_bytes + kv_bytes) / (ms_per_step / 1000.0) / 1e9

    # ---- decode, end to end through the Engine API (host token ids in and out every step)
    e2e = time_e2e(engine, vocab, batch, context, steps, warmup)

    # ---- prefill of 2,048 tokens in one step
    pre = time_prefill(runner, vocab, 5)
    pre_ms = statistics.median(pre)
    flops = prefill_flops(plan, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1000.0), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms / 1000.0) / (tf_peak * 1e12), "tflops": flops / (pre_ms / 1000.0) / 1e12,
               "peak_tflops": tf_peak, "peak_source": peak_src, "min_ms": min(pre), "mean_ms": statistics.fmean(pre)}

    # ---- other batch sizes at the same context
    points, detail = {}, {}
    for b in (1, 64):
        k = max(8, steps // 2)
        rids = fill_contexts(runner, b, context - warmup - k)
        pms, _, ps = time_decode(runner, rids, vocab, k, warmup)
        release(runner, rids)
        points[f"decode_b{b}"] = b * k / (pms / 1000.0)
        wb, kvb = decode_bytes(plan, runner, [context - k / 2] * b, esize)
        s = summary(ps)
        detail[f"decode_b{b}"] = {"us_per_step_min": s["min_ms"] * 1000, "us_per_step_mean": pms / k * 1000,
                                  "us_per_step_median": s["median_ms"] * 1000,
                                  "frac": (wb + kvb) / (pms / k / 1000.0) / 1e9 / hbm_peak}

    # ---- the closed loop of the reference's own benchmark: 128-token prompts, 256 generated tokens
    for b in (1, 8, 64):
        g = time_generation(engine, plan, vocab, b, hbm_peak, esize)
        points[f"gen_b{b}"] = g.pop("tokens_per_s")
        detail[f"gen_b{b}"] = g

    # ---- where the time goes, by class of kernel
    attn_layers = sum(1 for c in plan.resolved_schedule() if getattr(plan.layers[c.layer], "mixer", None) is not None)
    sizes = {"kv_bytes_per_token_per_layer": runner.cache.bytes_per_token() // max(1, attn_layers),
             "attn_flops_per_layer_prefill": (flops - 2 * plan.hidden_size * vocab
                                              - sum(2 * s.shape[0] * s.shape[1] * PREFILL_TOKENS
                                                    for c in plan.resolved_schedule()
                                                    for s in plan.layers[c.layer].tensors().values() if len(s.shape) == 2))
             // max(1, attn_layers)}
    kernels = profile_classes(runner, plan, sizes, batch, context, vocab, esize)

    def rounded(d):
        return {k: (round(v, 4) if isinstance(v, float) else v) for k, v in d.items()}

    mixer = plan.layers[0].mixer
    ffn = plan.layers[0].ffn
    line = {
        "metric": f"decode tok/s at batch {batch}, context {context} ({name} shape, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"{name} shape, random weights drawn on the device, seed 0", "layers": layers_full,
                   "layers_run": layers_run, "hidden": plan.hidden_size, "heads": mixer.num_heads,
                   "kv_heads": mixer.num_kv_heads, "head_dim": mixer.head_dim, "intermediate": ffn.intermediate_size,
                   "vocab": vocab, "global_batch": batch, "seq_len": context, "page_size": page,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 (weights {w_bytes / 1e9:.1f} GB + KV {kv_bytes / 1e9:.1f} GB)",
                   "context_fill": "random keys/values in pages"},
        "samples": rounded(summary(per_step)),
        "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "bytes_per_step": w_bytes + kv_bytes, "peak_source": peak_src},
        "points": points, "points_detail": {k: rounded(v) for k, v in detail.items()}, "kernels": kernels,
        "clocks": clock_report,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------------------------
# --designs: the post-norm recurrent/attention design (Kafunex) beside Qwen3 at equal sizes
FP32_LANES_PER_SM = 128            # float32 multiply-adds an SM issues per clock


def design_configs(size):
    """(Kafunex config.json mapping, Qwen3 config.json mapping) of about the same width, depth and parameter count.
    Layer pattern of the first: attention, recurrence, recurrence, attention, ..."""
    W, layers, H, G, d, rh, rd, rv, ff, chunk = {
        "s": (1024, 8, 16, 4, 64, 8, 64, 128, 3072, 512),
        "m": (2048, 8, 16, 4, 128, 16, 64, 128, 6144, 1024),
        "l": (4096, 8, 32, 8, 128, 32, 64, 128, 12288, 1024),
    }[size]
    vocab = 32768
    entries, params = [], 0
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff}
        if i % 4 in (0, 3):
            entries.append({"type": "attention", "mixer": {"dim": d, "heads": H, "kv_heads": G, "mask": {"size": chunk},
                                                          "scale": d ** -0.5, "vdim": d}, "mlp": mlp})
            params += W * (3 * H * d + G * d) + 2 * W * ff
        else:
            entries.append({"type": "hgrn2", "mixer": {"dim": rd, "heads": rh, "vdim": rv}, "mlp": mlp})
            params += W * (2 * rh * rd + 2 * rh * rv) + 2 * W * ff
    kaf = {"architecture": "Kafunex", "layers": entries, "norm": {"eps": 1e-5}, "vocab": vocab, "width": W}
    attn = W * (2 * H * d + 2 * G * d)
    inter = max(256, round((params / layers - attn) / (3 * W) / 256) * 256)
    qwen = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": W, "num_hidden_layers": layers, "num_attention_heads": H,
            "num_key_value_heads": G, "head_dim": d, "intermediate_size": inter, "vocab_size": vocab, "rope_theta": 1e6,
            "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 8192}
    return kaf, qwen


def hybrid_config(size):
    """A Lunelorn config.json mapping at the width, depth, head sizes and ACTIVE parameter count of design_configs(size):
    layers parallel (attention + minGRU), retention, wkv, parallel, ...; retention heads of the Kafunex recurrence's
    shape; 8 experts of which 2 run, each a third of the dense feed-forward's width (gate, up and down against up and
    down); a token side input of 32; no loop (the depth stays that of the other designs)."""
    W, layers, H, G, d, rh, rd, rv, ff, _ = {
        "s": (1024, 8, 16, 4, 64, 8, 64, 128, 3072, 512),
        "m": (2048, 8, 16, 4, 128, 16, 64, 128, 6144, 1024),
        "l": (4096, 8, 32, 8, 128, 32, 64, 128, 12288, 1024),
    }[size]
    mlp = {"kind": "moe", "expert": {"ff": ff // 3}, "router": {"experts": 8, "top": 2}}
    entries = []
    for i in range(layers):
        if i % 4 in (0, 3):
            entries.append({"type": "parallel", "mlp": mlp, "mixer": {
                "left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "rot": {"base": 1e6, "dims": d // 2}, "scale": d ** -0.5},
                "right": {"width": W // 2}, "left_scale": 1.0, "right_scale": 1.0}})
        elif i % 4 == 1:
            entries.append({"type": "retention", "mlp": mlp, "mixer": {
                "heads": rh, "dim": rd, "vdim": rv, "decay": [1.0 - 2.0 ** (-5 - 3 * j / max(1, rh - 1)) for j in range(rh)]}})
        else:
            entries.append({"type": "wkv", "mlp": mlp, "mixer": {"heads": W // 64, "dim": 64, "rank": 64}})
    return {"architecture": "Lunelorn", "layers": entries, "norm": {"eps": 1e-6}, "vocab": 32768, "width": W,
            "token_side": {"dim": 32}, "logit_softcap": 30.0}


def latent_config(size):
    """A Filorax config.json mapping at the width, depth, head count and ACTIVE parameter count of hybrid_config(size):
    layers rotated-causal, window + sink + gate, window + ordinary softmax, rotated-causal, ...; heads of the attention's
    size with a latent of twice and a rotated part of a quarter of it; 8 experts in 4 groups of which 2 are kept and 2
    experts run, each a sixth of the dense feed-forward's width, beside a shared expert of a third (together the two
    thirds that run in hybrid_config); four taps, two norm groups."""
    W, layers, H, _, d, _, _, _, ff, window = {
        "s": (1024, 8, 16, 4, 64, 8, 64, 128, 3072, 512),
        "m": (2048, 8, 16, 4, 128, 16, 64, 128, 6144, 1024),
        "l": (4096, 8, 32, 8, 128, 32, 64, 128, 12288, 1024),
    }[size]
    mlp = {"kind": "moe", "expert": {"ff": ff // 6}, "shared": {"ff": ff // 3},
           "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    entries = []
    for i in range(layers):
        mixer = {"heads": H, "dim": d, "vdim": d, "kv_rank": 2 * d, "scale": (d + (d // 4 if i % 4 in (0, 3) else 0)) ** -0.5}
        if i % 4 in (0, 3):
            mixer.update(rot_dim=d // 4, rot={"base": 1e6, "dims": d // 4})
            entries.append({"type": "latent_attention_2", "mixer": mixer, "mlp": mlp})
        else:
            mixer.update(mask={"size": window})
            entries.append({"type": "latent_attention" if i % 4 == 1 else "latent_attention_3", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Filorax", "canon": {"taps": 4}, "layers": entries, "norm": {"eps": 1e-6, "groups": 2},
            "residual_mult": 0.5, "vocab": 32768, "width": W}


def recurrent_config(size):
    """A Golonex config.json mapping at the width, depth, head count and ACTIVE parameter count of hybrid_config(size):
    layers latent attention, latent attention, attention whose values are its keys, real-gated recurrence, and again;
    latent attention with heads of the attention's size, a latent of twice and a rotated part of a quarter of it, queries
    through a latent of half the width, a window, sinks and a gate per head; attention rotated on half of each head with
    stretched frequencies under the same window; a recurrence as wide as the model in blocks of 128 channels with four
    taps; 8 experts of which 2 run, each a sixth of the dense feed-forward's width, beside a shared expert of a third; a
    token side input of 32 and a soft cap."""
    W, layers, H, G, d, _, _, _, ff, window = {
        "s": (1024, 8, 16, 4, 64, 8, 64, 128, 3072, 512),
        "m": (2048, 8, 16, 4, 128, 16, 64, 128, 6144, 1024),
        "l": (4096, 8, 32, 8, 128, 32, 64, 128, 12288, 1024),
    }[size]
    mlp = {"kind": "moe", "expert": {"ff": ff // 6}, "shared": {"ff": ff // 3}, "router": {"experts": 8, "top": 2}}
    entries = []
    for i in range(layers):
        if i % 4 in (0, 1):
            entries.append({"type": "latent_attention", "mlp": mlp, "mixer": {
                "heads": H, "dim": d, "rot_dim": d // 4, "vdim": d, "kv_rank": 2 * d, "q_rank": W // 2, "scale": (d + d // 4) ** -0.5,
                "rot": {"base": 1e6, "dims": d // 4}, "mask": {"size": window}}})
        elif i % 4 == 2:
            entries.append({"type": "attention", "mlp": mlp, "mixer": {
                "heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": window},
                "rot": {"base": 1e6, "dims": d // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}})
        else:
            entries.append({"type": "rglru", "mlp": mlp, "mixer": {"width": W, "blocks": W // 128, "conv": 4}})
    return {"architecture": "Golonex", "layers": entries, "norm": {"eps": 1e-6}, "vocab": 32768, "width": W,
            "token_side": {"dim": 32}, "logit_softcap": 30.0}


def window_pairs(window, positions):
    """Sum over query positions of the keys each sees under a sliding window."""
    return sum(min(p + 1, window) for p in positions)


def attention_shape(conf):
    """(key/value heads, head size, chunk or None) of a design's attention layers, from its config.json mapping."""
    if "layers" not in conf:
        return conf["num_key_value_heads"], conf["head_dim"], None
    if conf.get("architecture") == "Golonex":             # a window, not a chunk: the caller counts its pairs
        for layer in conf["layers"]:
            if layer["type"] == "attention":
                return layer["mixer"]["kv_heads"], layer["mixer"]["dim"], None
    for layer in conf["layers"]:
        m = layer["mixer"]
        if layer["type"] == "attention":
            return m["kv_heads"], m["dim"], (m.get("mask") or {}).get("size")
        if layer["type"] == "parallel":
            return m["left"]["kv_heads"], m["left"]["dim"], None
        if layer["type"].startswith("latent_attention"):
            return 1, m["kv_rank"] // 2, None              # a latent of kv_rank entries stands for a key and a value
    return 1, 1, None


class DesignTimer(KernelClassTimer):
    """Events around every launch of either design's kernels, with what each launch has to do at the least: tensor-core
    flops, float32 flops on the ordinary pipes, and bytes of device memory.  ``pairs``: (query, visible key) pairs of
    one attention call of the step, set by the caller (the step's composition decides it)."""
    METHODS = KernelClassTimer.METHODS + ("embed_sinusoid", "residual_postnorm", "cast_rows", "wide_norm_store", "gated_scan",
                                          "attention_talk", "residual_norm_update", "add_rows", "scaled_sum", "token_side_gate",
                                          "softcap", "token_shift_mix", "linear_scan", "gated_unit_scan", "rotary_store",
                                          "rotate_rows", "paged_attention_streams", "moe_route", "moe_plan", "moe_linear",
                                          "moe_combine", "moe_plan_padded", "moe_gather", "moe_linear_grouped", "moe_route_plan",
                                          "group_rmsnorm", "depth_average", "causal_conv", "latent_prepare", "latent_attention",
                                          "gate_heads", "rglru_conv", "rglru_scan", "moe_gather_scaled")

    def __init__(self, kernels, vocab, pairs, key_bytes, positions=(), head_weights=()):
        super().__init__(kernels, vocab)
        self.pairs, self.key_bytes = pairs, key_bytes
        self.positions = list(positions)           # the step's query positions (latent attention: a window per layer)
        self.head_weights = set(head_weights)      # data pointers of per-head matrices that run as grouped products
        self.work = []            # per record: (tensor flops, float32 flops, bytes)

    def _classify(self, name, a, kw):
        tf = ff = by = 0
        cls = "rest"
        if name == "paged_attention":
            cls, tf, by = "attention", 4 * a[1] * a[3] * self.pairs, self.key_bytes
        elif name == "attention_talk":
            H, d = a[1], a[3]
            cls, tf, ff, by = "attention", 4 * H * d * self.pairs, 2 * H * H * self.pairs, self.key_bytes
        elif name == "gated_scan":
            proj, out, heads, dim, vdim = a[0], a[12], a[13], a[14], a[15]
            n = proj.shape[0]
            cls, ff = "recurrence", 6 * n * heads * dim * vdim
            by = proj.numel() * 4 + out.numel() * out.element_size() + 2 * a[11].numel() * heads * dim * vdim * 4
        elif name == "paged_attention_streams":
            cls, tf, by = "attention", 2 * a[1] * (a[3] + a[4]) * self.pairs, self.key_bytes
        elif name == "linear_scan":
            q, heads, dim, vdim, out = a[0], a[4], a[5], a[6], a[11]
            n = q.shape[0]
            cls, ff = "recurrence", 6 * n * heads * dim * vdim
            by = n * heads * (3 * dim + 2 * vdim) * 4 + out.numel() * out.element_size() + 2 * a[10].numel() * heads * dim * vdim * 4
        elif name == "gated_unit_scan":
            proj, out = a[0], a[7]
            cls, ff, by = "recurrence", 10 * out.numel(), proj.numel() * 4 + out.numel() * out.element_size()
        elif name == "rglru_scan":
            gates, u, out = a[0], a[5], a[13]
            # the least: the gates' two numbers, u and the gelu branch's input read once, the result written; per element
            # two sigmoids, two exponentials, a root, a tanh and a dozen products and sums
            cls, ff, by = "recurrence", 40 * out.numel(), out.numel() * (4 * 4 + out.element_size())
        elif name == "latent_attention":
            q_lat, lat_pages, rot_pages, window = a[0], a[2], a[3], a[11]
            H, _, R = q_lat.shape
            r = rot_pages.shape[3] if rot_pages is not None else 0
            seen = [min(p + 1, window) if window else p + 1 for p in self.positions]
            # the least: scores and sums over the latent itself (keys and values are never formed); every latent a query of the
            # step sees is read once
            span = max(seen) + len(seen) - 1 if len(set(self.positions)) > 1 else sum(seen)
            cls, tf, by = "attention", H * (4 * R + 2 * r) * sum(seen), span * (R + r) * lat_pages.element_size()
        elif name in ("moe_linear", "moe_linear_grouped") and a[1].data_ptr() in self.head_weights:
            w, out = a[1], a[5] if name == "moe_linear" else a[3]
            rows = len(self.positions) * w.shape[0]
            cls, tf, by = "head products", 2 * rows * w.shape[1] * w.shape[2], w.numel() * w.element_size()
        elif name == "moe_linear":
            x, w, out = a[0], a[1], a[5]
            experts = min(w.shape[0], out.shape[0])           # experts whose matrices a step has to read at the least
            cls, tf, by = "experts", 2 * out.shape[0] * w.shape[1] * w.shape[2], experts * w.shape[1] * w.shape[2] * w.element_size()
        elif name == "moe_linear_grouped":
            w, tiles, out = a[1], a[2], a[3]
            pairs = out.shape[0] - w.shape[0] * 127          # the rows of the padded list that are pairs, at the least
            cls, tf, by = "experts", 2 * max(pairs, 0) * w.shape[1] * w.shape[2], w.numel() * w.element_size()
        elif name in ("linear", "linear_residual_norm"):
            x, w = a[0], a[1]
            cls = "lm_head" if w.shape[0] == self.vocab else "products"
            tf, by = 2 * x.shape[0] * w.numel(), w.numel() * w.element_size()
        self.work.append((tf, ff, by))
        return cls, by, tf

    def report_bounds(self, steps, tc_peak, fp32_peak, hbm_peak):
        """Per class: ms a step, launches, and the bound: the slowest of (tensor flops / tensor peak, float32 flops /
        float32 peak, bytes / copy bandwidth), summed over the launches, over the time measured."""
        import torch
        torch.cuda.synchronize()
        out = {}
        for (cls, _, _, s, e), (tf, ff, by) in zip(self.records, self.work):
            d = out.setdefault(cls, {"ms": 0.0, "bound_ms": 0.0, "launches": 0, "tensor_flops": 0, "fp32_flops": 0, "bytes": 0})
            d["ms"] += s.elapsed_time(e)
            d["bound_ms"] += 1e3 * max(tf / (tc_peak * 1e12), ff / (fp32_peak * 1e12), by / (hbm_peak * 1e9))
            d["launches"] += 1
            d["tensor_flops"] += tf; d["fp32_flops"] += ff; d["bytes"] += by
        rep = {}
        for cls, d in out.items():
            r = {"ms_per_step": round(d["ms"] / steps, 4), "launches_per_step": d["launches"] // steps}
            if d["bound_ms"]:
                r["of_bound"] = round(d["bound_ms"] / d["ms"], 4)
                which = max((d["tensor_flops"] / tc_peak / 1e3, "tensor"), (d["fp32_flops"] / fp32_peak / 1e3, "fp32"),
                            (d["bytes"] / hbm_peak, "hbm"))[1]
                r["bound"] = which
            rep[cls] = r
        return rep


def visible_pairs(plan_layer_chunk, positions):
    """Sum over query positions of the keys each sees: all earlier ones, or those of its own chunk."""
    if not plan_layer_chunk:
        return sum(p + 1 for p in positions)
    return sum(p % plan_layer_chunk + 1 for p in positions)


def run_designs(args):
    """Prefill (2,048 tokens in one step) and decode (batch 8, each request 2,048 tokens in) of the Kafunex design and
    of Qwen3 at equal width, depth and parameter count, random weights, bfloat16; and where the time of each goes by
    class of kernel, against the least each class has to do.  One JSON line."""
    import torch
    from infurnace_b200.engine import Engine, EngineOptions
    from infurnace_b200.engine.runner import StepEntry
    hbm_peak, tc_peak, peak_src = read_peaks()
    props = torch.cuda.get_device_properties(0)
    clock_ghz = 1.965
    fp32_peak = props.multi_processor_count * FP32_LANES_PER_SM * 2 * clock_ghz / 1e3          # TFLOP/s, nominal
    batch, context = 8, 2040          # the next position stands near the end of a chunk of 512 or 1,024
    sampler = ClockSampler()
    sampler.start()
    results = {}
    for size in args.design_sizes.split(","):
        kaf, qwen = design_configs(size)
        pair = (("lunelorn", hybrid_config(size)), ("kafunex", kaf)) if args.hybrid else (("kafunex", kaf), ("qwen3", qwen))
        if args.latent:
            pair = (("filorax", latent_config(size)), ("lunelorn", hybrid_config(size)))
        if args.recurrent:
            pair = (("golonex", recurrent_config(size)), ("lunelorn", hybrid_config(size)))
        for design, conf in pair:
            pool = batch * (context + 64) + PREFILL_TOKENS + 64
            opts = EngineOptions(dtype="bfloat16", page_size=16, num_pages=pool // 16, max_num_seqs=batch,
                                 max_num_batched_tokens=PREFILL_TOKENS, max_model_len=context + 64)
            eng = Engine.from_random(conf, 1, opts)
            runner, plan = eng.runner, eng.plan
            vocab = plan.vocab_size
            params = sum(math.prod(t.shape) for t in plan.tensors().values())
            G_, d_, chunk = attention_shape(conf)
            ms = time_prefill(runner, vocab, 3)
            pre = statistics.median(ms)
            rids = fill_contexts(runner, batch, context)
            randomize_pages(runner)
            steps = min(args.steps, 48)                     # a request has room for 64 more tokens
            total, launches, per = time_decode(runner, rids, vocab, steps, max(3, args.warmup))
            release(runner, rids)
            dec = statistics.median(per)
            r = {"params_m": round(params / 1e6, 1), "prefill_ms": round(pre, 3), "prefill_tok_s": round(PREFILL_TOKENS / pre * 1e3),
                 "decode_ms": round(dec, 4), "decode_tok_s": round(batch / dec * 1e3), "decode_launches": launches // steps}
            # where the time goes: an eager pass with events around every launch
            K = runner.rt.kernels
            graphs, runner.use_graphs = runner.use_graphs, False
            mixers = [getattr(layer, "mixer", None) for layer in runner.model.layers]
            heads_w = [w.data_ptr() for m in mixers for w in (getattr(m, "w_absorb", None), getattr(m, "w_values", None),
                                                             getattr(m, "w_gates", None)) if w is not None]
            window = next((layer["mixer"]["mask"]["size"] for layer in conf.get("layers", ()) if design == "golonex"
                           and layer["type"] == "attention" and layer["mixer"].get("mask")), None)
            pairs_of = (lambda positions: window_pairs(window, positions)) if window else (lambda positions: visible_pairs(chunk, positions))
            toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(2)).tolist()
            runner.cache.add_request("kp")
            with DesignTimer(K, vocab, pairs_of(range(PREFILL_TOKENS)), 2 * PREFILL_TOKENS * G_ * d_ * 2,
                             positions=range(PREFILL_TOKENS), head_weights=heads_w) as t:
                torch.cuda.synchronize()
                hold_the_device(20.0)
                runner.step([StepEntry("kp", toks, [PREFILL_TOKENS - 1])])
                r["prefill_kernels"] = t.report_bounds(1, tc_peak, fp32_peak, hbm_peak)
            runner.cache.free_request("kp")
            rids = fill_contexts(runner, batch, context, prefix="k")
            zeros = [0.0] * batch
            step = lambda: runner.step_and_sample([StepEntry(x, [1], [0]) for x in rids], zeros, zeros)      # noqa: E731
            step()
            seen = pairs_of([context + 1])          # keys a decoded token sees
            with DesignTimer(K, vocab, batch * seen, batch * seen * G_ * d_ * 2 * 2, positions=[context + 1] * batch,
                             head_weights=heads_w) as t:
                for _ in range(3):
                    torch.cuda.synchronize()
                    hold_the_device()
                    step()
                r["decode_kernels"] = t.report_bounds(3, tc_peak, fp32_peak, hbm_peak)
            release(runner, rids)
            runner.use_graphs = graphs
            results.setdefault(size, {})[design] = r
            del eng, runner
            torch.cuda.empty_cache()
    clocks = sampler.stop()
    print(json.dumps({"metric": "designs_prefill_and_decode", "dtype": "bfloat16", "data": "synthetic (random weights)",
                      "prefill_tokens": PREFILL_TOKENS, "decode": {"batch": batch, "context": context},
                      "peaks": {"hbm_gbs": hbm_peak, "tensor_tflops": tc_peak, "fp32_tflops_nominal": round(fp32_peak, 1),
                                "source": peak_src}, "sizes": results, "clocks": clocks}))
    return 0


def time_design_kernels(args):
    """The talking attention and the gated recurrence alone, on tensors made on the device at the sizes of design_configs:
    a 2,048-token prompt, four such prompts in one step, and a decode step of 8 requests 2,040 tokens in.  Microseconds
    by CUDA events over 20 calls after 3; one JSON line.  (Also the small case for a profiler: --design-sizes s.)"""
    import torch
    from infurnace_b200.kernels import load_cuda_kernels
    K = load_cuda_kernels()
    g = torch.Generator(device="cuda").manual_seed(1)

    def timed(f, reps=20):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            f()
        e.record()
        torch.cuda.synchronize()
        return round(s.elapsed_time(e) / reps * 1e3, 1)

    def step_arrays(lens_new):
        news = [n for _, n in lens_new]
        cu = torch.tensor([0] + [sum(news[:i + 1]) for i in range(len(news))], dtype=torch.int32, device="cuda")
        return cu, torch.tensor([L for L, _ in lens_new], dtype=torch.int32, device="cuda"), sum(news)

    def attention(H, G, d, chunk, lens_new, ps=16):
        cu, seq, n = step_arrays(lens_new)
        R, maxp = len(lens_new), max(-(-L // ps) for L, _ in lens_new)
        pages = torch.randn(R * maxp + 1, 2, G, ps, d, device="cuda", generator=g).bfloat16()
        bt = torch.arange(R * maxp, dtype=torch.int32, device="cuda").view(R, maxp).contiguous()
        q = torch.randn(n, H * d, device="cuda", generator=g).bfloat16()
        talk = (torch.eye(H, device="cuda") + 0.3 * torch.randn(H, H, device="cuda", generator=g)).bfloat16()
        gate = torch.randn(n, H * d, device="cuda", generator=g)
        out = torch.empty_like(q)
        mq, ms = max(x for _, x in lens_new), max(L for L, _ in lens_new)
        return timed(lambda: K.attention_talk(q, H, G, d, pages, bt, cu, seq, out, d ** -0.5, chunk=chunk, slope_exponent=8.0,
                                              talk=talk, gate=gate, max_q_len=mq, max_seq_len=ms))

    def recurrence(heads, dim, vdim, lens_new):
        cu, seq, n = step_arrays(lens_new)
        R, hd, hv = len(lens_new), heads * dim, heads * vdim
        proj = torch.randn(n, 2 * hd + hv, device="cuda", generator=g)
        state = torch.zeros(R, heads, dim, vdim, device="cuda")
        out = torch.empty(n, hv, device="cuda", dtype=torch.bfloat16)
        bias, lower, nw = (torch.rand(k, device="cuda", generator=g).bfloat16() for k in (hd, hd, vdim))
        slots = torch.arange(R, dtype=torch.int32, device="cuda")
        mq = max(x for _, x in lens_new)
        return timed(lambda: K.gated_scan(proj, 0, hd, 2 * hd, bias, lower, nw, 1e-5, state, slots, cu, seq, out, heads, dim, vdim,
                                          max_q_len=mq))

    prompt, four, decode = [(PREFILL_TOKENS, PREFILL_TOKENS)], [(PREFILL_TOKENS, PREFILL_TOKENS)] * 4, [(2041, 1)] * 8
    out = {}
    for size in args.design_sizes.split(","):
        kaf, _ = design_configs(size)
        a = next(e["mixer"] for e in kaf["layers"] if e["type"] == "attention")
        r = next(e["mixer"] for e in kaf["layers"] if e["type"] == "hgrn2")
        att = (a["heads"], a["kv_heads"], a["dim"], a["mask"]["size"])
        rec = (r["heads"], r["dim"], r["vdim"])
        out[size] = {"attention_us": {"prompt": attention(*att, prompt), "four_prompts": attention(*att, four),
                                      "decode_b8": attention(*att, decode)},
                     "recurrence_us": {"prompt": recurrence(*rec, prompt), "decode_b8": recurrence(*rec, decode)}}
    print(json.dumps({"metric": "design_kernels_alone", "unit": "us", "dtype": "bfloat16", "sizes": out,
                      "tensor_core_attention_calls": K.talk_mma_calls, "blocked_recurrence_calls": K.scan_blocked_calls}))
    return 0


def time_hybrid_kernels(args):
    """Lunelorn's own kernels alone, on tensors made on the device at the sizes of hybrid_config: the experts' grouped
    products (2,048 tokens, and a decode step of 8), the matrix-state recurrence in retention's and in time mixing's form
    and the minGRU (a 2,048-token prompt; a decode step of 8 requests).  Microseconds by CUDA events over 20 calls after
    3, with the fraction of the bound (tensor flops over the measured rate, float32 flops over the nominal 74.4 TFLOP/s,
    bytes over the measured copy bandwidth, whichever is slowest); one JSON line.  (Also the small case for a profiler.)"""
    import torch
    from infurnace_b200.kernels import load_cuda_kernels
    K = load_cuda_kernels()
    hbm_peak, tc_peak, peak_src = read_peaks()
    fp32_peak = torch.cuda.get_device_properties(0).multi_processor_count * FP32_LANES_PER_SM * 2 * 1.965 / 1e3
    g = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, generator=g, device="cuda").to(dtype)      # noqa: E731

    def timed(f, reps=20):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            f()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / reps * 1e3

    def entry(us, tf=0.0, ff=0.0, by=0.0):
        bound = max(tf / (tc_peak * 1e12), ff / (fp32_peak * 1e12), by / (hbm_peak * 1e9)) * 1e6
        return {"us": round(us, 1), "of_bound": round(bound / us, 4)}

    def step_arrays(lens_new):
        cu = torch.tensor([0] + list(torch.tensor(lens_new).cumsum(0)), dtype=torch.int32, device="cuda")
        return cu, torch.tensor([n + 5 for n in lens_new], dtype=torch.int32, device="cuda"), \
            torch.arange(len(lens_new), dtype=torch.int32, device="cuda")

    out = {}
    for size in args.design_sizes.split(","):
        conf = hybrid_config(size)
        W = conf["width"]
        ret = next(l["mixer"] for l in conf["layers"] if l["type"] == "retention")
        mix = next(l["mixer"] for l in conf["layers"] if l["type"] == "wkv")
        unit = next(l["mixer"]["right"]["width"] for l in conf["layers"] if l["type"] == "parallel")
        mlp = conf["layers"][0]["mlp"]
        E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
        r = {}
        w1, w2 = rnd(E, 2 * ff, W, dtype=torch.bfloat16) / 32, rnd(E, W, ff, dtype=torch.bfloat16) / 32
        for label, n in (("prompt_2048", 2048), ("decode_8", 8)):
            pairs = n * top
            h, logits = rnd(n, W, dtype=torch.bfloat16), rnd(n, E)
            ids, gates = torch.zeros(n, top, dtype=torch.int32, device="cuda"), torch.zeros(n, top, device="cuda")
            off, perm, pos = (torch.zeros(E + 1, dtype=torch.int32, device="cuda"), torch.zeros(pairs, dtype=torch.int32, device="cuda"),
                              torch.zeros(pairs, dtype=torch.int32, device="cuda"))
            act, y = torch.zeros(pairs, ff, dtype=torch.bfloat16, device="cuda"), torch.zeros(pairs, W, device="cuda")
            delta = torch.zeros(n, W, device="cuda")
            used = min(E, pairs)
            r["experts_" + label] = {
                "route_and_list": entry(timed(lambda: (K.moe_route(logits, top, ids, gates), K.moe_plan(ids, E, off, perm, pos)))),
                "gate_up": entry(timed(lambda: K.moe_linear(h, w1, off, perm, top, act, epilogue="silu_gate")),
                                 tf=2.0 * pairs * 2 * ff * W, by=used * 2 * ff * W * 2),
                "down": entry(timed(lambda: K.moe_linear(act, w2, off, None, 1, y)), tf=2.0 * pairs * ff * W, by=used * ff * W * 2),
                "sum": entry(timed(lambda: K.moe_combine(y, pos, gates, delta)), by=pairs * W * 4 + n * W * 4)}
        for form, heads, dim, vdim in (("retention", ret["heads"], ret["dim"], ret["vdim"]), ("time_mixing", mix["heads"], mix["dim"], mix["dim"])):
            hd, hv = heads * dim, heads * vdim
            state = torch.zeros(8, heads, dim, vdim, device="cuda")
            for label, lens in (("prompt_2048", [2048]), ("decode_8", [1] * 8)):
                n = sum(lens)
                cu, seq, slots = step_arrays(lens)
                q, k, v, gate, wraw = rnd(n, hd), rnd(n, hd), rnd(n, hv), rnd(n, hv), rnd(n, hd)
                o = torch.zeros(n, hv, dtype=torch.bfloat16, device="cuda")
                if form == "retention":
                    decay = torch.full((heads,), 0.97, device="cuda")
                    f = lambda: K.linear_scan(q, k, v, None, heads, dim, vdim, state, slots, cu, seq, o, 1e-6, decay=decay,      # noqa: E731
                                              key_scale=dim ** -0.5, gate=gate, max_q_len=max(lens))
                else:
                    w0, u, nw = rnd(hd) - 1.5, rnd(hd) / 2, 1 + rnd(hv) / 5
                    f = lambda: K.linear_scan(q, k, v, wraw, heads, dim, vdim, state, slots, cu, seq, o, 1e-6, w_bias=w0, bonus=u,      # noqa: E731
                                              norm_weight=nw, gate=gate, max_q_len=max(lens))
                r[f"{form}_{label}"] = entry(timed(f), ff=6.0 * n * heads * dim * vdim,
                                             by=n * (3 * hd + 2 * hv) * 4 + n * hv * 2 + 2 * len(lens) * heads * dim * vdim * 4)
                state.zero_()
        ustate, zb, xb = torch.zeros(8, unit, device="cuda"), rnd(unit), rnd(unit)
        for label, lens in (("prompt_2048", [2048]), ("decode_8", [1] * 8)):
            n = sum(lens)
            cu, seq, slots = step_arrays(lens)
            proj, o = rnd(n, 3 * unit), torch.zeros(n, unit, dtype=torch.bfloat16, device="cuda")
            r["gated_unit_" + label] = entry(timed(lambda: K.gated_unit_scan(proj, zb, xb, ustate, slots, cu, seq, o, max_q_len=max(lens))),
                                             ff=10.0 * n * unit, by=n * unit * 14)
        out[size] = r
    K.check_device_errors()
    print(json.dumps({"metric": "hybrid_kernels_alone", "dtype": "bfloat16 operands, float32 recurrences", "peaks": {
        "hbm_gbs": hbm_peak, "tensor_tflops": tc_peak, "fp32_tflops_nominal": round(fp32_peak, 1), "source": peak_src}, "sizes": out}))
    return 0


def time_recurrent_kernels(args):
    """The real-gated recurrence's kernels each alone (its convolution, the block-diagonal gate product, the walk), beside
    the element-wise recurrence of the closest design (minGRU) and the framework's other short convolution (the one in
    front of Filorax's sublayers, bfloat16 in and out) at the same width: a 2,048-token prompt in one step and a
    decode step of 8 requests, CUDA events over 20 repetitions, against the bytes each has to move at the least over the
    measured copy bandwidth; one JSON line.  (Also the small case for a profiler.)"""
    import torch
    from infurnace_b200.kernels import load_cuda_kernels
    K = load_cuda_kernels()
    hbm_peak, tc_peak, peak_src = read_peaks()
    g = torch.Generator(device="cuda").manual_seed(1)
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, generator=g, device="cuda").to(dtype)      # noqa: E731
    flush = torch.empty(160 << 20, dtype=torch.uint8, device="cuda")                # larger than L2

    def timed(f, reps=20):
        for _ in range(3):
            f()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            f()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / reps * 1e3

    def entry(us, tf=0.0, by=0.0):
        bound = max(tf / (tc_peak * 1e12), by / (hbm_peak * 1e9)) * 1e6
        return {"us": round(us, 1), "of_bound": round(bound / us, 4)}

    out = {}
    for size in args.design_sizes.split(","):
        conf = recurrent_config(size)
        m = next(l["mixer"] for l in conf["layers"] if l["type"] == "rglru")
        W, B, taps = m["width"], m["blocks"], m["conv"]
        bs = W // B
        xb, cw, cb = rnd(W), rnd(W, taps), rnd(W)
        ab, ib, yb, lam = rnd(W), rnd(W), rnd(W), rnd(W) - 3
        wg = rnd(B, 2 * bs, 2 * bs, dtype=torch.bfloat16) / 8          # two terms of u meet the matrix repeated along k
        zb, xb2 = rnd(W), rnd(W)
        r = {}
        for label, lens in (("prompt_2048", [2048]), ("decode_8", [1] * 8)):
            n = sum(lens)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
            seq = torch.tensor([x + 5 for x in lens], dtype=torch.int32, device="cuda")
            slots = torch.arange(len(lens), dtype=torch.int32, device="cuda")
            req = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32, device="cuda"), torch.tensor(lens, device="cuda"))
            req = req.to(torch.int32)
            tile = K.MOE_TILE if K.moe_grouped_tc_ok(n * B, torch.bfloat16, wg) else 0
            seg = -(-n // tile) * tile if tile else n
            proj, u = rnd(n, 2 * W), torch.zeros(n, W, device="cuda")
            ub = torch.zeros(B, seg, 2 * bs, dtype=torch.bfloat16, device="cuda")
            off = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
            tiles = torch.zeros(B * seg // tile, dtype=torch.int32, device="cuda") if tile else None
            cstate, state = torch.zeros(8, max(taps - 1, 1), W, device="cuda"), torch.zeros(8, W, device="cuda")
            gates = torch.zeros(B * seg, 2 * bs, device="cuda")
            o = torch.zeros(n, W, dtype=torch.bfloat16, device="cuda")
            r["convolution_" + label] = entry(timed(lambda: K.rglru_conv(proj, W, xb, cw, cb, cstate, slots, cu, seq, req, u, ub, off,
                                                                         tiles, tile)), by=n * W * (4 + 4 + 4))
            if tile:
                f = lambda: K.moe_linear_grouped(ub.view(B * seg, 2 * bs), wg, tiles, gates)      # noqa: E731
            else:
                f = lambda: K.moe_linear(ub.view(B * seg, 2 * bs), wg, off, None, 1, gates)      # noqa: E731
            r["gate_product_" + label] = entry(timed(f), tf=2.0 * n * B * 2 * bs * 2 * bs, by=n * W * (4 + 8) + wg.numel() * 2)
            r["recurrence_" + label] = entry(timed(lambda: K.rglru_scan(gates.view(B, seg, 2 * bs), ab, ib, lam, 8.0, u, proj, 0, yb, state,
                                                                        slots, cu, seq, o, max_q_len=max(lens))), by=n * W * 18)
            h16, cw16, o16 = rnd(n, W, dtype=torch.bfloat16), rnd(W, taps, dtype=torch.bfloat16), torch.zeros(n, W, dtype=torch.bfloat16, device="cuda")
            r["input_convolution_" + label] = entry(timed(lambda: K.causal_conv(h16, cw16, cstate, slots, cu, seq, req, o16)), by=n * W * 4)
            proj3, ustate = rnd(n, 3 * W), torch.zeros(8, W, device="cuda")
            r["gated_unit_" + label] = entry(timed(lambda: K.gated_unit_scan(proj3, zb, xb2, ustate, slots, cu, seq, o, max_q_len=max(lens))),
                                             by=n * W * 14)
        out[size] = r
    K.check_device_errors()
    print(json.dumps({"metric": "recurrent_kernels_alone", "dtype": "bfloat16 operands, float32 recurrences",
                      "config": "L2 flushed between repetitions", "peaks": {"hbm_gbs": hbm_peak, "tensor_tflops": tc_peak, "source": peak_src},
                      "sizes": out}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096, help="tokens each request holds in the timed decode steps")
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "qwen3-0.6b.json"),
                    help="config.json of the model whose sizes are run (random weights)")
    ap.add_argument("--layers", type=int, default=0, help="run only this many layers (0: all the configuration has)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per page of the key/value cache")
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--mode", default="all", choices=("all", "decode", "prefill", "generate"),
                    help="decode / prefill / generate: only that part, on a pool just large enough (for profiling a small case)")
    ap.add_argument("--eager", action="store_true", help="launch every kernel of a decode step instead of replaying a graph")
    ap.add_argument("--designs", action="store_true",
                    help="instead of the default workload: the Kafunex design beside Qwen3 at equal sizes (prefill and decode)")
    ap.add_argument("--hybrid", action="store_true",
                    help="with --designs: the Lunelorn design beside Kafunex (equal width, depth and active parameters)")
    ap.add_argument("--latent", action="store_true",
                    help="with --designs: the Filorax design beside Lunelorn (equal width, depth and active parameters)")
    ap.add_argument("--recurrent", action="store_true",
                    help="with --designs: the Golonex design beside Lunelorn (equal width, depth and active parameters)")
    ap.add_argument("--design-sizes", default="s,m", help="with --designs: which of the sizes s, m, l (commas between)")
    ap.add_argument("--kernels-alone", action="store_true",
                    help="with --designs: only the talking attention and the gated recurrence, each alone (a small case)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference's model and runner import tinygrad, which is not installed and has no wheel "
                          "offline (pip install --no-deps succeeds, import infurnace.executor.tinygrad.model fails)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.designs:
        if args.kernels_alone:
            if args.recurrent:
                return time_recurrent_kernels(args)
            return time_hybrid_kernels(args) if args.hybrid else time_design_kernels(args)
        return run_designs(args)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
