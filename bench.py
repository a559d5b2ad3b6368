#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 while the contexts grow
from 2,048 to 4,096 tokens: the K timed steps are taken in up to four runs of consecutive steps
placed evenly along that growth (the first run starts at 2,048 tokens, the last ends at 4,096), on
the device with CUDA events around the engine's step function (random bfloat16 weights, random
token ids, synthetic cache contents); ``points`` holds the two ends and the same mean at batch 1
and 64.  ``e2e`` is the same through the Python entry point's engine: requests with prompts of
2,048 tokens generate up to 4,096, every step copies its inputs from pinned host memory to the
device and reads the sampled token ids back, and the same runs of steps are timed by the wall
clock.  ``prefill`` times one 2,048-token prompt in one step; ``roofline`` sets the decode steps'
bytes (every weight once, plus the cache of the live requests) against the memory bandwidth.  A
decode step reads about 15 GB, far more than the 126 MB of L2, so consecutive steps cannot serve
each other from cache.

``--impl reference`` runs the unmodified jiamumuzhao/vllm-cpp (built by baseline/build_reference.py
into baseline/_ref) on the same configuration and the same runs of steps, through its own model
interface as its engine drives it: one forward per token and sequence (baseline/ref_driver.cpp).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 32768, "hidden_act": "silu", "initializer_range": 0.02,
}
# further sizes of the same architecture, for --size (layers, hidden, heads, kv heads, intermediate, rms eps)
SIZES = {
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, rms_norm_eps=1e-6),
    "14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=13824, rms_norm_eps=1e-5),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, rms_norm_eps=1e-6),
}
CONTEXT_START = 2048          # the contexts of the decode measurement grow from here ...
CONTEXT = 4096                # ... to here
SLACK = 64                    # room beyond CONTEXT: requests that began a few steps earlier than others pass it
PREFILL_TOKENS = 2048
METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B bf16)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            burst = float(p.get("bf16_tflops"))
            return {"hbm_gbs": float(p.get("hbm_gbs")), "bf16_tflops": burst,
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or burst), "source": "measured"}
        except (ValueError, TypeError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def decode_runs(steps: int):
    """[(context at the run's first step, steps)]: ``steps`` timed decode steps in up to four runs of
    consecutive steps placed evenly along the growth of the contexts from CONTEXT_START to CONTEXT; the
    last run ends with the contexts at CONTEXT."""
    n = 4 if steps >= 8 else 2 if steps >= 2 else 1
    sizes = [steps // n + (1 if i < steps % n else 0) for i in range(n)]
    if n == 1:
        return [(CONTEXT - sizes[0], sizes[0])]
    last = CONTEXT - sizes[-1]
    return [(CONTEXT_START + round(i * (last - CONTEXT_START) / (n - 1)), k) for i, k in enumerate(sizes)]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the measurements run; ``mark`` names the
    stretch of time that follows, so that every sample can be laid to the measurement it fell into."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.marks = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self, name):
        self.marks.append((time.time(), name))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.mark(None)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        by_region, mx, reasons = {}, None, {}
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                stamp = time.mktime(time.strptime(f[0][:19], "%Y/%m/%d %H:%M:%S")) + float("0" + f[0][19:])
                mhz, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            region = None
            for t, name in self.marks:
                if stamp >= t:
                    region = name
            if region is None:
                continue
            by_region.setdefault(region, []).append(mhz)
            for n, v in zip(self.NAMES, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.setdefault(region, set()).add(n)
        decode = [m for r, v in by_region.items() if r != "prefill" for m in v]
        info = {"sm_mhz": statistics.median(decode) if decode else None, "sm_max_mhz": mx,
                "reasons": sorted(set().union(*[v for r, v in reasons.items() if r != "prefill"])) if reasons else [],
                "samples": len(decode)}
        if by_region.get("prefill"):
            info["prefill_sm_mhz"] = statistics.median(by_region["prefill"])
            info["prefill_reasons"] = sorted(reasons.get("prefill", ()))
        return info


def write_timeline(path, batch, runner, cache, rng, vocab):
    """Kernel start and end times of one steady decode step, from the profiler's device-side records.
    Under programmatic dependent launch a kernel starts (its CTAs become resident) long before the
    kernel before it ends, so the column to read is how much later than its predecessor it ENDS."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from vllm_cpp_b200.engine.runner import StepEntry
    ids = [f"t{i}" for i in range(batch)]
    for r in ids:
        cache.add_request(r)
        cache.reserve(r, CONTEXT - 64)
        cache.commit(r, CONTEXT - 64)

    def one():
        runner.step([StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in ids])

    for _ in range(4):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            one()
        torch.cuda.synchronize()
    tmp = path + ".trace.json"
    prof.export_chrome_trace(tmp)
    with open(tmp) as f:
        ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    os.remove(tmp)
    for r in ids:
        cache.free_request(r)
    ev.sort(key=lambda e: e["ts"])
    ev = ev[len(ev) // 2:]                          # the second step
    t0 = ev[0]["ts"]
    rows = sorted(((e["ts"] + e["dur"] - t0, e["ts"] - t0, e["name"]) for e in ev))
    with open(path, "w") as f:
        f.write(f"# one decode step, batch {batch}, contexts {CONTEXT - 60}: end, start (us from the step's first kernel), "
                "end minus previous end, kernel\n")
        prev = 0.0
        for end, start, name in rows:
            f.write(f"{end:9.2f} {start:9.2f} {end - prev:8.2f}  {name[:90]}\n")
            prev = end


def run_mix(cfg, a) -> int:
    """Continuous batching through the engine's own API: requests of mixed lengths arrive at once, prompts
    are read in portions of at most 2,048 tokens a step beside the tokens other requests decode.  Also
    prints where a step's time goes (the engine's per-phase timers)."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.engine.llm_engine import Engine
    n_req, gen, budget = 32, 256, 2048
    rng = np.random.default_rng(3)
    lens = rng.integers(128, 4097, size=n_req)
    pages = int(sum(-(-(int(n) + gen) // 16) for n in lens)) + 64
    ecfg = EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                        num_gpu_blocks=pages, max_num_seqs=n_req, max_model_len=4096 + gen,
                        max_num_batched_tokens=budget, max_tokens_per_step=budget, time_phases=True)
    engine = Engine(ecfg)
    sp = SamplingParams(max_tokens=gen, temperature=0.0, ignore_eos=True)

    def run():
        for n in lens:
            engine.add_request(rng.integers(0, cfg["vocab_size"], size=int(n)).tolist(), sp)
        torch.cuda.synchronize()
        t, steps, out = time.perf_counter(), 0, 0
        phases = {}
        while engine.has_pending_work():
            out += len(engine.step())
            steps += 1
            for k, v in engine.last_stats.phase_ms.items():
                phases[k] = phases.get(k, 0.0) + v
        torch.cuda.synchronize()
        return time.perf_counter() - t, steps, out, phases

    run()                                             # warm-up: sizes workspaces, captures graphs
    dt, steps, out, phases = run()
    prompt = int(lens.sum())
    print(json.dumps({"metric": "continuous batching: 32 requests, prompts 128-4096, 256 generated each, 2048 tokens a step",
                      "value": round(out / dt, 1), "unit": "generated tokens/s", "seconds": round(dt, 3), "steps": steps,
                      "prompt_tokens": prompt, "generated_tokens": out,
                      "all_tokens_per_s": round((prompt + out) / dt, 1), "preemptions": engine.scheduler.num_preemptions,
                      "phase_ms_per_step": {k: round(v / steps, 4) for k, v in sorted(phases.items())},
                      "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"]}}))
    return 0


def model_numbers(cfg):
    h, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = h // nh
    inter, v, layers = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    per_layer = (nh + 2 * nkv) * d * h + nh * d * h + 3 * inter * h
    return {"layer_params": per_layer, "matrix_params": layers * per_layer + v * h,
            "kv_bytes_per_token": layers * 2 * nkv * d * 2, "d": d}


def flat_config(cfg, a, nums, extra):
    out = {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"],
           "layers_of_configuration": SIZES[a.size]["num_hidden_layers"], "hidden": cfg["hidden_size"],
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": nums["d"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": a.batch,
           "seq_len": CONTEXT, "decode_contexts": f"{CONTEXT_START} growing to {CONTEXT}", "kv_block": 16,
           "parallelism": "single GPU"}
    out.update(extra)
    return out


# ------------------------------------------------------------------------------------------- the C++ host
def run_cpp_host(cfg, a) -> int:
    """Decode throughput through the C++ host runtime (vllm::Engine behind include/vllm/vllm.hpp): the same random
    weights, requests with prompts of 2,048 tokens generating up to 4,096, the same runs of timed steps as the
    e2e figure of the Python host, by the wall clock around Engine::step (which returns the sampled ids)."""
    import numpy as np
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    folder = tempfile.mkdtemp(prefix="vcb_cpp_model_")          # config.json alone: the weights come from the seed
    try:
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        batch, lead = a.batch, 16
        pages = batch * ((CONTEXT + SLACK) // 16 + 1) + 16
        t0 = time.time()
        eng = CppEngine(folder, dtype="bfloat16", block_size=16, num_gpu_blocks=pages, max_num_seqs=max(batch, 8),
                        max_model_len=CONTEXT + SLACK, max_num_batched_tokens=PREFILL_TOKENS, max_tokens_per_step=PREFILL_TOKENS,
                        fused_decode_tokens=int(os.environ.get("VCB_FUSED_DECODE_TOKENS", "64")), load_format="random", seed=0)
        load_s = time.time() - t0
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    rng = np.random.default_rng(0)
    prompt_len = CONTEXT_START - lead
    for _ in range(batch):
        eng.add_request(rng.integers(0, cfg["vocab_size"], size=prompt_len).tolist(), max_tokens=CONTEXT + SLACK - prompt_len,
                        temperature=0.0, ignore_eos=True)
    produced = [0] * batch
    def step():
        outs = eng.step()
        for rid, _, _ in outs:
            produced[rid] += 1
        return len(outs)
    while min(produced) == 0 or len(set(produced)) > 1 and max(produced) < 2:      # until every request decodes
        step()
    runs, timed, seconds = decode_runs(max(1, a.steps)), 0, 0.0
    for ctx0, k in runs:
        while prompt_len + min(produced) < ctx0:
            step()
        t = time.perf_counter()
        got = sum(step() for _ in range(k))
        seconds += time.perf_counter() - t
        assert got == batch * k, (got, batch, k)
        timed += k
    print(json.dumps({"host": "cpp", "metric": METRIC, "value": round(batch * timed / seconds, 1), "unit": "tokens/s",
                      "ms_per_step": round(seconds / timed * 1e3, 4), "steps": timed, "batch": batch,
                      "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"],
                                 "decode_contexts": f"{CONTEXT_START} growing to {CONTEXT}", "load_s": round(load_s, 1),
                                 "pool_gb": round(eng.pool_total_bytes / 1e9, 2)}}))
    return 0


# ---------------------------------------------------------------------------------------- kernels one by one
def run_kernels(cfg) -> int:
    """Every kernel of the step alone at the benchmark's layer sizes: microseconds (CUDA events around a CUDA
    graph of several launches on rotating buffers, so that neither the host nor the L2 cache flatters them) and
    what that is in GB/s of the bytes the kernel must move or in TFLOP/s.  One text table."""
    import numpy as np
    import torch
    from vllm_cpp_b200.csrc import ops
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    h, nh, nkv, inter, vocab = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                 "intermediate_size", "vocab_size"))
    d, page, bf = h // nh, 16, torch.bfloat16
    dev = "cuda"
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, fn, n_copies, bytes_=0, flops=0):
        us = ops.time_in_graph(fn, reps=max(4, n_copies))
        rows.append((name, us, bytes_ / us / 1e3 if bytes_ else None, flops / us / 1e6 if flops else None))

    for t in (8, 2048):
        copies = 6 if t == 8 else 3
        ids = torch.randint(0, vocab, (t,), dtype=torch.int32, device=dev)
        table = rnd(vocab, h, scale=0.02)
        res = [torch.zeros(t, h, device=dev) for _ in range(copies)]
        add(f"embedding, {t} tokens", lambda i: ops.embedding(table, ids, res[i % copies]), copies, bytes_=t * h * 6)
        delta, normed = [rnd(t, h) for _ in range(copies)], [torch.empty(t, h, dtype=bf, device=dev) for _ in range(copies)]
        gain = torch.ones(h, device=dev)
        add(f"residual add + RMSNorm, {t} tokens",
            lambda i: ops.add_rmsnorm(res[i % copies], delta[i % copies], gain, normed[i % copies], 1e-6), copies, bytes_=t * h * 12)
        del table
        # bias + rotation + cache write
        width = (nh + 2 * nkv) * d
        qkv, q_out = [rnd(t, width) for _ in range(copies)], torch.empty(t, nh * d, dtype=bf, device=dev)
        cache = torch.zeros(t // page + 2, 2, nkv, page * d, dtype=bf, device=dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        req = torch.zeros(t, dtype=torch.int32, device=dev)
        bt = torch.arange(t // page + 2, dtype=torch.int32, device=dev).view(1, -1)
        denom = torch.from_numpy(np.power(np.float32(1e6), np.arange(d // 2, dtype=np.float32) * 2 / d).astype(np.float32)).to(dev)
        bias = torch.zeros(width, device=dev)
        add(f"q/k/v bias + rotation + cache write, {t} tokens",
            lambda i: ops.rope_cache_write(qkv[i % copies], bias, pos, req, bt, denom, q_out, cache, num_heads=nh, num_kv_heads=nkv,
                                           head_dim=d, rotary_dim=d, pairing=0, page_size=page, write_kv=True),
            copies, bytes_=t * width * 4)
    # SwiGLU on the library's gate-and-up product (prefill)
    t = 2048
    gu, act = [rnd(t, 2 * inter) for _ in range(2)], torch.empty(t, inter, dtype=bf, device=dev)
    add("silu(gate) * up, 2,048 tokens", lambda i: ops.silu_mul(gu[i % 2], act), 2, bytes_=t * inter * 6)
    del gu, act
    # products: the engine's kernel at 8 tokens (plain epilogue; the fused ones are in the decode timeline), the library's at 2,048
    shapes = [("qkv", (nh + 2 * nkv) * d, h), ("output projection", h, nh * d), ("gate and up", 2 * inter, h), ("down", h, inter)]
    for name, n, k in shapes:
        copies = 6 if n * k < 1e8 else 3
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        for w in ws:
            ops.tile_weights(w)
        x8, o8 = rnd(8, k), torch.empty(8, n, dtype=bf, device=dev)
        add(f"product {name} [{n} x {k}], 8 tokens (tcgen05)", lambda i: ops.gemm_bf16_tcgen05(x8, ws[i % copies], o8), copies,
            bytes_=n * k * 2)
        x, o = rnd(2048, k), torch.empty(2048, n, dtype=bf, device=dev)
        add(f"product {name}, 2,048 tokens (cuBLAS)", lambda i: ops._library_mm(x, ws[i % copies], o), copies, flops=2.0 * 2048 * n * k)
        del ws
    head = rnd(vocab, h, scale=0.02)
    ops.tile_weights(head)
    x8, logits = rnd(8, h), torch.empty(8, vocab, device=dev)
    add(f"output product [{vocab} x {h}], 8 rows, float32 logits", lambda i: ops.gemm_bf16_tcgen05(x8, head, logits), 4, bytes_=vocab * h * 2)
    del head
    # attention
    for t in (2048, 8192):
        n_pages = t // page + 2
        cache = rnd(n_pages, 2, nkv, page * d, scale=0.5)
        q, out = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        q_start = torch.tensor([0, t], dtype=torch.int32, device=dev)
        ctx = torch.zeros(1, dtype=torch.int32, device=dev)
        g = nh // nkv
        n_tiles = -(-t * g // ops.TC_ATTENTION_TILE_ROWS)
        order = np.argsort(-np.arange(n_tiles), kind="stable")          # the tiles with the most keys first
        tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
        tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[order].copy()).to(dev)
        add(f"prefill attention, one prompt of {t}", lambda i: ops.attention_prefill_tc(
            q, cache, out, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
            window=0, scale=d ** -0.5), 4, flops=4.0 * nh * d * t * (t + 1) / 2)
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    part = PagedAttention(h, nh, nkv, d, True, False, 0, PartSpec("none"), bf, dev)
    mixed = [128 + round(i * (4352 - 128) / 31) for i in range(32)]
    for batch, contexts, label in ((8, [CONTEXT - 1] * 8, f"contexts of {CONTEXT}"), (64, [CONTEXT - 1] * 64, f"contexts of {CONTEXT}"),
                                   (32, mixed, "contexts of 128 to 4,352")):
        blocks = -(-(max(contexts) + 1) // page)
        cache = rnd(batch * blocks + 1, 2, nkv, page * d, scale=0.5)
        q, out = rnd(batch, nh * d), torch.empty(batch, nh * d, dtype=bf, device=dev)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        ctx = torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, list(contexts), page)
        split_tiles = torch.from_numpy(part.step_arrays()[part._splits_key()](host)).to(dev)
        nsplit = host.shapes[part._splits_key()]
        need = batch * nh * nsplit
        po, pml = torch.empty(need * d, device=dev), torch.empty(need * 2, device=dev)
        tickets = torch.zeros(batch * nkv, dtype=torch.int32, device=dev)
        add(f"decode attention, batch {batch}, {label}", lambda i: ops.attention_decode_mma(
            q, cache, out, q_start, ctx, bt, None, batch, nsplit, po, pml, tickets, num_heads=nh, num_kv_heads=nkv, head_dim=d,
            page_size=page, window=0, scale=d ** -0.5, split_tiles=split_tiles), 4,
            bytes_=sum(c + 1 for c in contexts) * 2 * nkv * d * 2)
        del cache
    logits = rnd(64, vocab, dtype=torch.float32)
    temp, uni, ids = torch.zeros(64, device=dev), torch.zeros(64, device=dev), torch.empty(64, dtype=torch.int32, device=dev)
    add("sampling (greedy), 64 rows", lambda i: ops.sample(logits, temp, uni, ids), 4, bytes_=64 * vocab * 4)
    temp.fill_(0.8)
    add("sampling (temperature), 64 rows", lambda i: ops.sample(logits, temp, uni, ids), 4, bytes_=64 * vocab * 4)
    w = torch.empty(2 * inter, h, dtype=bf, device=dev)
    add("random weights, one gate-and-up matrix", lambda i: ops.random_normal(w, 12345 + i, 0.0, 0.02), 4, bytes_=w.numel() * 2)
    ops.check_status()
    peaks = load_peaks()
    print(f"# kernels alone, Qwen2.5-7B layer sizes, bfloat16; peaks ({peaks['source']}): {peaks['hbm_gbs']:.0f} GB/s, "
          f"{peaks['bf16_tflops']:.0f} TFLOP/s (burst)")
    print(f"{'kernel':<62s} {'us':>9s} {'GB/s':>8s} {'TFLOP/s':>8s} {'of peak':>8s}")
    for name, us, gbs, tf in rows:
        frac = gbs / peaks["hbm_gbs"] if gbs else tf / peaks["bf16_tflops"]
        print(f"{name:<62s} {us:9.1f} {gbs if gbs else float('nan'):8.0f} {tf if tf else float('nan'):8.1f} {frac:8.2f}")
    return 0


# ------------------------------------------------------------------- the Rolesun design beside Qwen2
# Layer sizes that resemble real models' (width, heads, head size, feed-forward width, layers measured).  Rolesun
# with a latent of 128 and a window that holds the whole context; Qwen2 at equal width, heads, head size and
# feed-forward width with one key/value head, the nearest it has to one cached row per token.
ROLESUN_SIZES = {"2k": dict(width=2048, heads=16, dim=128, ff=8192, layers=8),
                 "4k": dict(width=4096, heads=32, dim=128, ff=14336, layers=4)}
ROLESUN_VOCAB, ROLESUN_RANK, ROLESUN_CONTEXT, ROLESUN_PROMPT = 32000, 128, 2048, 2048


def rolesun_configs(size):
    z = ROLESUN_SIZES[size]
    mixer = {"heads": z["heads"], "dim": z["dim"], "vdim": z["dim"], "kv_rank": ROLESUN_RANK, "scale": z["dim"] ** -0.5,
             "mask": {"size": 2 * ROLESUN_CONTEXT}}
    rolesun = {"architecture": "Rolesun", "vocab": ROLESUN_VOCAB, "width": z["width"], "residual_mult": 0.5, "logit_scale": 1.0,
               "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
               "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": {"kind": "dense", "ff": z["ff"]}}
                          for _ in range(z["layers"])]}
    qwen = dict(QWEN25_7B, hidden_size=z["width"], num_hidden_layers=z["layers"], num_attention_heads=z["heads"],
                num_key_value_heads=1, head_dim=z["dim"], intermediate_size=z["ff"], vocab_size=ROLESUN_VOCAB)
    return rolesun, qwen


def run_rolesun(a) -> int:
    """Prefill and decode throughput of the Rolesun design beside Qwen2 at equal layer sizes (random weights, synthetic
    cache contents, device time by CUDA events around the engine's step function), and the design's own kernels alone
    beside the like kernels of Qwen2's layer with their share of the measured peaks.  One JSON line."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.llm_engine import Engine
    from vllm_cpp_b200.engine.runner import StepEntry
    peaks = load_peaks()
    steps, warmup = max(1, a.steps), max(3, a.warmup)
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    sampler.mark("decode")
    out = {"metric": "prefill and decode tok/s of Rolesun beside Qwen2 at equal layer sizes (bf16, random weights)",
           "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic", "sizes": {}, "peaks": peaks}

    def measure(cfg, batches):
        max_batch = max(batches)
        ctx_room = ROLESUN_CONTEXT + steps + warmup + 64
        pages = max_batch * (ctx_room // 16 + 1) + ROLESUN_PROMPT // 16 + 16
        engine = Engine(EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                                     num_gpu_blocks=pages, max_num_seqs=max_batch, max_model_len=ctx_room,
                                     max_num_batched_tokens=ROLESUN_PROMPT, max_tokens_per_step=ROLESUN_PROMPT))
        runner, cache, model = engine.runner, engine.cache, engine.model
        gen = torch.Generator(device="cuda").manual_seed(1)
        for g in cache.paged:
            g.pages.normal_(0.0, 0.5, generator=gen)
        # what a decode step must read: every tensor but the embedding table (its rows are a gather), and the cache
        weight_bytes = sum(t.numel() * t.element_size() for t in model.tensors() if t is not model.embed)
        cache_bytes_per_token = cache.bytes_per_page(model.cache_specs(), 16, model.dtype) // 16
        res = {"weight_gb_per_step": round(weight_bytes / 1e9, 3), "cache_bytes_per_token": cache_bytes_per_token}
        times = []
        for k in range(warmup + 3):
            cache.add_request("p")
            toks = rng.integers(0, ROLESUN_VOCAB, size=ROLESUN_PROMPT).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry("p", toks, [ROLESUN_PROMPT - 1])])
            e1.record()
            torch.cuda.synchronize()
            cache.free_request("p")
            if k >= warmup:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        res["prefill"] = {"tokens": ROLESUN_PROMPT, "ms": round(ms, 3), "tok_s": round(ROLESUN_PROMPT / ms * 1e3)}
        res["decode"] = {}
        for batch in batches:
            temperature, uniform = torch.zeros(batch, device="cuda"), torch.zeros(batch, device="cuda")
            ids_out = torch.empty(batch, dtype=torch.int32, device="cuda")
            toks = rng.integers(0, ROLESUN_VOCAB, size=(steps + warmup, batch))
            ids = [f"d{batch}_{i}" for i in range(batch)]
            for r in ids:
                cache.add_request(r)
                cache.reserve(r, ROLESUN_CONTEXT)
                cache.commit(r, ROLESUN_CONTEXT)

            def one(j):
                logits = runner.step([StepEntry(r, [int(toks[j, i])], [0]) for i, r in enumerate(ids)])
                ops.sample(logits, temperature, uniform, ids_out)

            for j in range(warmup):
                one(j)
            torch.cuda.synchronize()
            before = ops.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for j in range(warmup, warmup + steps):
                one(j)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            bytes_ = weight_bytes + batch * (ROLESUN_CONTEXT + warmup + steps / 2) * cache_bytes_per_token
            res["decode"][str(batch)] = {"ms_per_step": round(ms, 4), "tok_s": round(batch / ms * 1e3),
                                         "of_hbm_peak": round(bytes_ / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3),
                                         "launches_per_step": (ops.launch_count() - before) // steps}
            for r in ids:
                cache.free_request(r)
        ops.check_status()
        del engine, runner, cache, model
        torch.cuda.empty_cache()
        return res

    for size in (a.rolesun.split(",") if a.rolesun != "all" else sorted(ROLESUN_SIZES)):
        rolesun, qwen = rolesun_configs(size)
        out["sizes"][size] = {"layers": ROLESUN_SIZES[size], "rolesun": measure(rolesun, (8, 64)), "qwen2_one_kv_head": measure(qwen, (8, 64))}
    out["kernels"] = rolesun_kernels(ROLESUN_SIZES["4k"], peaks)
    clocks = sampler.stop()
    out["clocks"] = clocks
    big = out["sizes"].get("4k") or next(iter(out["sizes"].values()))
    out.update(value=big["rolesun"]["decode"]["8"]["tok_s"], unit="tokens/s (Rolesun, 4k-wide layers, batch 8)",
               higher_is_better=True, gpu_launches=big["rolesun"]["decode"]["8"]["launches_per_step"] * steps,
               config={"sizes": ROLESUN_SIZES, "latent": ROLESUN_RANK, "context": ROLESUN_CONTEXT, "prompt": ROLESUN_PROMPT,
                       "l2": "a step's weights exceed the 126 MB of L2"})
    print(json.dumps(out))
    return 0


def rolesun_kernels(z, peaks):
    """The design's own kernels alone at one layer size, each beside the like kernel of Qwen2's layer:
    [{kernel, us, GB/s or TFLOP/s, share of the measured peak}, ...] (CUDA graphs on rotating buffers)."""
    import numpy as np
    import torch
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    h, nh, d, r, page, bf, dev = z["width"], z["heads"], z["dim"], ROLESUN_RANK, 16, torch.bfloat16, "cuda"
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, like, fn, copies, bytes_=0, flops=0):
        us = ops.time_in_graph(fn, reps=max(4, copies))
        rate = bytes_ / us / 1e3 if bytes_ else flops / us / 1e6
        rows.append({"kernel": name, "like": like, "us": round(us, 2), ("gb_s" if bytes_ else "tflop_s"): round(rate, 1),
                     "of_peak": round(rate / (peaks["hbm_gbs"] if bytes_ else peaks["bf16_tflops"]), 3)})

    for t in (64, 2048):
        c = 6 if t == 64 else 3
        x = [rnd(t, h, dtype=torch.float32) for _ in range(c)]
        y, g, o1, o2 = ([rnd(t, h) for _ in range(c)] for _ in range(4))
        mu, bias, one, gain = torch.rand(h, device=dev), torch.zeros(h, device=dev), torch.ones(1, device=dev), torch.ones(h, device=dev)
        state = torch.zeros(1, h, device=dev)
        q_start = torch.tensor([0, t], dtype=torch.int32, device=dev)
        req, pos, slots = torch.zeros(t, dtype=torch.int32, device=dev), torch.arange(t, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
        add(f"token shift, {t} tokens", "", lambda i: ops.token_shift(x[i % c], mu, state, o1[i % c], o2[i % c], q_start, req, pos, slots), c, bytes_=t * h * 8)
        add(f"gate + norm + residual, {t} tokens", "", lambda i: ops.gated_norm_residual(y[i % c], g[i % c], bias, one, x[i % c], o1[i % c], 0.5, 1e-6), c,
            bytes_=t * h * 14)
        add(f"Qwen2: residual add + RMSNorm, {t} tokens", "like the two above", lambda i: ops.add_rmsnorm(x[i % c], y[i % c], gain, o1[i % c], 1e-6), c, bytes_=t * h * 12)
        width = nh * d + r + nh * d
        proj = [rnd(t, width) for _ in range(c)]
        n_pages = t // page + 2
        lat = torch.zeros(n_pages, page * r, dtype=bf, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        gr = torch.ones(r, device=dev)
        add(f"latent norm + cache write, {t} tokens", "", lambda i: ops.latent_cache_write(proj[i % c][:, nh * d: nh * d + r], gr, pos, req, bt, lat, page_size=page, eps=1e-6),
            c, bytes_=t * r * 4)
        qw = (nh + 2) * d
        qkv, q_out = [rnd(t, qw) for _ in range(c)], torch.empty(t, nh * d, dtype=bf, device=dev)
        kvc = torch.zeros(n_pages, 2, 1, page * d, dtype=bf, device=dev)
        denom = torch.from_numpy(np.power(np.float32(1e6), np.arange(d // 2, dtype=np.float32) * 2 / d).astype(np.float32)).to(dev)
        qb = torch.zeros(qw, device=dev)
        add(f"Qwen2: q/k/v bias + rotation + cache write, {t} tokens", "like the one above (it also moves q)",
            lambda i: ops.rope_cache_write(qkv[i % c], qb, pos, req, bt, denom, q_out, kvc, num_heads=nh, num_kv_heads=1, head_dim=d, rotary_dim=d,
                                           pairing=0, page_size=page, write_kv=True), c, bytes_=t * qw * 4)
        wk = [rnd(nh, r, d, scale=0.05) for _ in range(6)]
        ql = torch.empty(t, nh * r, dtype=bf, device=dev)
        kind = dict(bytes_=nh * r * d * 2) if t <= ops.HEADWISE_LIBRARY_TOKENS else dict(flops=2.0 * t * nh * r * d)
        add(f"queries into the latent space (per head), {t} tokens", "", lambda i: ops.headwise_linear(proj[i % c][:, : nh * d], wk[i % 6], ql), 6, **kind)
        wv = [rnd(nh, d, r, scale=0.05) for _ in range(6)]
        ol, og = rnd(t, nh * r), torch.empty(t, nh * d, dtype=bf, device=dev)
        add(f"result out of the latent space + output gate (per head), {t} tokens", "",
            lambda i: ops.headwise_linear(ol, wv[i % 6], og, gate=proj[i % c][:, nh * d + r:]), 6, **kind)
        wd = [rnd(nh * d, nh * d, scale=0.02) for _ in range(6)]
        for w in wd:
            ops.tile_weights(w)
        xo, oo = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev)
        if t <= 128:
            add(f"Qwen2: a dense product of the same width [{nh * d} x {nh * d}], {t} tokens (tcgen05)", "like the two above, 32x their weights",
                lambda i: ops.gemm_bf16_tcgen05(xo, wd[i % 6], oo), 6, bytes_=nh * d * nh * d * 2)
        else:
            add(f"Qwen2: a dense product of the same width, {t} tokens (cuBLAS)", "like the two above, 32x their work",
                lambda i: ops._library_mm(xo, wd[i % 6], oo), 6, flops=2.0 * t * nh * d * nh * d)
    # prefill attention: one prompt
    t = 2048
    n_pages = t // page + 2
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
    q_start, ctx = torch.tensor([0, t], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    n_tiles = -(-t * nh // ops.TC_ATTENTION_TILE_ROWS)
    tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
    tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[::-1].copy()).to(dev)
    q, o = rnd(t, nh * r), torch.empty(t, nh * r, dtype=bf, device=dev)
    for planes, name, like in ((1, "attention over latent rows, prompt of 2,048", ""), (2, "Qwen2: attention, one kv head, prompt of 2,048", "like the one above")):
        kv = rnd(n_pages, planes, 1, page * r, scale=0.5)
        add(name, like, lambda i: ops.attention_prefill_tc(q, kv, o, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=1, head_dim=r,
                                                           page_size=page, window=0, scale=d ** -0.5, planes=planes), 4, flops=4.0 * nh * r * t * (t + 1) / 2)
    # decode attention
    part = PagedAttention(h, nh, 1, r, True, False, 0, PartSpec("none"), bf, dev)
    for batch in (8, 64):
        contexts = [ROLESUN_CONTEXT - 1] * batch
        blocks = -(-ROLESUN_CONTEXT // page)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start, ctx = torch.arange(batch + 1, dtype=torch.int32, device=dev), torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, contexts, page)
        split_tiles = torch.from_numpy(part.step_arrays()[part._splits_key()](host)).to(dev)
        nsplit = host.shapes[part._splits_key()]
        need = batch * nh * nsplit
        share = ops.decode_head_groups(nh, 1)
        po, pml, tickets = torch.empty(need * r, device=dev), torch.empty(need * 2, device=dev), torch.zeros(batch * share, dtype=torch.int32, device=dev)
        q, o = rnd(batch, nh * r), torch.empty(batch, nh * r, dtype=bf, device=dev)
        for planes, name, like in ((1, f"attention over latent rows, decode, batch {batch}, contexts of {ROLESUN_CONTEXT}", ""),
                                   (2, f"Qwen2: attention, one kv head, decode, batch {batch}", "like the one above")):
            kv = rnd(batch * blocks + 1, planes, 1, page * r, scale=0.5)
            add(name, like, lambda i: ops.attention_decode_mma(q, kv, o, q_start, ctx, bt, None, batch, nsplit, po, pml, tickets, num_heads=nh, num_kv_heads=share,
                                                               head_dim=r, page_size=page, window=0, scale=d ** -0.5, split_tiles=split_tiles, planes=planes,
                                                               kv_share=share),
                4, bytes_=batch * ROLESUN_CONTEXT * planes * r * 2)
    ops.check_status()
    return rows


# ------------------------------------------------------------------- the Retodra design beside Qwen2
# Layer sizes that resemble real models'.  Retodra: layers of gated linear attention with a dense feed-forward in turn
# with layers of windowed attention (capped scores, bias by distance) beside lightning attention with routed experts.
# Qwen2 at equal width, heads, kv heads, head size, window and dense feed-forward width is the nearest model the
# engine has.
RETODRA_SIZES = {"2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, experts=16, top=2, expert_ff=2048, layers=4),
                 "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, experts=32, top=4, expert_ff=2048, layers=4)}
RETODRA_VOCAB, RETODRA_CONTEXT, RETODRA_PROMPT, RETODRA_WINDOW = 32000, 2048, 2048, 1024


def retodra_configs(size):
    z = RETODRA_SIZES[size]
    w, h = z["width"], z["heads"]
    gla = {"type": "gla", "mixer": {"heads": h, "dim": 64, "vdim": w // h, "tau": 16.0}, "mlp": {"kind": "dense", "ff": z["ff"]}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": h, "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                              "softcap": 30.0, "bias_max": float(RETODRA_WINDOW), "mask": {"size": RETODRA_WINDOW}},
                     "right": {"heads": h, "dim": 64, "vdim": w // h, "decay": [1.0 - 2.0 ** (-5 - 3 * i / h) for i in range(h)]},
                     "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0},
                   "router": {"experts": z["experts"], "identity": 1, "top": z["top"]}}}
    retodra = {"architecture": "Retodra", "vocab": RETODRA_VOCAB, "width": w, "embedding": {"scale": float(w) ** 0.5},
               "norm": {"eps": 1e-6}, "layers": [dict(gla if i % 2 == 0 else par) for i in range(z["layers"])]}
    qwen = dict(QWEN25_7B, hidden_size=w, num_hidden_layers=z["layers"], num_attention_heads=h, num_key_value_heads=z["kv_heads"],
                head_dim=z["dim"], intermediate_size=z["ff"], vocab_size=RETODRA_VOCAB, use_sliding_window=True,
                sliding_window=RETODRA_WINDOW, max_window_layers=0)
    return retodra, qwen


def decode_step_bytes(model, cache, batch, context):
    """Bytes a decode step of ``batch`` requests with ``context`` cached tokens must move: every weight matrix once (of
    routed experts only as many as the step's tokens can reach), the cached rows inside each layer's window, and every
    request's recurrent state in and out."""
    from vllm_cpp_b200.parts.base import PagedKVSpec, StateSpec, flatten_specs
    total = 0
    seen = set()

    def walk(part):
        nonlocal total
        for v in vars(part).values():
            if hasattr(v, "data_ptr") and v.data_ptr() not in seen and v is not model.embed:
                seen.add(v.data_ptr())
                nbytes = v.numel() * v.element_size()
                if v.dim() == 3 and hasattr(part, "top"):                     # stacked experts
                    nbytes = nbytes * min(v.shape[0], batch * part.top) // v.shape[0]
                total += nbytes
            elif hasattr(v, "param_specs"):
                walk(v)
    for blk in model.blocks:
        for part in blk.parts.values():
            walk(part)
    walk(model.final_norm)
    total += model.lm_head.numel() * model.lm_head.element_size()
    el = model.embed.element_size()
    for spec in flatten_specs(model.cache_specs()):
        if isinstance(spec, PagedKVSpec):
            keys = min(context, spec.window) if spec.window else context
            total += batch * keys * spec.planes * spec.num_kv_heads * spec.head_dim * el
        elif isinstance(spec, StateSpec):
            n = 4
            for d in spec.shape:
                n *= d
            total += 2 * batch * n
    return total


def measure_design(cfg, batches, steps, warmup, rng, peaks, vocab, context, prompt):
    """Prefill of one prompt and decode steps of a design's engine on synthetic cache contents: device time by CUDA
    events around the engine's step function (decode steps replay captured graphs, sampling included)."""
    import torch
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.llm_engine import Engine
    from vllm_cpp_b200.engine.runner import StepEntry
    max_batch = max(batches)
    ctx_room = context + steps + warmup + 64
    pages = max_batch * (ctx_room // 16 + 1) + prompt // 16 + 16
    engine = Engine(EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                                 num_gpu_blocks=pages, max_num_seqs=max_batch, max_model_len=ctx_room,
                                 max_num_batched_tokens=prompt, max_tokens_per_step=prompt))
    runner, cache, model = engine.runner, engine.cache, engine.model
    gen = torch.Generator(device="cuda").manual_seed(1)
    for g in cache.paged:
        g.pages.normal_(0.0, 0.5, generator=gen)
    res = {"weight_gb": round(sum(t.numel() * t.element_size() for t in model.tensors() if t is not model.embed) / 1e9, 3)}
    times = []
    for k in range(warmup + 3):
        cache.add_request("p")
        toks = rng.integers(0, vocab, size=prompt).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("p", toks, [prompt - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.free_request("p")
        if k >= warmup:
            times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    res["prefill"] = {"tokens": prompt, "ms": round(ms, 3), "tok_s": round(prompt / ms * 1e3)}
    res["decode"] = {}
    for batch in batches:
        temperature, uniform = torch.zeros(batch, device="cuda"), torch.zeros(batch, device="cuda")
        ids_out = torch.empty(batch, dtype=torch.int32, device="cuda")
        toks = rng.integers(0, vocab, size=(steps + warmup, batch))
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            cache.add_request(r)
            cache.reserve(r, context)
            cache.commit(r, context)

        def one(j):
            logits = runner.step([StepEntry(r, [int(toks[j, i])], [0]) for i, r in enumerate(ids)])
            ops.sample(logits, temperature, uniform, ids_out)

        for j in range(warmup):
            one(j)
        torch.cuda.synchronize()
        before = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for j in range(warmup, warmup + steps):
            one(j)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        bytes_ = decode_step_bytes(model, cache, batch, context + warmup + steps // 2)
        res["decode"][str(batch)] = {"ms_per_step": round(ms, 4), "tok_s": round(batch / ms * 1e3), "gb_per_step": round(bytes_ / 1e9, 3),
                                     "of_hbm_peak": round(bytes_ / (ms * 1e-3) / (peaks["hbm_gbs"] * 1e9), 3),
                                     "launches_per_step": (ops.launch_count() - before) // steps}
        for r in ids:
            cache.free_request(r)
    ops.check_status()
    del engine, runner, cache, model
    torch.cuda.empty_cache()
    return res


def run_retodra(a) -> int:
    """Prefill and decode throughput of the Retodra design beside Qwen2 at equal layer sizes (random weights, synthetic
    cache contents), and the design's own kernels alone beside the like kernels of Qwen2's layer with their share of the
    measured peaks.  One JSON line."""
    import numpy as np
    peaks = load_peaks()
    steps, warmup = max(1, a.steps), max(3, a.warmup)
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    sampler.mark("decode")
    out = {"metric": "prefill and decode tok/s of Retodra beside Qwen2 at equal layer sizes (bf16, random weights)",
           "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic", "sizes": {}, "peaks": peaks}
    sizes = a.retodra.split(",") if a.retodra != "all" else sorted(RETODRA_SIZES)
    for size in sizes:
        retodra, qwen = retodra_configs(size)
        args = (steps, warmup, rng, peaks, RETODRA_VOCAB, RETODRA_CONTEXT, RETODRA_PROMPT)
        out["sizes"][size] = {"layers": RETODRA_SIZES[size], "retodra": measure_design(retodra, (8, 64), *args),
                              "qwen2_windowed": measure_design(qwen, (8, 64), *args)}
    out["kernels"] = retodra_kernels(RETODRA_SIZES[sizes[-1]], peaks)
    out["clocks"] = sampler.stop()
    big = out["sizes"][sizes[-1]]
    out.update(value=big["retodra"]["decode"]["8"]["tok_s"], unit=f"tokens/s (Retodra, {sizes[-1]}-wide layers, batch 8)",
               higher_is_better=True, gpu_launches=big["retodra"]["decode"]["8"]["launches_per_step"] * steps,
               config={"sizes": RETODRA_SIZES, "context": RETODRA_CONTEXT, "prompt": RETODRA_PROMPT, "window": RETODRA_WINDOW,
                       "l2": "a step's weights exceed the 126 MB of L2"})
    print(json.dumps(out))
    return 0


def retodra_kernels(z, peaks):
    """The design's own kernels alone at one layer size, each beside the like kernel of Qwen2's layer:
    [{kernel, like, us, GB/s or TFLOP/s, share of the measured peak}, ...] (CUDA graphs on rotating buffers)."""
    import numpy as np
    import torch
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    h, nh, nkv, d, page, bf, dev = z["width"], z["heads"], z["kv_heads"], z["dim"], 16, torch.bfloat16, "cuda"
    dk, dv, W = 64, h // nh, RETODRA_WINDOW
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, like, fn, copies, bytes_=0, flops=0):
        us = ops.time_in_graph(fn, reps=max(4, copies))
        rate = bytes_ / us / 1e3 if bytes_ else flops / us / 1e6
        rows.append({"kernel": name, "like": like, "us": round(us, 2), ("gb_s" if bytes_ else "tflop_s"): round(rate, 1),
                     "of_peak": round(rate / (peaks["hbm_gbs"] if bytes_ else peaks["bf16_tflops"]), 4)})

    # ---- the recurrence: single tokens (state in and out) and a prompt
    for batch in (8, 64):
        c = 3
        state = [torch.zeros(batch, nh, dk, dv, device=dev) for _ in range(c)]
        q, k, v, pre = rnd(batch, nh * dk), rnd(batch, nh * dk, scale=0.1), rnd(batch, nh * dv), rnd(batch, nh * dk)
        o = torch.empty(batch, nh * dv, device=dev)
        q_start, slots = torch.arange(batch + 1, dtype=torch.int32, device=dev), torch.arange(batch, dtype=torch.int32, device=dev)
        bias = torch.zeros(nh * dk, device=dev)
        add(f"recurrence (decay per channel), decode, batch {batch}", "Qwen2 decode attention below (bytes of the state against bytes of the keys)",
            lambda i: ops.decayed_state_scan(q, k, v, state[i % c], o, q_start, slots, batch, num_heads=nh, decay_pre=pre, decay_bias=bias,
                                             tau=16.0, q_scale=0.125), c, bytes_=batch * nh * dk * dv * 8)
    t = RETODRA_PROMPT
    state = torch.zeros(1, nh, dk, dv, device=dev)
    q, k, v, pre = rnd(t, nh * dk), rnd(t, nh * dk, scale=0.1), rnd(t, nh * dv), rnd(t, nh * dk)
    o = torch.empty(t, nh * dv, device=dev)
    q_start, slots = torch.tensor([0, t], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    bias, lam = torch.zeros(nh * dk, device=dev), torch.full((nh,), 0.98, device=dev)
    starts, per_req = ops.scan_pieces([t])
    count = len(starts) - 1
    pieces = {"start": torch.from_numpy(starts).to(dev), "req": torch.from_numpy(per_req).to(dev),
              "slots": torch.arange(count, dtype=torch.int32, device=dev), "count": count,
              "state": torch.empty(count, nh, dk, dv, device=dev), "qp": torch.empty(t, nh * dk, device=dev),
              "dtot": torch.empty(count, nh * dk, device=dev)}
    add(f"recurrence (decay per channel), prompt of {t}, token by token", "",
        lambda i: ops.decayed_state_scan(q, k, v, state, o, q_start, slots, 1, num_heads=nh, decay_pre=pre, decay_bias=bias, tau=16.0, q_scale=0.125),
        2, flops=4.0 * t * nh * dk * dv)
    add(f"recurrence (decay per channel), prompt of {t}, pieces of {ops.SCAN_PIECE} side by side (three kernels)",
        "Qwen2 prefill attention below (float FMA against tensor cores)",
        lambda i: ops.decayed_state_scan(q, k, v, state, o, q_start, slots, 1, num_heads=nh, decay_pre=pre, decay_bias=bias, tau=16.0, q_scale=0.125,
                                         pieces=pieces), 2, flops=6.0 * t * nh * dk * dv)
    add(f"recurrence (decay per head), prompt of {t}, pieces side by side", "",
        lambda i: ops.decayed_state_scan(q, k, v, state, o, q_start, slots, 1, num_heads=nh, decay_const=lam, silu_inputs=True, pieces=pieces), 2,
        flops=6.0 * t * nh * dk * dv)
    # ---- rows of the residual stream
    for t in (64, 2048):
        c = 6 if t == 64 else 3
        x = [rnd(t, h, dtype=torch.float32) for _ in range(c)]
        y, o1 = ([rnd(t, h) for _ in range(c)] for _ in range(2))
        gain = torch.ones(h, device=dev)
        add(f"post norm + layer scale + addition + next norm, {t} tokens", "", lambda i: ops.norm_residual_norm(y[i % c], gain, x[i % c], 1e-6, next_gain=gain,
                                                                                                             next_out=o1[i % c], next_eps=1e-6), c, bytes_=t * h * 12)
        add(f"Qwen2: residual add + RMSNorm, {t} tokens", "like the one above", lambda i: ops.add_rmsnorm(x[i % c], y[i % c], gain, o1[i % c], 1e-6), c, bytes_=t * h * 12)
        of = [rnd(t, nh * dv, dtype=torch.float32) for _ in range(c)]
        gt, gw = rnd(t, nh * dv), torch.ones(dv, device=dev)
        add(f"norm per head + silu gate, {t} tokens", "like the one above", lambda i: ops.gated_group_norm(of[i % c], gt, gw, o1[i % c][:, : nh * dv], group=dv, eps=1e-6,
                                                                                                        gate_act="silu"), c, bytes_=t * nh * dv * 8)
        width = (nh + 2 * nkv) * d
        proj = [rnd(t, width) for _ in range(c)]
        n_pages = t // page + 2
        kvc = torch.zeros(n_pages, 2 * nkv * page * d, dtype=bf, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        req, pos = torch.zeros(t, dtype=torch.int32, device=dev), torch.arange(t, dtype=torch.int32, device=dev)
        wq, wk, q_out = torch.ones(nh * d, device=dev), torch.ones(nkv * d, device=dev), torch.empty(t, nh * d, dtype=bf, device=dev)
        add(f"q/k norm over the projection + cache write, {t} tokens", "", lambda i: ops.qk_norm_cache_write(
            proj[i % c], 0, nh * d, (nh + nkv) * d, wq, wk, q_out, kvc, pos, req, bt, num_heads=nh, num_kv_heads=nkv, head_dim=d, v_head_dim=d, row=d,
            page_size=page, eps=1e-6, write_kv=True), c, bytes_=t * width * 2 + t * (nh + 2 * nkv) * d * 2)
        denom = torch.from_numpy(np.power(np.float32(1e6), np.arange(d // 2, dtype=np.float32) * 2 / d).astype(np.float32)).to(dev)
        qb, kv4 = torch.zeros(width, device=dev), kvc.view(n_pages, 2, nkv, page * d)
        add(f"Qwen2: q/k/v bias + rotation + cache write, {t} tokens", "like the one above", lambda i: ops.rope_cache_write(
            proj[i % c], qb, pos, req, bt, denom, q_out, kv4, num_heads=nh, num_kv_heads=nkv, head_dim=d, rotary_dim=d, pairing=0, page_size=page,
            write_kv=True), c, bytes_=t * width * 4)
    # ---- attention with shaped scores beside plain scores: a prompt, then single tokens
    t = RETODRA_PROMPT
    n_pages = t // page + 2
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
    q_start, ctx = torch.tensor([0, t], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    G = nh // nkv
    n_tiles = -(-t * G // ops.TC_ATTENTION_TILE_ROWS)
    tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
    tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[::-1].copy()).to(dev)
    q, o = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev)
    kv = rnd(n_pages, 2, nkv, page * d, scale=0.5)
    bias_t = rnd(nh, W, dtype=torch.float32)
    seen = sum(min(i + 1, W) for i in range(t))
    for shaped, name, like in ((True, f"attention, capped and biased scores, window {W}, prompt of {t}", ""),
                               (False, f"Qwen2: attention, window {W}, prompt of {t}", "like the one above")):
        kw = dict(cap=30.0, bias_t=bias_t) if shaped else {}
        add(name, like, lambda i: ops.attention_prefill_tc(q, kv, o, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=nkv, head_dim=d,
                                                           page_size=page, window=W, scale=d ** -0.5, **kw), 4, flops=4.0 * nh * d * seen)
    part = PagedAttention(h, nh, nkv, d, True, False, W, PartSpec("none"), bf, dev)
    for batch in (8, 64):
        contexts = [RETODRA_CONTEXT - 1] * batch
        blocks = -(-RETODRA_CONTEXT // page)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start, ctx = torch.arange(batch + 1, dtype=torch.int32, device=dev), torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, contexts, page)
        split_tiles = torch.from_numpy(part.step_arrays()[part._splits_key()](host)).to(dev)
        nsplit = host.shapes[part._splits_key()]
        need = batch * nh * nsplit
        share = ops.decode_head_groups(nh, nkv)
        po, pml, tickets = torch.empty(need * d, device=dev), torch.empty(need * 2, device=dev), torch.zeros(batch * nkv * share, dtype=torch.int32, device=dev)
        q, o = rnd(batch, nh * d), torch.empty(batch, nh * d, dtype=bf, device=dev)
        kv = rnd(batch * blocks + 1, 2, nkv, page * d, scale=0.5)
        for shaped, name, like in ((True, f"attention, capped and biased scores, decode, batch {batch}, window {W}", ""),
                                   (False, f"Qwen2: attention, decode, batch {batch}, window {W}", "like the one above")):
            kw = dict(cap=30.0, bias_t=bias_t) if shaped else {}
            add(name, like, lambda i: ops.attention_decode_mma(q, kv, o, q_start, ctx, bt, None, batch, nsplit, po, pml, tickets, num_heads=nh,
                                                               num_kv_heads=nkv * share, head_dim=d, page_size=page, window=W, scale=d ** -0.5,
                                                               split_tiles=split_tiles, kv_share=share, **kw), 4, bytes_=batch * W * 2 * nkv * d * 2)
    # ---- routed experts beside a dense gated feed-forward of the width the chosen experts have together
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.mlp import GatedMLP
    from vllm_cpp_b200.parts.moe import RoutedExperts
    E, top, ff = z["experts"], z["top"], z["expert_ff"]
    moe = RoutedExperts(h, ff, E, 1, top, 7.0, bf, dev)
    tensors = {"router": rnd(E + 1, h, dtype=torch.float32, scale=0.05), "correction": torch.zeros(E + 1, device=dev)}
    for e in range(E):
        tensors.update({f"e{e}.gate": rnd(ff, h, scale=0.02), f"e{e}.up": rnd(ff, h, scale=0.02), f"e{e}.down": rnd(h, ff, scale=0.02)})
    moe.load_params(tensors)
    del tensors
    dense = [GatedMLP(h, top * ff, "silu", bf, dev) for _ in range(3)]
    for m in dense:
        m.load_params({"gate_proj.weight": rnd(top * ff, h, scale=0.02), "up_proj.weight": rnd(top * ff, h, scale=0.02),
                       "down_proj.weight": rnd(h, top * ff, scale=0.02)})
        ops.tile_weights(m.w_gate_up, top * ff)
        ops.tile_weights(m.w_down)
    ws = Workspace(dev, 1 << 30)
    for t in (8, 64, 2048):
        x, out = rnd(t, h), torch.empty(t, h, dtype=bf, device=dev)

        def run_moe(i):
            ws.reset()
            moe.forward(x, out, None, ws)

        def run_dense(i):
            ws.reset()
            dense[i % 3].forward(x, out, None, ws)

        reach = min(E, t * top)
        if t <= 128:
            add(f"routed experts ({top} of {E}, six kernels), {t} tokens", "", run_moe, 3, bytes_=reach * 3 * ff * h * 2)
            add(f"Qwen2: gated feed-forward of width {top * ff}, {t} tokens", "like the one above", run_dense, 3, bytes_=3 * top * ff * h * 2)
        else:
            add(f"routed experts ({top} of {E}, six kernels), {t} tokens", "", run_moe, 3, flops=6.0 * t * top * ff * h)
            add(f"Qwen2: gated feed-forward of width {top * ff}, {t} tokens", "like the one above", run_dense, 3, flops=6.0 * t * top * ff * h)
    ops.check_status()
    return rows


# ------------------------------------------------------------------- the Lutodra design beside Retodra
# Layer sizes that resemble real models'.  Lutodra: a real-gated linear recurrent unit with a dense feed-forward, attention
# with sinks and routed experts, the gated delta rule with a dense feed-forward, attention again; four residual streams.
# Retodra (recurrent layers in turn with attention layers, dense and routed feed-forwards) at equal width, heads, head
# size, feed-forward widths and experts is the nearest model the engine has; its attention has a window, Lutodra's has not.
LUTODRA_SIZES = {"2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, experts=16, top=2, expert_ff=2048, layers=4, streams=4),
                 "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, experts=32, top=4, expert_ff=2048, layers=4, streams=4)}
LUTODRA_VOCAB, LUTODRA_CONTEXT, LUTODRA_PROMPT = 32000, 2048, 2048


def lutodra_configs(size):
    z = LUTODRA_SIZES[size]
    w, h = z["width"], z["heads"]
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": h, "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                     "rot": {"base": 1e6, "dims": z["dim"] // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    rec = {"type": "rglru", "mixer": {"width": w, "blocks": h, "conv": 4}, "mlp": dense}
    dlt = {"type": "channel_delta", "mixer": {"heads": h, "kv_heads": h // 2, "dim": 128, "vdim": w // h, "conv": 4}, "mlp": dense}
    lutodra = {"architecture": "Lutodra", "vocab": LUTODRA_VOCAB, "width": w, "streams": z["streams"], "norm": {"eps": 1e-6},
               "logit_scale": 1.0, "layers": [dict((rec, att, dlt, att)[i % 4]) for i in range(z["layers"])]}
    return lutodra


def run_lutodra(a) -> int:
    """Prefill and decode throughput of the Lutodra design beside Retodra at equal layer sizes (random weights, synthetic
    cache contents), and the design's own kernels alone beside the like kernels of the engine's other models with their
    share of the measured peaks.  One JSON line."""
    import numpy as np
    peaks = load_peaks()
    steps, warmup = max(1, a.steps), max(3, a.warmup)
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    sampler.mark("decode")
    out = {"metric": "prefill and decode tok/s of Lutodra beside Retodra at equal layer sizes (bf16, random weights)",
           "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic", "sizes": {}, "peaks": peaks}
    sizes = a.lutodra.split(",") if a.lutodra != "all" else sorted(LUTODRA_SIZES)
    for size in sizes:
        args = (steps, warmup, rng, peaks, LUTODRA_VOCAB, LUTODRA_CONTEXT, LUTODRA_PROMPT)
        out["sizes"][size] = {"layers": LUTODRA_SIZES[size], "lutodra": measure_design(lutodra_configs(size), (8, 64), *args),
                              "retodra": measure_design(retodra_configs(size)[0], (8, 64), *args)}
    if not a.skip_points:
        out["kernels"] = lutodra_kernels(LUTODRA_SIZES[sizes[-1]], peaks)
    out["clocks"] = sampler.stop()
    big = out["sizes"][sizes[-1]]
    out.update(value=big["lutodra"]["decode"]["8"]["tok_s"], unit=f"tokens/s (Lutodra, {sizes[-1]}-wide layers, batch 8)",
               higher_is_better=True, gpu_launches=big["lutodra"]["decode"]["8"]["launches_per_step"] * steps,
               config={"sizes": LUTODRA_SIZES, "context": LUTODRA_CONTEXT, "prompt": LUTODRA_PROMPT,
                       "retodra_window": RETODRA_WINDOW, "l2": "a step's weights exceed the 126 MB of L2"})
    print(json.dumps(out))
    return 0


def lutodra_kernels(z, peaks):
    """The design's own kernels alone at one layer size, each beside the like kernel of another model of the engine:
    [{kernel, like, us, GB/s or TFLOP/s, share of the measured peak}, ...] (CUDA graphs on rotating buffers)."""
    import numpy as np
    import torch
    from vllm_cpp_b200.csrc import ops
    h, nh, nkv, d, S, page, bf, dev = z["width"], z["heads"], z["kv_heads"], z["dim"], z["streams"], 16, torch.bfloat16, "cuda"
    dk, dv, G, J = 128, h // nh, nh // 2, 4
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, like, fn, copies, bytes_=0, flops=0, peak=None):
        us = ops.time_in_graph(fn, reps=max(4, copies))
        rate = bytes_ / us / 1e3 if bytes_ else flops / us / 1e6
        row = {"kernel": name, "like": like, "us": round(us, 2), ("gb_s" if bytes_ else "tflop_s"): round(rate, 1)}
        if bytes_ or peak != "none":
            row["of_peak"] = round(rate / (peaks["hbm_gbs"] if bytes_ else peaks["bf16_tflops"]), 4)
        rows.append(row)

    ones = lambda n: torch.ones(n, device=dev)
    # ---- rows of the residual streams
    for t in (64, 2048):
        c = 6 if t == 64 else 3
        x = [rnd(S, t, h, dtype=torch.float32) for _ in range(c)]
        y, o1 = ([rnd(t, h) for _ in range(c)] for _ in range(2))
        mix, coef, gain, bias = torch.eye(S, device=dev), ones(S), ones(h), torch.zeros(h, device=dev)
        add(f"{S} streams rejoined + next sublayer's read + layer norm, {t} tokens", "", lambda i: ops.stream_join(
            x[i % c], y[i % c], mix, coef, 1e-6, next_coef=coef, next_w=gain, next_b=bias, next_out=o1[i % c]), c, bytes_=t * h * (8 * S + 4))
        x1 = [rnd(t, h, dtype=torch.float32) for _ in range(c)]
        add(f"Retodra: post norm + layer scale + addition + next norm, {t} tokens", "like the one above",
            lambda i: ops.norm_residual_norm(y[i % c], gain, x1[i % c], 1e-6, next_gain=gain, next_out=o1[i % c], next_eps=1e-6), c, bytes_=t * h * 12)
    # ---- the short convolutions and the recurrent unit: single tokens of a batch, then a prompt
    for n_reqs, per in ((8, 1), (64, 1), (1, LUTODRA_PROMPT)):
        t, c = n_reqs * per, 3
        what = f"decode, batch {n_reqs}" if per == 1 else f"prompt of {per}"
        q_start = torch.arange(0, t + 1, per, dtype=torch.int32, device=dev)
        slots = torch.arange(n_reqs, dtype=torch.int32, device=dev)
        xin = [rnd(t, 2 * h) for _ in range(c)]
        u = [torch.empty(t, h, device=dev) for _ in range(c)]
        state = torch.zeros(n_reqs, J, h, device=dev)
        taps, lam = rnd(h, J, dtype=torch.float32), torch.full((h,), 0.5, device=dev)
        add(f"causal convolution of {J} taps, {h} channels, {what}", "Retodra: token shift is the nearest (two rows mixed)",
            lambda i: ops.causal_conv(xin[i % c][:, h:], taps, state[:, 1:], u[i % c], q_start, slots, n_reqs, per, pre_bias=lam, bias=lam), c,
            bytes_=t * h * 6 + 2 * n_reqs * (J - 1) * h * 4)
        bs = h // nh
        wa, wi = rnd(nh, bs, bs, scale=bs ** -0.5), rnd(nh, bs, bs, scale=bs ** -0.5)
        decay, drive = ([torch.empty(t, h, device=dev) for _ in range(c)] for _ in range(2))
        kw = dict(flops=4.0 * t * h * bs, peak="none") if per > 1 else dict(bytes_=2 * nh * bs * bs * 2 + t * h * 12)
        add(f"gates of the recurrent unit ({nh} blocks of {bs}, float FMA), {what}", "", lambda i: ops.gate_blocks(
            u[i % c], wa, wi, lam, lam, lam, decay[i % c], drive[i % c], 8.0), c, **kw)
        for k in range(c):
            decay[k].uniform_(0.5, 1.0)
        act = [torch.empty(t, h, dtype=bf, device=dev) for _ in range(c)]
        add(f"linear recurrence + gelu branch, {h} channels, {what}", "", lambda i: ops.linear_recurrence(
            decay[i % c], drive[i % c], xin[i % c][:, :h], lam, state[:, 0], act[i % c], q_start, slots, n_reqs, per), c,
            bytes_=t * h * 12 + 2 * n_reqs * h * 4)
    # ---- the gated delta rule beside Retodra's recurrence with a decay per channel (64 key channels there, 128 here)
    for n_reqs, per in ((8, 1), (64, 1), (1, LUTODRA_PROMPT)):
        t = n_reqs * per
        what = f"decode, batch {n_reqs}" if per == 1 else f"prompt of {per}, token by token"
        q_start = torch.arange(0, t + 1, per, dtype=torch.int32, device=dev)
        slots = torch.arange(n_reqs, dtype=torch.int32, device=dev)
        c = 3 if per == 1 else 1
        state = [torch.zeros(n_reqs, nh, dk, dv, device=dev) for _ in range(c)]
        q, k, v = rnd(t, G * dk, dtype=torch.float32), rnd(t, G * dk, dtype=torch.float32), rnd(t, nh * dv, dtype=torch.float32)
        beta, pre, o = rnd(t, nh), rnd(t, nh * dk), torch.empty(t, nh * dv, device=dev)
        a_log, dtb = torch.zeros(nh, device=dev), torch.zeros(nh * dk, device=dev)
        kw = dict(bytes_=n_reqs * nh * dk * dv * 8) if per == 1 else dict(flops=8.0 * t * nh * dk * dv, peak="none")
        work = torch.empty(t * ops.gated_delta_work_row(nh, G, dk), device=dev)
        add(f"gated delta rule, {nh} heads of {dk} x {dv}, {what}", "", lambda i: ops.gated_delta_scan(
            q, k, v, beta, pre, a_log, dtb, state[i % c], o, q_start, slots, n_reqs, num_heads=nh, num_qk_heads=G, q_scale=dk ** -0.5,
            unit_eps=1e-6, max_q_len=per, work=work), max(2, c), **kw)
        state2 = [torch.zeros(n_reqs, nh, 64, dv, device=dev) for _ in range(c)]
        q2, k2, pre2, bias2 = rnd(t, nh * 64), rnd(t, nh * 64, scale=0.1), rnd(t, nh * 64), torch.zeros(nh * 64, device=dev)
        v2 = rnd(t, nh * dv)
        kw = dict(bytes_=n_reqs * nh * 64 * dv * 8) if per == 1 else dict(flops=4.0 * t * nh * 64 * dv, peak="none")
        add(f"Retodra: recurrence (decay per channel), {nh} heads of 64 x {dv}, {what}", "like the one above", lambda i: ops.decayed_state_scan(
            q2, k2, v2, state2[i % c], o, q_start, slots, n_reqs, num_heads=nh, decay_pre=pre2, decay_bias=bias2, tau=16.0, q_scale=0.125),
            max(2, c), **kw)
    for t in (64, 2048):
        c = 3
        of = [rnd(t, nh * dv, dtype=torch.float32) for _ in range(c)]
        gt, gw, o1 = rnd(t, nh * dv), ones(dv), [torch.empty(t, nh * dv, dtype=bf, device=dev) for _ in range(c)]
        add(f"norm per head + sigmoid gate, {t} tokens", "the same kernel as Retodra's (silu there)", lambda i: ops.gated_group_norm(
            of[i % c], gt, gw, o1[i % c], group=dv, eps=1e-6, gate_act="sigmoid"), c, bytes_=t * nh * dv * 8)
        # ---- q/k norm per head + partial rotation + cache write beside Retodra's norm + cache write
        width = (nh + 2 * nkv) * d + nh
        proj = [rnd(t, width) for _ in range(c)]
        n_pages = t // page + 2
        kvc = torch.zeros(n_pages, 2 * nkv * page * d, dtype=bf, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        req, pos = torch.zeros(t, dtype=torch.int32, device=dev), torch.arange(t, dtype=torch.int32, device=dev)
        q_out = torch.empty(t, nh * d, dtype=bf, device=dev)
        inv_freq = torch.from_numpy(np.power(1e6, -np.arange(d // 4, dtype=np.float64) * 4 / d).astype(np.float32)).to(dev)
        sizes = dict(num_heads=nh, num_kv_heads=nkv, head_dim=d, v_head_dim=d, row=d, page_size=page, eps=1e-6, write_kv=True)
        g_head, g_q, g_k = ones(d), ones(nh * d), ones(nkv * d)
        add(f"q/k norm per head + rotation of {d // 2} of {d} + cache write, {t} tokens", "", lambda i: ops.qk_head_rope_cache_write(
            proj[i % c], 0, nh * d, (nh + nkv) * d, g_head, g_head, inv_freq, q_out, kvc, pos, req, bt, **sizes), c,
            bytes_=t * (nh + 2 * nkv) * d * 4)
        add(f"Retodra: q/k norm over the projection + cache write, {t} tokens", "like the one above", lambda i: ops.qk_norm_cache_write(
            proj[i % c], 0, nh * d, (nh + nkv) * d, g_q, g_k, q_out, kvc, pos, req, bt, **sizes), c,
            bytes_=t * (nh + 2 * nkv) * d * 4)
    rows += lutodra_attention_kernels(z, peaks, add, rnd)
    return rows


def lutodra_attention_kernels(z, peaks, add, rnd):
    """Attention with a sink and a gate per head beside plain attention (the same kernels without the epilogue), and the
    routed experts with grouped sigmoid routing beside a dense gated feed-forward of the chosen experts' width."""
    import numpy as np
    import torch
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    from vllm_cpp_b200.parts.base import Workspace
    from vllm_cpp_b200.parts.mlp import GatedMLP
    from vllm_cpp_b200.parts.moe import RoutedExperts
    h, nh, nkv, d, page, bf, dev = z["width"], z["heads"], z["kv_heads"], z["dim"], 16, torch.bfloat16, "cuda"
    t = LUTODRA_PROMPT
    n_pages = t // page + 2
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
    q_start, ctx = torch.tensor([0, t], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    G = nh // nkv
    n_tiles = -(-t * G // ops.TC_ATTENTION_TILE_ROWS)
    tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
    tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[::-1].copy()).to(dev)
    q, o = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev)
    kv = rnd(n_pages, 2, nkv, page * d, scale=0.5)
    sink, gate = rnd(nh, dtype=torch.float32), rnd(t, nh)
    seen = t * (t + 1) // 2
    for epi, name, like in ((True, f"attention with sink, head gate and two-term weights, prompt of {t}", ""),
                            (False, f"Qwen2: attention, prompt of {t}", "like the one above")):
        kw = dict(sink=sink, head_gate=gate, precise_weights=True) if epi else {}
        add(name, like, lambda i: ops.attention_prefill_tc(q, kv, o, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=nkv, head_dim=d,
                                                           page_size=page, window=0, scale=d ** -0.5, **kw), 4, flops=4.0 * nh * d * seen)
    part = PagedAttention(h, nh, nkv, d, True, False, 0, PartSpec("none"), bf, dev)
    for batch in (8, 64):
        contexts = [LUTODRA_CONTEXT - 1] * batch
        blocks = -(-LUTODRA_CONTEXT // page)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start, ctx = torch.arange(batch + 1, dtype=torch.int32, device=dev), torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, contexts, page)
        split_tiles = torch.from_numpy(part.step_arrays()[part._splits_key()](host)).to(dev)
        nsplit = host.shapes[part._splits_key()]
        need = batch * nh * nsplit
        share = ops.decode_head_groups(nh, nkv)
        po, pml, tickets = torch.empty(need * d, device=dev), torch.empty(need * 2, device=dev), torch.zeros(batch * nkv * share, dtype=torch.int32, device=dev)
        q, o = rnd(batch, nh * d), torch.empty(batch, nh * d, dtype=bf, device=dev)
        kv = rnd(batch * blocks + 1, 2, nkv, page * d, scale=0.5)
        gate = rnd(batch, nh)
        for epi, name, like in ((True, f"attention with sink, head gate and two-term weights, decode, batch {batch}, context {LUTODRA_CONTEXT}", ""),
                                (False, f"Qwen2: attention, decode, batch {batch}, context {LUTODRA_CONTEXT}", "like the one above")):
            kw = dict(sink=sink, head_gate=gate, precise_weights=True) if epi else {}
            add(name, like, lambda i: ops.attention_decode_mma(q, kv, o, q_start, ctx, bt, None, batch, nsplit, po, pml, tickets, num_heads=nh,
                                                               num_kv_heads=nkv * share, head_dim=d, page_size=page, window=0, scale=d ** -0.5,
                                                               split_tiles=split_tiles, kv_share=share, **kw), 4,
                bytes_=batch * LUTODRA_CONTEXT * 2 * nkv * d * 2)
    # ---- routed experts (sigmoid scores, groups) beside a dense gated feed-forward of the width the chosen experts have together
    E, top, ff = z["experts"], z["top"], z["expert_ff"]
    moe = RoutedExperts(h, ff, E, 0, top, float("inf"), bf, dev, activation="silu", score="sigmoid", correction=False, groups=4, keep_groups=2,
                        group_top=2, normalize=True, sum_eps=1e-20, route_scale=2.5)
    tensors = {"router": rnd(E, h, dtype=torch.float32, scale=0.05)}
    for e in range(E):
        tensors.update({f"e{e}.gate": rnd(ff, h, scale=0.02), f"e{e}.up": rnd(ff, h, scale=0.02), f"e{e}.down": rnd(h, ff, scale=0.02)})
    moe.load_params(tensors)
    del tensors
    dense = [GatedMLP(h, top * ff, "silu", bf, dev) for _ in range(3)]
    for m in dense:
        m.load_params({"gate_proj.weight": rnd(top * ff, h, scale=0.02), "up_proj.weight": rnd(top * ff, h, scale=0.02),
                       "down_proj.weight": rnd(h, top * ff, scale=0.02)})
        ops.tile_weights(m.w_gate_up, top * ff)
        ops.tile_weights(m.w_down)
    ws = Workspace(dev, 1 << 30)
    for t in (8, 64, 2048):
        x, out = rnd(t, h), torch.empty(t, h, dtype=bf, device=dev)

        def run_moe(i):
            ws.reset()
            moe.forward(x, out, None, ws)

        def run_dense(i):
            ws.reset()
            dense[i % 3].forward(x, out, None, ws)

        reach = min(E, t * top)
        kw = dict(bytes_=reach * 3 * ff * h * 2) if t <= 128 else dict(flops=6.0 * t * top * ff * h)
        add(f"routed experts ({top} of {E} in 4 groups of which 2 stay), {t} tokens", "", run_moe, 3, **kw)
        kw = dict(bytes_=3 * top * ff * h * 2) if t <= 128 else dict(flops=6.0 * t * top * ff * h)
        add(f"Qwen2: gated feed-forward of width {top * ff}, {t} tokens", "like the one above", run_dense, 3, **kw)
    ops.check_status()
    return []


# ------------------------------------------------------------------- the Gipinex design beside Lutodra's attention layers
# Layer sizes that resemble real models'.  Gipinex: latent attention (queries through a latent, one rotated key part, a cached
# row of kv_rank + rot_dim = 128) with a dense clamped feed-forward and with routed experts beside a shared expert, then
# two layers of attention with talking heads and a distance bias with routed experts; the first two layers are walked twice.
# Lutodra with attention layers alone (head norms, rotation, a sink, a gate per head; dense and routed feed-forwards; the
# same loop) at equal width, heads, head size, feed-forward widths and experts is the nearest model the engine has.
GIPINEX_SIZES = {"1k": dict(width=1024, heads=8, kv_heads=2, dim=128, ff=4096, experts=8, top=2, expert_ff=1024, layers=4, q_rank=384),
                 "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, experts=16, top=2, expert_ff=2048, layers=4, q_rank=768)}
GIPINEX_VOCAB, GIPINEX_CONTEXT, GIPINEX_PROMPT, GIPINEX_RANK, GIPINEX_ROT = 32000, 2048, 2048, 96, 32


def gipinex_configs(size):
    z = GIPINEX_SIZES[size]
    w, h, d = z["width"], z["heads"], z["dim"]
    dense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["expert_ff"], "limit": 7.0}}
    lat = {"heads": h, "dim": d - GIPINEX_ROT, "rot_dim": GIPINEX_ROT, "vdim": d, "kv_rank": GIPINEX_RANK, "q_rank": z["q_rank"],
           "scale": d ** -0.5, "rot": {"base": 1e6, "dims": GIPINEX_ROT}}
    att = {"heads": h, "kv_heads": z["kv_heads"], "dim": d, "vdim": d, "scale": 0.125}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": dense}, {"type": "latent_attention", "mixer": lat, "mlp": moe},
              {"type": "attention", "mixer": att, "mlp": moe}, {"type": "attention", "mixer": att, "mlp": moe}]
    loop = {"start": 0, "stop": 2, "times": 2}
    gipinex = {"architecture": "Gipinex", "vocab": GIPINEX_VOCAB, "width": w, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
               "loop": loop, "layers": [layers[i % 4] for i in range(z["layers"])]}
    l_moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5}}
    l_att = {"heads": h, "kv_heads": z["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5, "rot": {"base": 1e6, "dims": d // 2}}
    lutodra = {"architecture": "Lutodra", "vocab": GIPINEX_VOCAB, "width": w, "norm": {"eps": 1e-6}, "loop": loop,
               "layers": [{"type": "attention", "mixer": l_att, "mlp": {"kind": "dense", "ff": z["ff"]} if i % 4 == 0 else l_moe}
                          for i in range(z["layers"])]}
    return gipinex, lutodra


def run_gipinex(a) -> int:
    """Prefill and decode throughput of the Gipinex design beside Lutodra's attention layers at equal layer sizes (random
    weights, synthetic cache contents), and the design's own kernels alone beside the like kernels of the engine's other
    models with their share of the measured peaks.  One JSON line."""
    import numpy as np
    peaks = load_peaks()
    steps, warmup = max(1, a.steps), max(3, a.warmup)
    rng = np.random.default_rng(0)
    sampler = ClockSampler()
    sampler.start()
    sampler.mark("decode")
    out = {"metric": "prefill and decode tok/s of Gipinex beside Lutodra's attention layers at equal layer sizes (bf16, random weights)",
           "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic", "sizes": {}, "peaks": peaks}
    sizes = a.gipinex.split(",") if a.gipinex != "all" else sorted(GIPINEX_SIZES)
    for size in sizes:
        gipinex, lutodra = gipinex_configs(size)
        args = (steps, warmup, rng, peaks, GIPINEX_VOCAB, GIPINEX_CONTEXT, GIPINEX_PROMPT)
        out["sizes"][size] = {"layers": GIPINEX_SIZES[size], "gipinex": measure_design(gipinex, (8, 64), *args),
                              "lutodra_attention": measure_design(lutodra, (8, 64), *args)}
    if not a.skip_points:
        out["kernels"] = gipinex_kernels(GIPINEX_SIZES[sizes[-1]], peaks)
    out["clocks"] = sampler.stop()
    big = out["sizes"][sizes[-1]]
    out.update(value=big["gipinex"]["decode"]["8"]["tok_s"], unit=f"tokens/s (Gipinex, {sizes[-1]}-wide layers, batch 8)",
               higher_is_better=True, gpu_launches=big["gipinex"]["decode"]["8"]["launches_per_step"] * steps,
               config={"sizes": GIPINEX_SIZES, "context": GIPINEX_CONTEXT, "prompt": GIPINEX_PROMPT, "kv_rank": GIPINEX_RANK,
                       "rot_dim": GIPINEX_ROT, "l2": "a step's weights exceed the 126 MB of L2"})
    print(json.dumps(out))
    return 0


def gipinex_kernels(z, peaks):
    """The design's own kernels alone at one layer size, each beside the like kernel of another model of the engine:
    [{kernel, like, us, GB/s or TFLOP/s, share of the measured peak}, ...] (CUDA graphs on rotating buffers)."""
    import numpy as np
    import torch
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.parts.talking_attention import TalkingHeadsAttention, distance_slopes
    h, nh, nkv, d, page, bf, dev = z["width"], z["heads"], z["kv_heads"], z["dim"], 16, torch.bfloat16, "cuda"
    rank, rot, ff = GIPINEX_RANK, GIPINEX_ROT, z["ff"]
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, like, fn, copies, bytes_=0, flops=0):
        us = ops.time_in_graph(fn, reps=max(4, copies))
        rate = bytes_ / us / 1e3 if bytes_ else flops / us / 1e6
        rows.append({"kernel": name, "like": like, "us": round(us, 2), ("gb_s" if bytes_ else "tflop_s"): round(rate, 1),
                     "of_peak": round(rate / (peaks["hbm_gbs"] if bytes_ else peaks["bf16_tflops"]), 4)})

    talk = TalkingHeadsAttention(h, nh, nkv, d, 0.125, 1e-6, bf, dev)
    mix = (torch.eye(nh, device=dev) + 0.1 * torch.randn(nh, nh, device=dev)).contiguous()
    slopes = torch.from_numpy(distance_slopes(nh, 8.0).astype(np.float32)).to(dev)
    plainatt = PagedAttention(h, nh, nkv, d, True, False, 0, PartSpec("none"), bf, dev)
    # ---- a prompt
    t = GIPINEX_PROMPT
    n_pages = t // page + 2
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
    q_start, ctx = torch.tensor([0, t], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    q, o, gate = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev), rnd(t, nh * d)
    kv = rnd(n_pages, 2 * nkv * page * d, scale=0.5)
    host = HostStep([t], [0], page)
    lists = talk.step_arrays()
    items = torch.from_numpy(lists[talk._items_key()](host)).to(dev)
    joins = torch.from_numpy(lists[talk._items_key() + "_joins"](host)).to(dev)       # tiles cut along their keys, joined by a second kernel
    wide = talk.max_wide_slots() * ops.TALKING_ITEM_ROWS * nh
    wo, wml = torch.empty(wide * d, device=dev), torch.empty(wide * 2, device=dev)
    seen = t * (t + 1) // 2
    add(f"attention with talking heads, distance bias, gate and two-term weights, prompt of {t}", "", lambda i: ops.attention_talking_mma(
        q, kv, o, gate, items, items.shape[0], q_start, ctx, bt, mix, slopes, nsplit=1, n_reqs=1, num_heads=nh, num_kv_heads=nkv, head_dim=d,
        page_size=page, window=0, scale=0.125, part_o=wo, part_ml=wml, merge=joins, n_merge=joins.shape[0]), 4, flops=4.0 * nh * d * seen)
    G = nh // nkv
    n_tiles = -(-t * G // ops.TC_ATTENTION_TILE_ROWS)
    tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
    tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[::-1].copy()).to(dev)
    kv4 = kv.view(n_pages, 2, nkv, page * d)
    hg = rnd(t, nh)
    add(f"Lutodra: attention with sink, head gate and two-term weights, prompt of {t}", "like the one above", lambda i: ops.attention_prefill_tc(
        q, kv4, o, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=0, scale=d ** -0.5,
        sink=slopes, head_gate=hg, precise_weights=True), 4, flops=4.0 * nh * d * seen)
    # ---- single tokens
    for batch in (8, 64):
        contexts = [GIPINEX_CONTEXT - 1] * batch
        blocks = -(-GIPINEX_CONTEXT // page)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start, ctx = torch.arange(batch + 1, dtype=torch.int32, device=dev), torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, contexts, page)
        items = torch.from_numpy(talk.step_arrays()[talk._items_key()](host)).to(dev)
        runs = host.shapes[talk._items_key() + "_runs"]
        po, pml = torch.empty(batch * runs * nh * d, device=dev), torch.empty(batch * runs * nh * 2, device=dev)
        q, o, gate = rnd(batch, nh * d), torch.empty(batch, nh * d, dtype=bf, device=dev), rnd(batch, nh * d)
        kv = rnd(batch * blocks + 1, 2 * nkv * page * d, scale=0.5)
        moved = batch * GIPINEX_CONTEXT * 2 * nkv * d * 2
        add(f"attention with talking heads, decode, batch {batch}, context {GIPINEX_CONTEXT} ({runs} runs of keys a request)", "",
            lambda i: ops.attention_talking_mma(q, kv, o, gate, items, items.shape[0], q_start, ctx, bt, mix, slopes, nsplit=runs, n_reqs=batch,
                                                num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page, window=0, scale=0.125,
                                                part_o=po, part_ml=pml, single_rows=True), 4, bytes_=moved)
        host = HostStep([1] * batch, contexts, page)
        split_tiles = torch.from_numpy(plainatt.step_arrays()[plainatt._splits_key()](host)).to(dev)
        nsplit = host.shapes[plainatt._splits_key()]
        share = ops.decode_head_groups(nh, nkv)
        need = batch * nh * nsplit
        p2, pm2, tickets = torch.empty(need * d, device=dev), torch.empty(need * 2, device=dev), torch.zeros(batch * nkv * share, dtype=torch.int32, device=dev)
        hg = rnd(batch, nh)
        add(f"Lutodra: attention with sink, head gate and two-term weights, decode, batch {batch}, context {GIPINEX_CONTEXT}", "like the one above",
            lambda i: ops.attention_decode_mma(q, kv.view(-1, 2, nkv, page * d), o, q_start, ctx, bt, None, batch, nsplit, p2, pm2, tickets,
                                               num_heads=nh, num_kv_heads=nkv * share, head_dim=d, page_size=page, window=0, scale=d ** -0.5,
                                               split_tiles=split_tiles, kv_share=share, sink=slopes, head_gate=hg, precise_weights=True), 4,
            bytes_=moved)
    # ---- rows: the latent's norm, the shared key part's rotation and the cache write; the queries' latent norm; the activation
    inv_freq = torch.from_numpy(np.power(1e6, -2.0 * np.arange(rot // 2) / rot).astype(np.float32)).to(dev)
    ones_d = torch.ones(d, device=dev)
    for t in (64, 2048):
        c = 6 if t == 64 else 3
        n_pages = t // page + 1
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        rot_ = torch.zeros(t, dtype=torch.int32, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        raw, qq = [rnd(t, rank + rot) for _ in range(c)], [rnd(t, nh * d) for _ in range(c)]
        cache1 = rnd(n_pages, page * (rank + rot))
        gain = torch.ones(rank, device=dev)
        add(f"latent norm + rotation of the shared key part and of {nh} query parts + cache write, {t} tokens", "", lambda i: ops.latent_rope_cache_write(
            raw[i % c], gain, qq[i % c], inv_freq, pos, rot_, bt, cache1, rank=rank, num_heads=nh, q_stride=d, q_off=d - rot, pairing=1,
            page_size=page, eps=1e-6), c, bytes_=t * ((rank + rot) * 4 + nh * rot * 4))
        proj = [rnd(t, (nh + 2 * nkv) * d) for _ in range(c)]
        qo = [torch.empty(t, nh * d, dtype=bf, device=dev) for _ in range(c)]
        cache2 = rnd(n_pages, 2 * nkv * page * d)
        add(f"q/k divided by their root mean square per head + cache write of both planes, {t} tokens", "Lutodra's kernel (there with rotation)",
            lambda i: ops.qk_head_rope_cache_write(proj[i % c], 0, nh * d, nh * d, ones_d, ones_d, None, qo[i % c], cache2, pos, rot_, bt,
                                                   num_heads=nh, num_kv_heads=nkv, head_dim=d, v_head_dim=d, row=d, page_size=page, eps=1e-6,
                                                   write_kv=True), c, bytes_=t * (nh + nkv) * d * 4 + t * nkv * d * 2)
        cq, cqo = [rnd(t, z["q_rank"]) for _ in range(c)], [torch.empty(t, z["q_rank"], dtype=bf, device=dev) for _ in range(c)]
        gq = torch.ones(z["q_rank"], device=dev)
        add(f"norm of the queries' latent ({z['q_rank']} wide), {t} tokens", "", lambda i: ops.rows_rmsnorm(cq[i % c], gq, cqo[i % c], 1e-6), c,
            bytes_=t * z["q_rank"] * 4)
        gu, act = [rnd(t, 2 * ff) for _ in range(c)], [torch.empty(t, ff, dtype=bf, device=dev) for _ in range(c)]
        bias = rnd(2 * ff, dtype=torch.float32, scale=0.1)
        add(f"clamped activation with biases, width {ff}, {t} tokens", "", lambda i: ops.clamped_swish_mul(gu[i % c], bias, act[i % c], limit=7.0, alpha=1.702), c,
            bytes_=t * ff * 6)
        add(f"Qwen2: silu(gate) * up, width {ff}, {t} tokens", "like the one above", lambda i: ops.silu_mul(gu[i % c], act[i % c]), c, bytes_=t * ff * 6)
        x = [rnd(t, h, dtype=torch.float32) for _ in range(c)]
        dl, pair = [rnd(t, h) for _ in range(c)], [torch.empty(t, 2 * h, dtype=bf, device=dev) for _ in range(c)]
        add(f"stream + 0.5 * addition into the left half of the re-making product's input, {t} tokens", "", lambda i: ops.cast_rows(
            x[i % c], dl[i % c], 0.5, pair[i % c][:, :h]), c, bytes_=t * h * 8)
        nrm, gh = [torch.empty(t, h, dtype=bf, device=dev) for _ in range(c)], torch.ones(h, device=dev)
        add(f"stream += 0.5 * addition, then the norm, {t} tokens", "the kernel Qwen2 runs with factor 1", lambda i: ops.add_rmsnorm(
            x[i % c], dl[i % c], gh, nrm[i % c], 1e-6, None, 0.5), c, bytes_=t * h * 12)
    ops.check_status()
    return rows


# ------------------------------------------------------------------------------------------ reference arm
REFERENCE_NOTES = ("the reference's own faults at these sizes, none of which changes the work of a step: an untied lm_head is "
                   "copied over the embedding table (src/model/qwen.cpp:279-281); the bias area of 3*1024 floats a layer "
                   "(qwen.cpp:67,113-114,179-181) is overrun by 7B's 4,608 and the surplus lands, inside the same pool, on "
                   "layer 0's rotation table below position 336")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
    return 0


def run_reference(cfg, a) -> int:
    """The reference's own speed on the same configuration: write the model folder, run baseline/_ref/ref_driver."""
    if a.gpus != 1:
        return unavailable("jiamumuzhao/vllm-cpp has no multi-GPU path")
    try:
        from baseline.build_reference import driver_env, driver_path
        driver = driver_path()
    except Exception as e:                                # the build's own message is the reason
        return unavailable(f"the reference could not be built here: {e}")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from vllm_cpp_b200.weights.random_init import write_random_model
    except Exception as e:
        return unavailable(f"cannot prepare the model folder: {e}")
    nums = model_numbers(cfg)
    params = nums["matrix_params"] + cfg["vocab_size"] * cfg["hidden_size"]          # with the embedding table
    need_file = params * 2 + (64 << 20)
    # the reference's loader keeps every tensor as host float32 (src/model/model_loader.cpp:61,100) beside the file
    need_ram = params * 4 + need_file + (8 << 30)
    with open("/proc/meminfo") as f:
        avail = next(int(l.split()[1]) * 1024 for l in f if l.startswith("MemAvailable"))
    where = next((d for d in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(d)
                  and shutil.disk_usage(d).free > need_file + (4 << 30)), None)
    if where is None:
        return unavailable(f"no room for the {need_file >> 30} GB model folder in /dev/shm or the temporary folder")
    if avail < need_ram:
        return unavailable(f"the reference's loader needs about {need_ram >> 30} GB of host memory "
                           f"(float32 copies of all tensors), {avail >> 30} GB are available")
    runs = decode_runs(max(1, a.steps))
    per_run = min(k for _, k in runs)
    runs = [(c, per_run) for c, _ in runs]                # the driver takes one length for all runs
    warm = max(3, a.warmup)
    folder = tempfile.mkdtemp(prefix="vcb_ref_model_", dir=where)
    try:
        t0 = time.time()
        write_random_model(folder, cfg, seed=0, dtype="bfloat16", device="cuda")
        torch.cuda.empty_cache()
        write_s = time.time() - t0
        print(f"[bench] model folder written in {write_s:.0f} s", file=sys.stderr, flush=True)
        # batch 64 is left out unless asked for: one forward of the reference at these contexts takes a
        # good part of a second, and a step of 64 sequences is 64 of them
        batches = [a.batch] + ([] if a.skip_points else [b for b in ((1, 64) if a.reference_b64 else (1,)) if b != a.batch])
        cmd = [driver, "bench", "--model", folder, "--batches", ",".join(map(str, batches)),
               "--contexts", ",".join(str(c) for c, _ in runs), "--steps-per-context", str(per_run),
               "--warmup", str(warm), "--prefill", str(PREFILL_TOKENS), "--max-model-len", str(CONTEXT + 16),
               "--block-size", "16", "--budget-s", str(a.reference_budget_s)]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=None, text=True, env=driver_env())
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    lines = [l for l in p.stdout.strip().splitlines() if l.startswith("{")]
    if p.returncode != 0 or not lines:
        tail = p.stdout.strip().splitlines()[-3:]
        return unavailable(f"the reference's run ended with code {p.returncode}: {' | '.join(tail)}")
    res = json.loads(lines[-1])
    if "error" in res:
        return unavailable(f"the reference's run stopped: {res['error']}")
    by_batch = {r["batch"]: r["decode"] for r in res["runs"]}
    main = by_batch[a.batch]
    steps = per_run * len(main)
    ms = sum(d["device_ms_per_step"] for d in main) / len(main)
    e2e_ms = sum(d["e2e_ms_per_step"] for d in main) / len(main)
    points = {f"decode_b{a.batch}_ctx{main[0]['context']}": round(a.batch / (main[0]["device_ms_per_step"] * 1e-3), 2),
              f"decode_b{a.batch}_ctx{main[-1]['context'] + per_run}": round(a.batch / (main[-1]["device_ms_per_step"] * 1e-3), 2)}
    for b, dec in by_batch.items():
        if b != a.batch:
            points[f"decode_b{b}"] = round(b / (sum(d["device_ms_per_step"] for d in dec) / len(dec) * 1e-3), 2)
    blocks = res["blocks_per_seq"]
    line = {
        "impl": "reference", "metric": METRIC, "value": round(a.batch / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warm, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulation, activations and cache (the reference's only mode)",
        "data": "synthetic: the same random weights N(0,0.02) as the other arm, written as a bfloat16 model folder; random token ids",
        "config": flat_config(cfg, a, nums, {
            "how": "QwenModel::forward, one call per token and sequence, as Engine::decode and Engine::prefill call it",
            "cache": "zeros as the reference's pool is cleared to, plus what the steps write",
            "load_s": res["load_s"], "write_model_s": round(write_s, 1), "notes": REFERENCE_NOTES}),
        "e2e": {"value": round(a.batch / (e2e_ms * 1e-3), 2), "unit": "tokens/s",
                # per sequence: the token id, and per layer the block table and the context length; the logits back
                "h2d_bytes_per_step": a.batch * (4 + res["layers"] * 4 * (blocks + 1)),
                "d2h_bytes_per_step": a.batch * 4 * res["vocab"]},
        "gpu_launches": None,
        "prefill": ({"value": round(res["prefill"]["tokens"] / (res["prefill"]["ms"] * 1e-3), 1), "tokens": res["prefill"]["tokens"],
                     "ms": round(res["prefill"]["ms"], 1), "how": "one forward per token",
                     # a prompt cut short by the time budget is not the 2,048-token prompt of the metric
                     "same_config": res["prefill"]["tokens"] == PREFILL_TOKENS} if res["prefill"]["tokens"] else None),
        "points": points, "seconds": res["seconds"],
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ our arm
def main() -> int:
    global CONTEXT_START, CONTEXT, PREFILL_TOKENS, SLACK
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=QWEN25_7B["num_hidden_layers"],
                    help="fewer layers than the 28 of the configuration (recorded in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="7b", choices=sorted(SIZES),
                    help="layer sizes: Qwen2.5-7B (the benchmark's), 14B or 32B")
    ap.add_argument("--mix", action="store_true",
                    help="instead of the fixed-batch measurement: 32 requests with prompts of 128 to 4,096 tokens and "
                         "256 generated tokens each through the engine, 2,048 tokens a step (continuous batching)")
    ap.add_argument("--kernels", action="store_true",
                    help="instead of the step: every kernel alone at these layer sizes, a text table of microseconds "
                         "and achieved GB/s or TFLOP/s")
    ap.add_argument("--host", default="python", choices=["python", "cpp"],
                    help="cpp: decode throughput through the C++ host runtime (vllm::Engine) instead of the Python host")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help=f"with --only prefill: tokens of the one prompt instead of {PREFILL_TOKENS}")
    ap.add_argument("--contexts", default="",
                    help="START,END: the decode measurement's contexts grow from START to END tokens instead of "
                         f"{CONTEXT_START},{CONTEXT} (with --only decode; the default is the benchmark's configuration)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (for profiling); the other fields of the line are null")
    ap.add_argument("--no-pdl", action="store_true", help="ordinary launches instead of programmatic dependent launch")
    ap.add_argument("--library-gemm", action="store_true", help="cuBLAS for every bfloat16 product (no tcgen05 kernel)")
    ap.add_argument("--timeline", metavar="FILE", default=None,
                    help="with --only decode: also write the device timeline of one decode step (every kernel's "
                         "start and end as CUPTI reports them through torch.profiler) to FILE as text")
    ap.add_argument("--no-cuda-graphs", action="store_true",
                    help="launch every kernel of a decode step directly (for a profiler's launch list)")
    ap.add_argument("--utilization", type=int, default=0, metavar="PERCENT",
                    help="let the engine size its own cache from this share of the device's memory "
                         "(gpu_memory_utilization) instead of a fixed number of pages")
    ap.add_argument("--reference-budget-s", type=float, default=1300.0,
                    help="--impl reference: begin no further measurement after this many seconds")
    ap.add_argument("--reference-b64", action="store_true", help="--impl reference: measure batch 64 too (many minutes)")
    ap.add_argument("--rolesun", default="", metavar="SIZES",
                    help="instead of the benchmark's workload: prefill and decode throughput of the Rolesun design beside Qwen2 "
                         f"at equal layer sizes ({','.join(sorted(ROLESUN_SIZES))} or 'all'), and the design's kernels alone "
                         "beside the like kernels of Qwen2's layer")
    ap.add_argument("--lutodra", default="", metavar="SIZES",
                    help="instead of the benchmark's workload: prefill and decode throughput of the Lutodra design beside Retodra "
                         "at equal layer sizes, and the design's kernels alone: 'all' or a comma list of " + ",".join(sorted(LUTODRA_SIZES)))
    ap.add_argument("--gipinex", default="", metavar="SIZES",
                    help="instead of the benchmark's workload: prefill and decode throughput of the Gipinex design beside Lutodra's "
                         "attention layers at equal layer sizes, and the design's kernels alone: 'all' or a comma list of "
                         + ",".join(sorted(GIPINEX_SIZES)))
    ap.add_argument("--retodra", default="", metavar="SIZES",
                    help="instead of the benchmark's workload: prefill and decode throughput of the Retodra design beside Qwen2 "
                         f"at equal layer sizes ({','.join(sorted(RETODRA_SIZES))} or 'all'), and the design's kernels alone "
                         "beside the like kernels of Qwen2's layer")
    a = ap.parse_args()
    if a.contexts:
        CONTEXT_START, CONTEXT = (int(v) for v in a.contexts.split(","))
        if a.only != "decode" or not 0 < CONTEXT_START < CONTEXT:
            ap.error("--contexts START,END goes with --only decode and needs 0 < START < END")
    if a.prefill_tokens:
        if a.only != "prefill" or a.prefill_tokens < 2:
            ap.error("--prefill-tokens N goes with --only prefill")
        PREFILL_TOKENS = a.prefill_tokens
        CONTEXT_START, CONTEXT = max(CONTEXT_START, PREFILL_TOKENS), max(CONTEXT, PREFILL_TOKENS + 64)
    SLACK = max(SLACK, a.batch + 32)          # requests begin a prompt's step apart: the first is a batch of steps ahead of the last
    cfg = dict(QWEN25_7B, **SIZES[a.size])
    if a.size == "7b" or a.layers != QWEN25_7B["num_hidden_layers"]:
        cfg["num_hidden_layers"] = a.layers
    if a.impl == "reference":
        return run_reference(cfg, a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU (N=1); this engine has no multi-GPU path, --gpus {a.gpus} is not run")
        return 2
    steps, warmup = max(1, a.steps), max(3, a.warmup)

    import torch
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.llm_engine import Engine
    from vllm_cpp_b200.engine.runner import StepEntry

    if a.no_pdl:
        ops.set_pdl(False)
    if a.library_gemm:
        ops.set_tcgen05_linear(False)
    if a.rolesun:
        return run_rolesun(a)
    if a.retodra:
        return run_retodra(a)
    if a.lutodra:
        return run_lutodra(a)
    if a.gipinex:
        return run_gipinex(a)
    if a.mix:
        return run_mix(cfg, a)
    if a.kernels:
        return run_kernels(cfg)
    if a.host == "cpp":
        return run_cpp_host(cfg, a)
    nums = model_numbers(cfg)
    peaks = load_peaks()
    max_batch = a.batch if a.only != "all" else max(64, a.batch)        # the points at batch 1 and 64 use the same engine
    pages = max_batch * ((CONTEXT + SLACK) // 16 + 1) + PREFILL_TOKENS // 16 + 16
    ecfg = EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                        num_gpu_blocks=None if a.utilization else pages,
                        gpu_memory_utilization=a.utilization or 90, max_num_seqs=max_batch, max_model_len=CONTEXT + SLACK,
                        max_num_batched_tokens=PREFILL_TOKENS, max_tokens_per_step=PREFILL_TOKENS,
                        use_cuda_graphs=not a.no_cuda_graphs)
    t0 = time.time()
    engine = Engine(ecfg)
    runner, cache = engine.runner, engine.cache
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator(device="cuda").manual_seed(1)
    for g in cache.paged:                       # synthetic cache contents for the decode runs
        g.pages.normal_(0.0, 0.5, generator=gen)
    vocab = cfg["vocab_size"]
    rng = __import__("numpy").random.default_rng(0)
    runs = decode_runs(steps)

    def time_decode(batch, n_warm):
        """Device time of the timed runs of decode steps at ``batch`` requests: [(context, steps, ms)], launches."""
        temperature = torch.zeros(batch, device="cuda")
        uniform = torch.zeros(batch, device="cuda")
        out = torch.empty(batch, dtype=torch.int32, device="cuda")
        results, launches = [], 0
        for ctx0, k in runs:
            toks = rng.integers(0, vocab, size=(max(k, n_warm), batch))

            def requests(tag):                  # requests whose caches hold ctx0 tokens (synthetic contents)
                ids = [f"d{batch}_{ctx0}_{tag}{i}" for i in range(batch)]
                for r in ids:
                    cache.add_request(r)
                    cache.reserve(r, ctx0)
                    cache.commit(r, ctx0)
                return ids

            def one(ids, j):
                logits = runner.step([StepEntry(r, [int(toks[j, i])], [0]) for i, r in enumerate(ids)])
                ops.sample(logits, temperature, uniform, out)

            # warm-up: the run itself once over, with requests of its own, so that the timed steps find
            # their launch shapes captured (a step whose longest context enters a new power-of-two bucket,
            # as 2,048 -> 2,049 does, is otherwise launched directly once and captured once)
            ids = requests("w")
            for j in range(max(k, n_warm)):
                one(ids, j)
            for r in ids:
                cache.free_request(r)
            ids = requests("t")
            torch.cuda.synchronize()
            before = ops.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push("timed_decode")
            e0.record()
            for j in range(k):
                one(ids, j)
            e1.record()
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            results.append((ctx0, k, e0.elapsed_time(e1)))
            launches += ops.launch_count() - before
            for r in ids:
                cache.free_request(r)
        return results, launches

    def summary(batch, results):
        """tokens/s over all runs, ms per step, bytes the steps had to read."""
        total_ms = sum(ms for _, _, ms in results)
        n = sum(k for _, k, _ in results)
        kv = sum(batch * (c + (k - 1) / 2 + 1) * nums["kv_bytes_per_token"] * k for c, k, _ in results)
        return batch * n / (total_ms * 1e-3), total_ms / n, nums["matrix_params"] * 2 * n + kv

    def time_prefill(reps, n_warm):
        times = []
        for k in range(reps + n_warm):
            cache.add_request("p")
            toks = rng.integers(0, vocab, size=PREFILL_TOKENS).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if k >= n_warm:
                torch.cuda.nvtx.range_push("timed_prefill")
            e0.record()
            runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
            e1.record()
            torch.cuda.synchronize()
            if k >= n_warm:
                torch.cuda.nvtx.range_pop()
            cache.free_request("p")
            if k >= n_warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def time_e2e(batch):
        """Wall time of engine.step() over the same runs of steps: requests with prompts just short of
        CONTEXT_START tokens generate until their contexts reach CONTEXT; pinned inputs in, sampled ids out, every
        step.  A run is timed between two synchronisations; the steps between the runs are not timed."""
        lead = 64                               # steps before the first run: the prompts' steps leave reduced clocks behind
        prompt_len = CONTEXT_START - lead
        sp = SamplingParams(max_tokens=CONTEXT + SLACK - prompt_len, temperature=0.0, ignore_eos=True)
        ids = [engine.add_request(rng.integers(0, vocab, size=prompt_len).tolist(), sp) for _ in range(batch)]
        seqs = [engine.sequences[i] for i in ids]
        while engine.scheduler.waiting or any(s.remaining > 1 or s.output_len == 0 for s in seqs):
            engine.step()
        produced, seconds = 0, 0.0
        for ctx0, k in runs:
            while min(s.num_processed_tokens for s in seqs) < ctx0:
                engine.step()
            assert len(engine.scheduler.running) == batch
            torch.cuda.synchronize()
            t = time.perf_counter()
            got = 0
            for _ in range(k):
                got += len(engine.step())
            torch.cuda.synchronize()
            seconds += time.perf_counter() - t
            assert got == batch * k, (got, batch, k)
            produced += got
        h2d = int(runner.last_meta_bytes) + 4 * 4 * batch        # step metadata + four floats of sampling options a row
        for i in ids:
            engine.abort_request(i)
        return produced / seconds, h2d, 4 * batch

    def prefill_flops(t):
        """The products of every layer and the output product of the one wanted row, and causal attention."""
        return 2.0 * (nums["matrix_params"] - vocab * cfg["hidden_size"]) * t + 2.0 * vocab * cfg["hidden_size"] \
            + cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * nums["d"] * (t * (t + 1) / 2)

    if a.only == "prefill":
        ms = time_prefill(max(1, min(steps, 3)), 2)
        tf = prefill_flops(PREFILL_TOKENS) / (ms * 1e-3) / 1e12
        print(json.dumps({"metric": METRIC, "only": "prefill", "tokens": PREFILL_TOKENS, "prefill_ms": round(ms, 3),
                          "value": round(PREFILL_TOKENS / (ms * 1e-3), 1), "unit": "tokens/s", "tflops": round(tf, 1),
                          "frac": round(tf / peaks["bf16_tflops"], 4),
                          "frac_of_sustained_peak": round(tf / peaks["bf16_tflops_sustained"], 4)}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    clocks.mark("decode")
    results, launches = time_decode(a.batch, warmup)
    value, ms, step_bytes = summary(a.batch, results)
    if a.only == "decode":
        clock_info = clocks.stop()
        if a.timeline:
            write_timeline(a.timeline, a.batch, runner, cache, rng, vocab)
        print(json.dumps({"metric": METRIC, "only": "decode", "batch": a.batch, "ms_per_step": round(ms, 4),
                          "value": round(value, 1), "unit": "tokens/s", "gpu_launches": launches,
                          "contexts": [CONTEXT_START, CONTEXT],
                          "roofline": {"achieved": round(step_bytes / (ms * sum(k for _, k, _ in results) * 1e-3) / 1e9, 1),
                                       "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": round(step_bytes / (ms * sum(k for _, k, _ in results) * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)},
                          "runs": [[c, k, round(t / k, 4)] for c, k, t in results],
                          "product_grids": {f"{n}x{k} tile {bn}{' gated' if g else ''}{' residual' if r else ''}": c
                                            for (n, k, bn, g, r), c in sorted(ops._cta_choice.items())},
                          "layer_products_us": getattr(engine.model, "tuning_report", {}).get("layer_products_us"),
                          "cuda_graphs": not a.no_cuda_graphs, "clocks": clock_info}))
        return 0
    n_timed = sum(k for _, k, _ in results)
    achieved = step_bytes / (ms * n_timed * 1e-3) / 1e9

    # The decode figures first, the prefill last: the prefill steps run at the power limit, and what is
    # measured right after them runs at the reduced clocks they leave behind for a while.
    (c_first, k_first, t_first), (c_last, k_last, t_last) = results[0], results[-1]
    points = {f"decode_b{a.batch}_ctx{c_first}": round(a.batch * k_first / (t_first * 1e-3), 1),
              f"decode_b{a.batch}_ctx{c_last + k_last}": round(a.batch * k_last / (t_last * 1e-3), 1)}
    if not a.skip_points:
        for b in (1, 64):
            if b != a.batch:
                res_b, _ = time_decode(b, 3)
                points[f"decode_b{b}"] = round(summary(b, res_b)[0], 1)
    clocks.mark("e2e")
    e2e_value, h2d, d2h = time_e2e(a.batch)
    clocks.mark("prefill")
    prefill_ms = time_prefill(3, 2)
    clock_info = clocks.stop()
    t = PREFILL_TOKENS
    tflops = prefill_flops(t) / (prefill_ms * 1e-3) / 1e12
    prefill = {"value": round(t / (prefill_ms * 1e-3), 1), "tokens": t, "ms": round(prefill_ms, 3),
               # one step timed alone between synchronisations: the burst peak is its denominator
               "frac": round(tflops / peaks["bf16_tflops"], 4),
               "frac_of_sustained_peak": round(tflops / peaks["bf16_tflops_sustained"], 4), "tflops": round(tflops, 1)}

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": n_timed,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": flat_config(cfg, a, nums, {
            "l2": "inputs larger than L2 (a decode step reads %.1f GB)" % (step_bytes / n_timed / 1e9),
            "cuda_graphs": bool(ecfg.use_cuda_graphs), "overlap_steps": bool(ecfg.overlap_decode_steps),
            "peaks": peaks["source"], "load_s": round(load_s, 1), "kv_pages": cache.num_pages}),
        "clocks": clock_info,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
