#!/usr/bin/env python3
"""Benchmark: decode tokens/s (batch 1, 8, 64) and prefill tokens/s (2,048 tokens) of a
MiniCPM4-8B-sized model with random bf16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run is batch 8 with the
sequences ending at the context length of 4,096 tokens.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# MiniCPM4-8B layer sizes; random weights N(0, 0.02), seed 2; bf16.
MODEL = {
    "architectures": ["MiniCPMForCausalLM"], "model_type": "minicpm",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 16384, "vocab_size": 73448,
    "rope_theta": 10000.0, "max_position_embeddings": 65536, "rms_norm_eps": 1e-6,
    "scale_emb": 12, "dim_model_base": 256, "scale_depth": 1.4, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# MiniCPM4-0.5B layer sizes; random weights seed 3; tied head.
MODEL_HALF_B = dict(MODEL, num_hidden_layers=24, hidden_size=1024, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=64, intermediate_size=4096, tie_word_embeddings=True)
# InfLLM-v2 knobs of the long-context workload (8B sizes).
SPARSE_8B = {"kernel_size": 32, "kernel_stride": 16, "block_size": 64, "init_blocks": 1, "topk": 64,
             "window_size": 2048, "dense_len": 8192}
FULL_LAYERS = 32
CONTEXT = 4096
PREFILL_TOKENS = 2048
SEED = 2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def long_factors(n: int) -> list:
    import torch
    g = torch.Generator().manual_seed(SEED)
    return sorted((1.0 + 39.0 * torch.rand(n, generator=g)).tolist())


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as f:
            data = json.load(f)
        if "hbm_gbs" in data and "bf16_tflops" in data:
            out = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in data:
                out["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(steps: int, warmup: int) -> int:
    """Runs the unmodified reference, installed under baseline/_ref, through its own Python API in a process of
    its own (baseline/run_reference.py; nothing of this package is on that path) and passes its JSON line on.
    The install: a copy of the reference with its empty ``src/cutlass`` submodule folder filled from the CUTLASS
    header tree that ships with an installed package, built with CPMCU_CUDA_ARCH=100 CPMCU_DTYPE=bf16."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "cpmcu")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no installed reference (pip install --no-index --no-build-isolation "
                          "--target baseline/_ref of a copy of the reference whose src/cutlass holds CUTLASS headers)"}))
        return 0
    cfgd = dict(MODEL)
    cfgd["rope_scaling"] = {"rope_type": "longrope", "long_factor": long_factors(64), "short_factor": [1.0] * 64,
                            "original_max_position_embeddings": 32768}
    env = dict(os.environ, PYTHONPATH=ref + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--model-json", json.dumps(cfgd),
           "--steps", str(steps), "--warmup", str(max(3, warmup)), "--context", str(CONTEXT),
           "--prefill-tokens", str(PREFILL_TOKENS), "--seed", str(SEED)]
    try:
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=tempfile.gettempdir())
    except subprocess.TimeoutExpired:
        print(json.dumps({"impl": "reference", "unavailable": "the reference run did not end within 1500 s"}))
        return 0
    line = next((l for l in reversed(p.stdout.splitlines()) if l.startswith("{") and '"impl"' in l), None)
    if p.returncode != 0 or line is None:
        err = [l.strip() for l in (p.stderr + "\n" + p.stdout).splitlines() if l.strip() and not l.startswith("{")]
        picked = [l for l in err if "error" in l.lower() or "Error" in l or "Signal" in l][-3:] or err[-2:]
        print(json.dumps({"impl": "reference", "unavailable": f"the reference run failed (exit {p.returncode}): "
                          + (" | ".join(picked)[:400] if picked else "no output")}))
        sys.stderr.write(p.stderr[-6000:])
        return 0
    print(line)
    return 0


def build_engine(n_layers: int, max_tokens: int, max_batch: int, model: dict = None, seed: int = SEED,
                 max_seq_tokens: int = None, chunk_tokens: int = None, sparse: dict = None):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    cfgd = dict(model or MODEL, num_hidden_layers=n_layers)
    half = cfgd["head_dim"] // 2
    cfgd["rope_scaling"] = {"rope_type": "longrope", "long_factor": long_factors(half), "short_factor": [1.0] * half,
                            "original_max_position_embeddings": 32768}
    if sparse:
        cfgd["sparse_config"] = dict(sparse)
    arch = architecture("MiniCPMForCausalLM")
    cfg = arch.config_class.from_dict(cfgd)
    # the residual scale of the full depth, whatever number of layers is built
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    chunk = chunk_tokens or PREFILL_TOKENS
    # one arena: weights, step workspace, per-sequence state and the key-value pages (as the Python entry point does)
    if os.environ.get("CPMCU_BENCH_ARENA", "1") == "0":              # for comparisons: every tensor from torch's allocator
        from cpmcu_b200.cache import Cache
        model.load_weights(random_tensors(model.weight_specs(), seed, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
        cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=torch.bfloat16, device="cuda:0",
                      n_slots=max_batch + 2, max_seq_tokens=max_seq_tokens or CONTEXT + 64, max_step_tokens=chunk)
        return cfg, model, cache, Stepper(model, cache, chunk_tokens=chunk, graph_prompts=True)
    storage = make_storage(model, chunk, max_batch, max_tokens=max_tokens, max_seq_tokens=max_seq_tokens or CONTEXT + 64,
                           n_slots=max_batch + 2)
    model.load_weights(random_tensors(model.weight_specs(), seed, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
    torch.cuda.empty_cache()                                         # the loader's tensors: their copies live in the arena
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=chunk, graph_prompts=True)


def random_prompt(vocab: int, n: int, seed: int) -> list:
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def time_decode(stepper, batch: int, steps: int, warmup: int, vocab: int, sample_clocks: bool = False,
                context: int = None):
    """Sequences are prefilled so that the timed steps end at the context length; returns
    (ms per step, clocks, launches in the timed region, bytes of cache read per step)."""
    import torch
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.engine.decode import DecodeRunner
    from cpmcu_b200.ops import library
    from cpmcu_b200.sampling import SamplingParams

    context = context or CONTEXT
    start_len = context - steps - warmup - 1
    slots = stepper.open(batch)
    first = []
    for i, s in enumerate(slots):                       # one prompt per step keeps the workspace small
        out = stepper.step([SequenceStep(s, random_prompt(vocab, start_len, 100 + i), [start_len - 1])])
        first.append(int(out.argmax(dim=-1)[0]))
    runner = DecodeRunner(stepper, use_graph=True, seed=SEED)
    runner.start(slots, first, list(range(batch)), [1] * batch, [SamplingParams()] * batch)
    runner.step()
    for _ in range(max(0, warmup - 1)):
        runner.step()
    torch.cuda.synchronize()
    sampler = ClockSampler()
    if sample_clocks:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    clocks = sampler.stop() if sample_clocks else None
    mean_ctx = context - 1 - steps / 2
    cache_bytes = sum(stepper.model.blocks[e.layer].mixer.cache_bytes_read(int(mean_ctx)) for e in stepper.model.schedule) * batch
    launches = runner.launches_per_graph * steps
    for s in slots:
        stepper.close(s)
    stepper.close(runner.pad_slot)
    return ms, clocks, launches, cache_bytes


def time_prefill(stepper, cfg, reps: int = 3):
    import torch
    from cpmcu_b200.engine import SequenceStep

    times = []
    for r in range(reps + 1):
        ids = random_prompt(cfg.vocab_size, PREFILL_TOKENS, 500 + r)
        slot = stepper.open(1)[0]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stepper.step([SequenceStep(slot, ids, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if r > 0:
            times.append(e0.elapsed_time(e1))
        stepper.close(slot)
    return statistics.median(times)


def prefill_flops(cfg, n_layers: int, tokens: int) -> float:
    h, d = cfg.hidden_size, cfg.head_dim
    per_layer = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h + cfg.num_attention_heads * d * h \
        + 3 * cfg.intermediate_size * h
    gemm = 2.0 * tokens * per_layer * n_layers + 2.0 * cfg.vocab_size * h
    attn = 4.0 * cfg.num_attention_heads * d * tokens * tokens / 2 * n_layers
    return gemm + attn


def time_e2e(cfg, stepper, steps: int, batch: int):
    """The same decode metric through the Python entry point's loop: host token lists in,
    host token lists out, one device-to-host read of the sampled tokens per step."""
    import torch
    from cpmcu_b200.engine.backend import EngineBackend
    from cpmcu_b200.engine.generate import Request, run_requests
    from cpmcu_b200.sampling import SamplingParams

    backend = EngineBackend(stepper, max_batch=batch, use_graph=True, seed=SEED)
    n_new = steps + 1
    prompts = [random_prompt(cfg.vocab_size, CONTEXT - n_new, 900 + i) for i in range(batch)]
    reqs = [Request(p, n_new, SamplingParams(), (), key=i) for i, p in enumerate(prompts)]
    run_requests(backend, [Request(p[:64], 4, SamplingParams(), (), key=i) for i, p in enumerate(prompts)],
                 sync=torch.cuda.synchronize)                       # warm-up: graph capture
    h0, d0 = backend.h2d_bytes, backend.d2h_bytes
    results, stats = run_requests(backend, reqs, sync=torch.cuda.synchronize)
    assert all(len(r.tokens) == n_new for r in results)
    decode_steps = max(1, stats.decode_steps)
    prompt_bytes = 4 * sum(len(p) for p in prompts)
    return {
        "value": batch * decode_steps / stats.decode_time, "unit": "tokens/s",
        "h2d_bytes_per_step": (backend.h2d_bytes - h0 - prompt_bytes) / decode_steps,
        "d2h_bytes_per_step": (backend.d2h_bytes - d0) / (decode_steps + 1),
        "prefill_tokens_per_s": stats.prompt_tokens / stats.prefill_time,
    }


def loop_prefill(stepper, prompts, max_batch: int):
    """Prompts of one batch through the generation loop's backend (chunked as the stepper is set up), one new token
    each; returns (tokens per second, milliseconds)."""
    import torch
    from cpmcu_b200.engine.backend import EngineBackend
    from cpmcu_b200.engine.generate import Request, run_requests
    from cpmcu_b200.sampling import SamplingParams

    backend = EngineBackend(stepper, max_batch=max_batch, use_graph=True, seed=SEED)
    reqs = [Request(p, 1, SamplingParams(), (), key=i) for i, p in enumerate(prompts)]
    run_requests(backend, [Request(p[:64], 1, SamplingParams(), (), key=i) for i, p in enumerate(prompts)],
                 sync=torch.cuda.synchronize)                                   # warm-up
    best = None
    for _ in range(2):
        _, stats = run_requests(backend, reqs, sync=torch.cuda.synchronize)
        best = stats.prefill_time if best is None else min(best, stats.prefill_time)
    stepper.close(backend.runner.pad_slot)
    return sum(len(p) for p in prompts) / best, best * 1e3


def workload_half_b(steps: int, warmup: int) -> int:
    """MiniCPM4-0.5B layer sizes: 64 prompts of unequal lengths (uniform in [64, 2048]) prefilled in chunks of 512
    packed tokens, and decode steps of the 64 sequences that end at a context of 8,192 tokens."""
    import torch

    batch, context, chunk = 64, 8192, 512
    pk = peaks()
    cfg, model, cache, stepper = build_engine(MODEL_HALF_B["num_hidden_layers"], batch * (context + 64) + 128, batch,
                                              model=MODEL_HALF_B, seed=3, max_seq_tokens=context + 64, chunk_tokens=2048)
    stepper.chunk_tokens = chunk                                                # the workload's prompts: chunks of 512
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(64, 2049, (batch,), generator=g).tolist()
    prompts = [random_prompt(cfg.vocab_size, n, 300 + i) for i, n in enumerate(lens)]
    prefill_tps, prefill_ms = loop_prefill(stepper, prompts, batch)
    stepper.chunk_tokens = 2048                                                 # the long warm-up prompts in larger pieces
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab_size, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "workload": "half_b", "metric": "decode tokens/s (MiniCPM4-0.5B sizes, bf16, batch 64, context 8192)",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 3",
        "config": {"model": "MiniCPM4-0.5B sizes", "layers": cfg.num_hidden_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": True, "global_batch": batch,
                   "seq_len": context, "prompt_lengths": "uniform in [64, 2048]", "chunk_length": chunk, "cuda_graph": True,
                   "peaks": pk["source"]},
        "prefill": {"value": prefill_tps, "tokens": sum(lens), "ms": prefill_ms, "through": "generation loop"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "weight_bytes": weight_bytes, "cache_bytes": cache_bytes},
        "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


def workload_sparse8b(steps: int, warmup: int, layers: int) -> int:
    """MiniCPM4-8B layer sizes with InfLLM-v2 block-sparse attention: prompts of 16,384 and 30,000 tokens in one
    batch, prefilled in chunks of 2,048 packed tokens through the generation loop, then decode steps of the two
    sequences under a CUDA graph."""
    import torch
    from cpmcu_b200.engine import SequenceStep
    from cpmcu_b200.engine.decode import DecodeRunner
    from cpmcu_b200.sampling import SamplingParams

    lens, context = [16384, 30000], 32768
    pk = peaks()
    cfg, model, cache, stepper = build_engine(layers, 3 * context + 256, 2, seed=4, max_seq_tokens=context + 64,
                                              chunk_tokens=2048, sparse=SPARSE_8B)
    prompts = [random_prompt(cfg.vocab_size, n, 40 + i) for i, n in enumerate(lens)]
    prefill_tps, prefill_ms = loop_prefill(stepper, prompts, 2)
    stepper.ops.raise_on_kernel_error()
    slots = stepper.open(2)
    first = []
    for s_, p_ in zip(slots, prompts):
        out = stepper.step([SequenceStep(s_, p_, [len(p_) - 1])])
        first.append(int(out.argmax(dim=-1)[0]))
    runner = DecodeRunner(stepper, use_graph=True, seed=SEED)
    runner.start(slots, first, [0, 1], [1, 1], [SamplingParams()] * 2)
    for _ in range(max(3, warmup)):
        runner.step()
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        runner.step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    stepper.ops.raise_on_kernel_error()
    ms = e0.elapsed_time(e1) / steps
    mean_ctx = [n + max(3, warmup) + steps // 2 for n in lens]
    cache_bytes = sum(stepper.model.blocks[e.layer].mixer.cache_bytes_read(c) for e in stepper.model.schedule for c in mean_ctx)
    dense_bytes = sum(2 * c * cfg.num_key_value_heads * cfg.head_dim * 2 * layers for c in mean_ctx)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "workload": "sparse8b", "metric": "decode ms/step and prefill tokens/s (MiniCPM4-8B sizes, InfLLM-v2, batch 2, context 32768)",
        "value": 2 * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": max(3, warmup),
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 4",
        "config": {"model": "MiniCPM4-8B sizes", "layers": layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": 2, "seq_len": context,
                   "prompt_lengths": "16384 and 30000", "chunk_length": 2048, "attention": "InfLLM-v2 32/16/64/1/64/2048/8192",
                   "cuda_graph": True, "peaks": pk["source"]},
        "prefill": {"value": prefill_tps, "tokens": sum(lens), "ms": prefill_ms, "through": "generation loop"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "weight_bytes": weight_bytes, "cache_bytes": cache_bytes,
                     "cache_bytes_if_dense": dense_bytes},
        "clocks": clocks, "gpu_launches": runner.launches_per_graph * steps,
    }))
    return 0


def step_launches(name: str, batch: int, ctx: int, layers: int, reps: int, workload: str = "dense8b") -> int:
    """A few eager steps of a model with few layers of a workload's sizes, one kernel launch after the other, for
    a profiler's launch list: decode_step = one token for each of ``batch`` sequences that hold ``ctx`` tokens;
    prefill_step = a prompt of ``ctx`` tokens."""
    import torch
    from cpmcu_b200.engine import SequenceStep

    global CONTEXT
    CONTEXT = max(CONTEXT, ctx + 64)
    cfg, model, cache, stepper = build_engine(layers, batch * (ctx + 128) + 128, batch,
                                              model=MODEL_HALF_B if workload == "half_b" else MODEL,
                                              sparse=SPARSE_8B if workload == "sparse8b" else None)
    if name == "decode_step":
        slots = stepper.open(batch)
        for i, s in enumerate(slots):
            stepper.step([SequenceStep(s, random_prompt(cfg.vocab_size, ctx, i), [])])
        torch.cuda.synchronize()
        for _ in range(max(1, reps)):
            out = stepper.step([SequenceStep(s, [5], [0]) for s in slots])
            torch.cuda.synchronize()
    else:
        for r in range(max(1, reps)):
            slot = stepper.open(1)[0]
            out = stepper.step([SequenceStep(slot, random_prompt(cfg.vocab_size, ctx, r), [ctx - 1])])
            torch.cuda.synchronize()
            stepper.close(slot)
    print(json.dumps({"kernel": name, "workload": workload, "batch": batch, "ctx": ctx, "layers": layers, "logits": list(out.shape)}))
    return 0


def kernel_bench(name: str, batch: int, ctx: int, rows: int, n: int, k: int, reps: int) -> int:
    """One kernel alone at the benchmark's shapes, timed inside a CUDA graph with rotating
    buffers larger than L2 (also the target of the ncu captures under profiles/)."""
    import math
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import PREFILL_TILE_ROWS, Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops, dev = Ops(torch.bfloat16, "cuda:0"), "cuda:0"
    heads, kv, d = MODEL["num_attention_heads"], MODEL["num_key_value_heads"], MODEL["head_dim"]

    def timed(fn, n_inner):
        fn(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_inner):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * n_inner)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    out = {"kernel": name}
    if name == "skinny_gemm":
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        us = timed(lambda i: ops.linear(x, ws[i % copies]), copies * 2)
        out.update(rows=rows, n=n, k=k, us=us, gbs=n * k * 2 / 1e3 / us)
    elif name == "decode_attention":
        lanes = max(2, int(400e6 // (batch * ctx * kv * d * 4)) + 1)
        cache = Cache([CacheNeeds(kv_heads=kv, head_dim=d)] * lanes, max_tokens=batch * (ctx + 64), dtype=torch.bfloat16,
                      device=dev, n_slots=batch + 1, max_seq_tokens=ctx + 64)
        slots = cache.open_sequences(batch)
        for s_ in slots:
            cache.reserve(s_, ctx)
        cache.sync()
        for lane in cache.lanes:
            lane.k.normal_()
            lane.v.normal_()
        q = torch.randn(batch, heads, d, device=dev, dtype=torch.bfloat16)
        kv_len, sl = i32([ctx] * batch), i32(slots)
        us = timed(lambda i: ops.decode_attention(q, cache.lane(i % lanes).k, cache.lane(i % lanes).v, kv_len, sl,
                                                  cache.lane(0).page_table, kv, 1 / math.sqrt(d)), lanes * 2)
        out.update(batch=batch, ctx=ctx, us=us, gbs=batch * ctx * kv * d * 4 / 1e3 / us)
    elif name in ("prefill_attention", "prefill_attention_mma"):
        cache = Cache([CacheNeeds(kv_heads=kv, head_dim=d)], max_tokens=ctx + 64, dtype=torch.bfloat16, device=dev, n_slots=2)
        slot = cache.open_sequence()
        cache.reserve(slot, ctx)
        cache.sync()
        cache.lane(0).k.normal_()
        cache.lane(0).v.normal_()
        q = torch.randn(ctx, heads, d, device=dev, dtype=torch.bfloat16)
        n_tiles = (ctx + PREFILL_TILE_ROWS - 1) // PREFILL_TILE_ROWS
        tiles = (i32([0] * n_tiles), i32(list(range(0, ctx, PREFILL_TILE_ROWS))), n_tiles)
        cu, kv_len, sl = i32([0, ctx]), i32([ctx]), i32([slot])
        fn = ops.prefill_attention if name == "prefill_attention_mma" else ops.prefill_attention_tcgen05
        us = timed(lambda i: fn(q, cache.lane(0).k, cache.lane(0).v, tiles, cu, kv_len, sl,
                                cache.lane(0).page_table, kv, 1 / math.sqrt(d)), 4)
        out.update(tokens=ctx, us=us, tflops=4 * heads * d * ctx * ctx / 2 / us / 1e6,
                   error_code=ops.attention_tcgen05_error())
    elif name == "gemm_tcgen05":
        # the gated gate_up product of a prompt chunk: rows x k times (n x k)^T, silu(gate) * up in the epilogue
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        us = timed(lambda i: ops.linear_tcgen05(x, ws[i % copies], gated=True), copies * 2)
        out.update(rows=rows, n=n, k=k, us=us, tflops=2.0 * rows * n * k / us / 1e6, error_code=ops.tcgen05_error())
    else:
        print(f"unknown kernel '{name}'; known: skinny_gemm, decode_attention, prefill_attention, prefill_attention_mma, gemm_tcgen05")
        return 2
    print(json.dumps(out))
    return 0


# Reravik at sizes that resemble a real model's layers: eight layers (attention over a cached latent, two gated
# recurrences, attention, ...), the middle four run twice; random weights N(0, 0.02), vectors 1 + N(0, 0.02).
RERAVIK_SIZES = {
    "1k": dict(width=1024, ff=4096, heads=16, dim=64, vdim=64, q_rank=384, kv_rank=256, window=1024, vocab=32000),
    "2k": dict(width=2048, ff=8192, heads=16, dim=128, vdim=128, q_rank=768, kv_rank=512, window=2048, vocab=32000),
    "4k": dict(width=4096, ff=16384, heads=32, dim=128, vdim=128, q_rank=1536, kv_rank=512, window=4096, vocab=73448),
}


def reravik_config(z: dict) -> dict:
    att = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": z["ff"]},
           "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "q_rank": z["q_rank"], "kv_rank": z["kv_rank"],
                     "scale": z["dim"] ** -0.5, "mask": {"size": z["window"]}}}
    gru = {"type": "mingru", "mixer": {"width": z["width"]}, "mlp": {"kind": "dense", "ff": z["ff"]}}
    return {"architecture": "Reravik", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 12.0},
            "norm": {"eps": 1e-5}, "layers": [att, gru, gru, att, att, gru, gru, att], "loop": {"start": 2, "stop": 6, "times": 2}}


def build_reravik(z: dict, max_tokens: int, max_batch: int, context: int):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    arch = architecture("Reravik")
    cfg = arch.config_class.from_dict(reravik_config(z))
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    storage = make_storage(model, PREFILL_TOKENS, max_batch, max_tokens=max_tokens, max_seq_tokens=context + 64, n_slots=max_batch + 2)
    model.load_weights(random_tensors(model.weight_specs(), 4, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
    torch.cuda.empty_cache()
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=PREFILL_TOKENS, graph_prompts=True)


def time_prefill_any(stepper, vocab: int, reps: int = 3) -> float:
    import torch
    from cpmcu_b200.engine import SequenceStep

    times = []
    for r in range(reps + 1):
        ids = random_prompt(vocab, PREFILL_TOKENS, 500 + r)
        slot = stepper.open(1)[0]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stepper.step([SequenceStep(slot, ids, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        if r > 0:
            times.append(e0.elapsed_time(e1))
        stepper.close(slot)
    return statistics.median(times)


def reravik_kernels(z: dict, pk: dict, context: int, batch: int) -> dict:
    """Every kernel of the design alone, at the size's shapes, beside the like kernel of the dense model: a prompt of
    2,048 tokens and a decode step of ``batch`` sequences at ``context`` tokens.  CUDA events around one launch after
    a flush of L2 (a 512 MB buffer is written), median of five; bytes and FLOPs are the algorithmic ones."""
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds, QUERY_TILE_TOKENS, StepContext

    ops = Ops(torch.bfloat16)
    dev = "cuda:0"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    W, H, R, QR, d, vd, win = z["width"], z["heads"], z["kv_rank"], z["q_rank"], z["dim"], z["vdim"], z["window"]
    T = PREFILL_TOKENS
    i32 = dict(dtype=torch.int32, device=dev)

    def timed(fn):
        ts = []
        for _ in range(6):
            flush.fill_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[1:])

    def context_of(q_lens, starts, slots):
        pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
        seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
        cu = torch.tensor([0] + [sum(q_lens[:i + 1]) for i in range(len(q_lens))], **i32)
        kv = [s + n for n, s in zip(q_lens, starts)]
        ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                          q_lens=list(q_lens), kv_lens=kv, slots=list(slots), max_q_len=max(q_lens), max_kv_len=max(kv),
                          token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                          kv_len_dev=torch.tensor(kv, **i32), slot_dev=torch.tensor(list(slots), **i32))
        ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
        tr = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
        ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(tr, **i32), len(ts))
        return ctx

    out = {}

    def note(name, ms, nbytes=0.0, flops=0.0, like=None):
        row = {"us": ms * 1e3}
        if nbytes:
            row["gbs"] = nbytes / (ms * 1e-3) / 1e9
            row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if flops:
            row["tflops"] = flops / (ms * 1e-3) / 1e12
            row["frac_bf16"] = row["tflops"] / pk["bf16_tflops"]
        if like:
            row["like"] = like
        out[name] = row

    n_slots = batch + 2
    # latent lanes and dense lanes for the two designs' attention
    latent = Cache([CacheNeeds(kv_heads=1, head_dim=R, values=False)], max_tokens=(batch + 1) * (context + 64), dtype=torch.bfloat16,
                   device=dev, n_slots=n_slots)
    dense = Cache([CacheNeeds(kv_heads=2, head_dim=d)], max_tokens=(batch + 1) * (context + 64), dtype=torch.bfloat16, device=dev,
                  n_slots=n_slots)
    slots = []
    for c in (latent, dense):
        slots = [c.open_sequence() for _ in range(batch)]
        for s_ in slots:
            c.reserve(s_, context)
        c.sync()
        c.lane(0).k.normal_(0, 0.5)
        if c.lane(0).v is not None:
            c.lane(0).v.normal_(0, 0.5)
    for phase, q_lens, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx = context_of(q_lens, starts, slots[:len(q_lens)])
        n = ctx.n_tokens
        x = torch.randn(n, W, device=dev)
        a = torch.randn(n, W, device=dev).bfloat16()
        vec = [torch.randn(W, device=dev) for _ in range(5)]
        state = torch.zeros(n_slots, W, device=dev)
        note(f"{phase}/layernorm_shift", timed(lambda: ops.layernorm_shift(ctx, x, vec[0], vec[1], 1e-5, vec[2], state)), n * W * 6.0,
             like="add_rmsnorm")
        note(f"{phase}/post_norm_add+norm", timed(lambda: ops.post_norm_add(x, a, vec[0], vec[1], 1e-5, (vec[2], vec[3]))), n * W * 12.0,
             like="add_rmsnorm")
        wn = torch.ones(W, device=dev)
        note(f"{phase}/add_rmsnorm (dense model)", timed(lambda: ops.add_rmsnorm(x, a, 1.0, wn, 1e-5)), n * W * 12.0)
        proj = torch.randn(n, 3 * W, device=dev)
        gstate = torch.zeros(n_slots, W, device=dev)
        note(f"{phase}/mingru_scan", timed(lambda: ops.mingru_scan(ctx, proj, vec[0], vec[1], gstate, W)), n * W * 14.0)
        down = torch.randn(n, QR + R, device=dev)
        gq, gkv = torch.ones(QR, device=dev), torch.ones(R, device=dev)
        note(f"{phase}/latent_norm_store", timed(lambda: ops.latent_norm_store(ctx, down, gq, gkv, latent.lane(0), QR, R, 1e-5)),
             n * (QR + R) * 6.0, like="rope_store")
        qkv = torch.randn(n, (H + 4) * d, device=dev).bfloat16()
        inv = torch.ones(d // 2, device=dev)
        dl = dense.lane(0)
        note(f"{phase}/rope_store (dense model)",
             timed(lambda: ops.rope_store(qkv, H, 2, d, ctx.positions, ctx.token_seq, ctx.slot_dev, dl.page_table, dl.k, dl.v, inv, 1.0, d)),
             n * (H + 4) * d * 2.0 + n * H * d * 2.0 + n * 4 * d * 2.0)
        q = torch.randn(n, H * d, device=dev).bfloat16()
        w_uk = torch.randn(H, d, R, device=dev).bfloat16()
        w_uv = torch.randn(H, R, vd, device=dev).bfloat16()
        note(f"{phase}/head_project q->latent", timed(lambda: ops.head_project(q, w_uk, H, out_f32=True)),
             nbytes=n * H * (d * 2.0 + R * 4.0) + H * d * R * 2.0, flops=2.0 * n * H * d * R)
        q_lat = ops.head_project(q, w_uk, H, out_f32=True)
        keys = [min(win, s + j + 1) for nq, s in zip(q_lens, starts) for j in range(nq)]
        note(f"{phase}/latent_attention", timed(lambda: ops.latent_attention(ctx, q_lat, latent.lane(0), d ** -0.5, win)),
             nbytes=(sum(min(win, s + nq) for nq, s in zip(q_lens, starts)) * R * 2.0 + n * H * R * 8.0) if phase == "decode" else 0.0,
             flops=4.0 * H * R * sum(keys), like="attention")
        narrow = ops.head_project_by_library(n)            # as the mixer does: bf16 weighted latents for the library product
        o_lat = ops.latent_attention(ctx, q_lat, latent.lane(0), d ** -0.5, win, out_compute_dtype=narrow)
        note(f"{phase}/head_project latent->values", timed(lambda: ops.head_project(o_lat, w_uv, H, out_f32=False)),
             nbytes=n * H * (R * (2.0 if narrow else 4.0) + vd * 2.0) + H * vd * R * 2.0, flops=2.0 * n * H * vd * R)
        gu_w = torch.randn(2 * z["ff"], W, device=dev).bfloat16()
        yy = torch.randn(n, W, device=dev).bfloat16()
        note(f"{phase}/gate_up product with tanh-GELU", timed(lambda: ops.gated_linear(yy, gu_w, 8, 1)),
             nbytes=2.0 * (2 * z["ff"] * W + n * W + n * z["ff"]), flops=4.0 * n * z["ff"] * W, like="gate_up with SiLU")
        note(f"{phase}/gate_up product with SiLU (dense model)", timed(lambda: ops.gated_linear(yy, gu_w, 8, 0)),
             nbytes=2.0 * (2 * z["ff"] * W + n * W + n * z["ff"]), flops=4.0 * n * z["ff"] * W)
        qd = torch.randn(n, H, d, device=dev).bfloat16()
        all_keys = [s + j + 1 for nq, s in zip(q_lens, starts) for j in range(nq)]
        note(f"{phase}/attention (dense model, 2 kv heads, no window)", timed(lambda: ops.attention(ctx, qd, dl, 2, d ** -0.5)),
             nbytes=(sum(s + nq for nq, s in zip(q_lens, starts)) * 2 * 2 * d * 2.0) if phase == "decode" else 0.0,
             flops=4.0 * H * d * sum(all_keys))
    return out


def workload_reravik(steps: int, warmup: int, size: str, batch: int) -> int:
    """Reravik at one of RERAVIK_SIZES beside MiniCPM4 with equal hidden size, feed-forward size, heads and as many
    layers as the Reravik schedule has runs: decode steps of ``batch`` sequences ending at a context of 4,096 tokens
    under a CUDA graph, a prompt of 2,048 tokens, and every kernel of the design alone beside its like."""
    import torch

    z, pk, context = RERAVIK_SIZES[size], peaks(), CONTEXT
    cfg, model, cache, stepper = build_reravik(z, batch * (context + 64) + 128, batch, context)
    runs = len(model.schedule)
    pre_ms = time_prefill_any(stepper, cfg.vocab)
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    del model, cache, stepper
    torch.cuda.empty_cache()
    like = dict(MODEL, hidden_size=z["width"], intermediate_size=z["ff"], num_attention_heads=z["heads"], num_key_value_heads=2,
                head_dim=z["dim"], vocab_size=z["vocab"])
    dcfg, dmodel, dcache, dstepper = build_engine(runs, batch * (context + 64) + 128, batch, model=like, max_seq_tokens=context + 64)
    d_pre = time_prefill_any(dstepper, dcfg.vocab_size)
    d_ms, _, d_launches, d_cache = time_decode(dstepper, batch, steps, warmup, dcfg.vocab_size, False, context=context)
    d_weights = dmodel.weight_bytes_per_step()
    d_achieved = (d_weights + d_cache) / (d_ms * 1e-3) / 1e9
    del dmodel, dcache, dstepper
    torch.cuda.empty_cache()
    kernels = reravik_kernels(z, pk, context, batch)
    print(json.dumps({
        "workload": "reravik", "metric": f"decode tokens/s (Reravik {size} sizes, bf16, batch {batch}, context {context})",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 4",
        "config": dict(z, size=size, layers=len(cfg.layers), runs=runs, global_batch=batch, seq_len=context,
                       prefill_tokens=PREFILL_TOKENS, cuda_graph=True, peaks=pk["source"]),
        "prefill": {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "ms": pre_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "weight_bytes": weight_bytes, "cache_bytes": cache_bytes},
        "closest_model": {"model": f"MiniCPM4 with hidden {z['width']}, intermediate {z['ff']}, {z['heads']} heads of {z['dim']}, 2 kv heads, {runs} layers",
                          "decode_tokens_s": batch * 1000.0 / d_ms, "ms_per_step": d_ms, "prefill_tokens_s": PREFILL_TOKENS / (d_pre * 1e-3),
                          "prefill_ms": d_pre, "roofline_frac": d_achieved / pk["hbm_gbs"], "weight_bytes": d_weights,
                          "cache_bytes": d_cache, "gpu_launches": d_launches},
        "kernels": kernels, "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


# Mufevik at sizes that resemble a real model's layers: eight layers (gated delta rule, two layers of attention beside
# gated linear attention, delta rule, ...), four residual streams, routed experts; random weights N(0, 0.02), vectors
# 1 + N(0, 0.02), stream mixes the identity.
MUFEVIK_SIZES = {
    "1k": dict(width=1024, heads=16, kv_heads=4, dim=64, vdim=64, lin_heads=8, lin_dim=64, lin_vdim=128, delta_heads=16,
               delta_qk_heads=8, delta_dim=64, delta_vdim=64, conv=4, experts=32, top=4, groups=4, keep=2, ff=512, shared=1024,
               streams=4, vocab=32000),
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, lin_heads=16, lin_dim=64, lin_vdim=128, delta_heads=16,
               delta_qk_heads=8, delta_dim=128, delta_vdim=128, conv=4, experts=64, top=6, groups=8, keep=4, ff=768, shared=1536,
               streams=4, vocab=32000),
}


def mufevik_config(z: dict) -> dict:
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"], "keep": z["keep"]}},
           "expert": {"ff": z["ff"]}, "shared": {"ff": z["shared"]}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                              "scale": z["dim"] ** -0.5, "rot": {"dims": z["dim"], "base": 10000.0}},
                     "right": {"heads": z["lin_heads"], "dim": z["lin_dim"], "vdim": z["lin_vdim"], "tau": 8.0, "rank": 32}}}
    delta = {"type": "delta", "mlp": mlp, "mixer": {"heads": z["delta_heads"], "kv_heads": z["delta_qk_heads"], "dim": z["delta_dim"],
                                                     "vdim": z["delta_vdim"], "conv": z["conv"]}}
    return {"architecture": "Mufevik", "vocab": z["vocab"], "width": z["width"], "streams": z["streams"], "logit_scale": 1.0,
            "norm": {"eps": 1e-5}, "layers": [delta, par, par, delta, delta, par, par, delta]}


def build_mufevik(z: dict, max_tokens: int, max_batch: int, context: int):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    arch = architecture("Mufevik")
    cfg = arch.config_class.from_dict(mufevik_config(z))
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    storage = make_storage(model, PREFILL_TOKENS, max_batch, max_tokens=max_tokens, max_seq_tokens=context + 64, n_slots=max_batch + 2)
    tensors = random_tensors(model.weight_specs(), 5, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0")
    S = z["streams"]
    for name, t in tensors.items():
        if ".hc" in name and name.endswith(".mix"):
            t.copy_(torch.eye(S, dtype=t.dtype, device=t.device))
        elif ".hc" in name and name.endswith(".in"):
            t.fill_(1.0 / S)
        elif name.endswith(".talk"):
            t.copy_(torch.eye(t.shape[0], dtype=t.dtype, device=t.device))
        elif name.endswith((".conv", ".correction", ".A_log", ".dt_bias")):
            t.mul_(0.3)
    model.load_weights(tensors)
    del tensors
    torch.cuda.empty_cache()
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=PREFILL_TOKENS, graph_prompts=True)


def mufevik_kernels(z: dict, pk: dict, context: int, batch: int) -> dict:
    """Every kernel of the design alone, at the size's shapes, beside the like kernel of the closest models (the dense
    model's attention, norm, rotary store and gated product; the other recurrent design's scan): a prompt of 2,048
    tokens and a decode step of ``batch`` sequences at ``context`` tokens.  CUDA events around one launch after a
    flush of L2 (a 512 MB buffer is written), median of five; bytes and FLOPs are the algorithmic ones."""
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds, QUERY_TILE_TOKENS, StepContext

    ops = Ops(torch.bfloat16)
    dev = "cuda:0"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    W, H, G, d, dv, S = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["streams"]
    T = PREFILL_TOKENS
    i32 = dict(dtype=torch.int32, device=dev)

    def timed(fn):
        ts = []
        for _ in range(6):
            flush.fill_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[1:])

    def context_of(q_lens, starts, slots):
        pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
        seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
        cu = torch.tensor([0] + [sum(q_lens[:i + 1]) for i in range(len(q_lens))], **i32)
        kv = [s + n for n, s in zip(q_lens, starts)]
        ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                          q_lens=list(q_lens), kv_lens=kv, slots=list(slots), max_q_len=max(q_lens), max_kv_len=max(kv),
                          token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                          kv_len_dev=torch.tensor(kv, **i32), slot_dev=torch.tensor(list(slots), **i32))
        ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
        tr = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
        ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(tr, **i32), len(ts))
        return ctx

    out = {}

    def note(name, ms, nbytes=0.0, flops=0.0, like=None):
        row = {"us": ms * 1e3}
        if nbytes:
            row["gbs"] = nbytes / (ms * 1e-3) / 1e9
            row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if flops:
            row["tflops"] = flops / (ms * 1e-3) / 1e12
            row["frac_bf16"] = row["tflops"] / pk["bf16_tflops"]
        if like:
            row["like"] = like
        out[name] = row

    n_slots = batch + 2
    own = Cache([CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0)], max_tokens=(batch + 1) * (context + 64),
                dtype=torch.bfloat16, device=dev, n_slots=n_slots)
    dense = Cache([CacheNeeds(kv_heads=2, head_dim=d)], max_tokens=(batch + 1) * (context + 64), dtype=torch.bfloat16, device=dev,
                  n_slots=n_slots)
    slots = []
    for c in (own, dense):
        slots = [c.open_sequence() for _ in range(batch)]
        for s_ in slots:
            c.reserve(s_, context)
        c.sync()
        c.lane(0).k.normal_(0, 0.5)
        c.lane(0).v.normal_(0, 0.5)
    E, top, ff = z["experts"], z["top"], z["ff"]
    DH, DG, dd, ddv, K = z["delta_heads"], z["delta_qk_heads"], z["delta_dim"], z["delta_vdim"], z["conv"]
    LH, ld, ldv = z["lin_heads"], z["lin_dim"], z["lin_vdim"]
    wg = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wu = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wd = torch.randn(E, W, ff, device=dev).bfloat16() * 0.02
    for phase, q_lens, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx = context_of(q_lens, starts, slots[:len(q_lens)])
        n = ctx.n_tokens
        keys = [s + j + 1 for nq, s in zip(q_lens, starts) for j in range(nq)]
        X = torch.randn(n, S, W, device=dev)
        y = torch.randn(n, W, device=dev).bfloat16()
        mix, vec, gain = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(1, device=dev)
        note(f"{phase}/hyper_step (write + read + norm)", timed(lambda: ops.hyper_step(X, (y, mix, vec), (vec, gain), 1e-5)),
             n * W * (8.0 * S + 4.0), like="add_rmsnorm")
        x1 = torch.randn(n, W, device=dev)
        wn = torch.ones(W, device=dev)
        note(f"{phase}/add_rmsnorm (dense model)", timed(lambda: ops.add_rmsnorm(x1, y, 1.0, wn, 1e-5)), n * W * 12.0)
        # attention whose weights are mixed across heads, beside the dense model's
        qkv = torch.randn(n, (H + G) * d + G * dv, device=dev).bfloat16()
        inv = torch.ones(d // 2, device=dev)
        ol = own.lane(0)
        note(f"{phase}/rope_store_dv", timed(lambda: ops.rope_store_dv(ctx, qkv, ol, H, G, d, dv, inv, d)),
             n * ((H + G) * d + G * dv) * 2.0 * 2, like="rope_store")
        q = torch.randn(n, H, d, device=dev).bfloat16()
        temp, talk = torch.ones(H, device=dev), torch.eye(H, device=dev)
        note(f"{phase}/talking_attention", timed(lambda: ops.talking_attention(ctx, q, ol, G, dv, d ** -0.5, temp, talk)),
             nbytes=(sum(s + nq for nq, s in zip(q_lens, starts)) * G * (d + dv) * 2.0) if phase == "decode" else 0.0,
             flops=2.0 * H * (d + dv) * sum(keys), like="attention")
        dl = dense.lane(0)
        qkv2 = torch.randn(n, (H + 4) * d, device=dev).bfloat16()
        note(f"{phase}/rope_store (dense model)",
             timed(lambda: ops.rope_store(qkv2, H, 2, d, ctx.positions, ctx.token_seq, ctx.slot_dev, dl.page_table, dl.k, dl.v, inv, 1.0, d)),
             n * (H + 4) * d * 2.0 * 2)
        note(f"{phase}/attention (dense model, 2 kv heads)", timed(lambda: ops.attention(ctx, q, dl, 2, d ** -0.5)),
             nbytes=(sum(s + nq for nq, s in zip(q_lens, starts)) * 2 * 2 * d * 2.0) if phase == "decode" else 0.0,
             flops=4.0 * H * d * sum(keys))
        # the two recurrences, beside the other recurrent design's scan
        C = 2 * DG * dd + DH * ddv
        proj = torch.randn(n, C + DH * ddv + 2 * DH, device=dev)
        taps = torch.randn(C, K, device=dev) * 0.3
        cstate = torch.zeros(n_slots, K - 1, C, device=dev)
        al, db = torch.zeros(DH, device=dev), torch.zeros(DH, device=dev)
        note(f"{phase}/conv_prepare", timed(lambda: ops.conv_prepare(ctx, proj, taps, cstate, al, db, C + DH * ddv, C + DH * ddv + DH, DH, DG, dd, ddv, 1e-6)),
             n * C * 8.0, like="rope_store")
        qd, kd, vd_, beta, decay = ops.conv_prepare(ctx, proj, taps, cstate, al, db, C + DH * ddv, C + DH * ddv + DH, DH, DG, dd, ddv, 1e-6)
        dstate = torch.zeros(n_slots, DH, dd, ddv, device=dev)
        state_bytes = len(q_lens) * DH * dd * ddv * 8.0
        note(f"{phase}/linear_recurrence (delta rule)",
             timed(lambda: ops.linear_recurrence(ctx, qd, kd, vd_, decay, beta, dstate, DH, DG, dd, ddv, dd ** -0.5)),
             nbytes=state_bytes + n * (2 * DG * dd + 2 * DH * ddv) * 4.0, flops=6.0 * n * DH * dd * ddv, like="mingru_scan")
        ql, kl, vl = torch.randn(n, LH * ld, device=dev), torch.randn(n, LH * ld, device=dev), torch.randn(n, LH * ldv, device=dev)
        al2 = torch.rand(n, LH * ld, device=dev) * 0.1 + 0.9
        lstate = torch.zeros(n_slots, LH, ld, ldv, device=dev)
        note(f"{phase}/linear_recurrence (decay per channel)",
             timed(lambda: ops.linear_recurrence(ctx, ql, kl, vl, al2, None, lstate, LH, LH, ld, ldv, ld ** -0.5, vector_decay=True)),
             nbytes=len(q_lens) * LH * ld * ldv * 8.0 + n * (3 * LH * ld + 2 * LH * ldv) * 4.0, flops=4.0 * n * LH * ld * ldv,
             like="mingru_scan")
        gp = torch.randn(n, 3 * W, device=dev)
        gstate = torch.zeros(n_slots, W, device=dev)
        note(f"{phase}/mingru_scan (other recurrent design)", timed(lambda: ops.mingru_scan(ctx, gp, wn, wn, gstate, W)), n * W * 14.0)
        o = torch.randn(n, DH, ddv, device=dev)
        wv = torch.ones(ddv, device=dev)
        note(f"{phase}/gated_head_norm", timed(lambda: ops.gated_head_norm(o, proj[:, C:C + DH * ddv], wv, 1e-5)), n * DH * ddv * 10.0,
             like="add_rmsnorm")
        a2, b2 = torch.randn(n, W, device=dev).bfloat16(), torch.randn(n, W, device=dev).bfloat16()
        note(f"{phase}/dual_rmsnorm_mean", timed(lambda: ops.dual_rmsnorm_mean(a2, b2, wn, wn, 1e-5)), n * W * 6.0, like="add_rmsnorm")
        # routed experts, beside the dense model's gated product of the same active size
        logits = torch.randn(n, E + 1, device=dev)
        corr = torch.zeros(E, device=dev)
        note(f"{phase}/moe_route", timed(lambda: ops.moe_route(logits, corr, E, top, z["groups"], z["keep"], E)), n * (E + 1) * 4.0)
        chosen, weights, gate = ops.moe_route(logits, corr, E, top, z["groups"], z["keep"], E)
        yy = torch.randn(n, W, device=dev).bfloat16()
        used = int(torch.unique(chosen).numel())
        note(f"{phase}/moe_experts (group + gate/up + down)", timed(lambda: ops.moe_experts(yy, chosen, wg, wu, wd)),
             nbytes=used * 3.0 * ff * W * 2.0 + n * top * (W + ff) * 4.0, flops=6.0 * n * top * ff * W, like="gate_up product + down")
        act = top * ff
        gu_w = torch.randn(2 * act, W, device=dev).bfloat16() * 0.02
        dn_w = torch.randn(W, act, device=dev).bfloat16() * 0.02
        note(f"{phase}/gate_up product + down of {act} (dense model)", timed(lambda: ops.linear(ops.gated_linear(yy, gu_w, 8, 0), dn_w)),
             nbytes=3.0 * act * W * 2.0 + n * (2 * W + act) * 2.0, flops=6.0 * n * act * W)
        pairs = ops.moe_experts(yy, chosen, wg, wu, wd)
        note(f"{phase}/moe_combine", timed(lambda: ops.moe_combine(pairs, weights, yy, gate)), n * W * 2.0 * (top + 2), like="add_rmsnorm")
    return out


def workload_mufevik(steps: int, warmup: int, size: str, batch: int) -> int:
    """Mufevik at one of MUFEVIK_SIZES beside MiniCPM4 with equal hidden size and heads, a feed-forward as large as a
    token's active experts (``top`` routed and the shared one) and as many layers: decode steps of ``batch`` sequences
    ending at a context of 4,096 tokens under a CUDA graph, a prompt of 2,048 tokens, and every kernel of the design
    alone beside its like."""
    import torch

    z, pk, context = MUFEVIK_SIZES[size], peaks(), CONTEXT
    cfg, model, cache, stepper = build_mufevik(z, batch * (context + 64) + 128, batch, context)
    runs = len(model.schedule)
    pre_ms = time_prefill_any(stepper, cfg.vocab)
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    del model, cache, stepper
    torch.cuda.empty_cache()
    active = z["top"] * z["ff"] + z["shared"]
    like = dict(MODEL, hidden_size=z["width"], intermediate_size=active, num_attention_heads=z["heads"], num_key_value_heads=2,
                head_dim=z["dim"], vocab_size=z["vocab"])
    dcfg, dmodel, dcache, dstepper = build_engine(runs, batch * (context + 64) + 128, batch, model=like, max_seq_tokens=context + 64)
    d_pre = time_prefill_any(dstepper, dcfg.vocab_size)
    d_ms, _, d_launches, d_cache = time_decode(dstepper, batch, steps, warmup, dcfg.vocab_size, False, context=context)
    d_weights = dmodel.weight_bytes_per_step()
    d_achieved = (d_weights + d_cache) / (d_ms * 1e-3) / 1e9
    del dmodel, dcache, dstepper
    torch.cuda.empty_cache()
    kernels = mufevik_kernels(z, pk, context, batch)
    print(json.dumps({
        "workload": "mufevik", "metric": f"decode tokens/s (Mufevik {size} sizes, bf16, batch {batch}, context {context})",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 5",
        "config": dict(z, size=size, layers=len(cfg.layers), global_batch=batch, seq_len=context, prefill_tokens=PREFILL_TOKENS,
                       cuda_graph=True, peaks=pk["source"]),
        "prefill": {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "ms": pre_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "weight_bytes": weight_bytes, "cache_bytes": cache_bytes,
                     "note": "weights of a step: every layer's mixer, router, shared expert and `top` experts per token of one sequence"},
        "closest_model": {"model": f"MiniCPM4 with hidden {z['width']}, intermediate {active}, {z['heads']} heads of {z['dim']}, 2 kv heads, {runs} layers",
                          "decode_tokens_s": batch * 1000.0 / d_ms, "ms_per_step": d_ms, "prefill_tokens_s": PREFILL_TOKENS / (d_pre * 1e-3),
                          "prefill_ms": d_pre, "roofline_frac": d_achieved / pk["hbm_gbs"], "weight_bytes": d_weights,
                          "cache_bytes": d_cache, "gpu_launches": d_launches},
        "kernels": kernels, "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


# Kipizen at the sizes of MUFEVIK_SIZES (the closest design: softmax attention, a matrix-state recurrence and routed
# experts): eight layers (lightning attention, two layers of window attention of which the second reads the first one's
# keys and values, lightning, ...); random weights N(0, 0.02), vectors 1 + N(0, 0.02).
KIPIZEN_WINDOW = 1024


def kipizen_config(z: dict) -> dict:
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"]}}
    H = z["lin_heads"]
    lin = {"type": "lightning", "mlp": mlp,
           "mixer": {"heads": H, "dim": z["lin_dim"], "vdim": z["lin_vdim"], "decay": [1.0 - 2.0 ** (-1 - 7 * i / max(1, H - 1)) for i in range(H)]}}

    def att(kv_from=None):
        m = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
             "softcap": 30.0, "mask": {"size": KIPIZEN_WINDOW}, "rot": {"dims": z["dim"] // 2, "base": 10000.0, "scaling": {"factor": 2.0}}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "attention", "mlp": mlp, "mixer": m}
    return {"architecture": "Kipizen", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "layers": [lin, att(), att(1), lin, lin, att(), att(5), lin]}


def build_kipizen(z: dict, max_tokens: int, max_batch: int, context: int):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    arch = architecture("Kipizen")
    cfg = arch.config_class.from_dict(kipizen_config(z))
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    storage = make_storage(model, PREFILL_TOKENS, max_batch, max_tokens=max_tokens, max_seq_tokens=context + 64, n_slots=max_batch + 2)
    model.load_weights(random_tensors(model.weight_specs(), 6, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0"))
    torch.cuda.empty_cache()
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=PREFILL_TOKENS, graph_prompts=True)


def kipizen_kernels(z: dict, pk: dict, context: int, batch: int) -> dict:
    """Every kernel of the design alone, at the size's shapes, beside the like kernel of the closest models (the dense
    attention with as many key-value heads, Mufevik's rotary store, recurrence with a decay per channel, head norm and
    routing): a prompt of 2,048 tokens and a decode step of ``batch`` sequences at ``context`` tokens.  CUDA events
    around one launch after a flush of L2 (a 512 MB buffer is written), median of five; bytes and FLOPs are the
    algorithmic ones (attention: the keys a window holds)."""
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds, QUERY_TILE_TOKENS, StepContext

    ops = Ops(torch.bfloat16)
    dev = "cuda:0"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    W, H, G, d, dv = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    T, win = PREFILL_TOKENS, KIPIZEN_WINDOW
    i32 = dict(dtype=torch.int32, device=dev)

    def timed(fn):
        ts = []
        for _ in range(6):
            flush.fill_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[1:])

    def context_of(q_lens, starts, slots):
        pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
        seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
        cu = torch.tensor([0] + [sum(q_lens[:i + 1]) for i in range(len(q_lens))], **i32)
        kv = [s + n for n, s in zip(q_lens, starts)]
        ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                          q_lens=list(q_lens), kv_lens=kv, slots=list(slots), max_q_len=max(q_lens), max_kv_len=max(kv),
                          token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                          kv_len_dev=torch.tensor(kv, **i32), slot_dev=torch.tensor(list(slots), **i32))
        ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
        tr = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
        ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(tr, **i32), len(ts))
        return ctx

    out = {}

    def note(name, ms, nbytes=0.0, flops=0.0, like=None):
        row = {"us": ms * 1e3}
        if nbytes:
            row["gbs"] = nbytes / (ms * 1e-3) / 1e9
            row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if flops:
            row["tflops"] = flops / (ms * 1e-3) / 1e12
            row["frac_bf16"] = row["tflops"] / pk["bf16_tflops"]
        if like:
            row["like"] = like
        out[name] = row

    n_slots = batch + 2
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0)], max_tokens=(batch + 1) * (context + 64),
                  dtype=torch.bfloat16, device=dev, n_slots=n_slots)
    slots = [cache.open_sequence() for _ in range(batch)]
    for s_ in slots:
        cache.reserve(s_, context)
    cache.sync()
    lane = cache.lane(0)
    lane.k.normal_(0, 0.5)
    lane.v.normal_(0, 0.5)
    E, top, ff = z["experts"], z["top"], z["ff"]
    LH, ld, ldv = z["lin_heads"], z["lin_dim"], z["lin_vdim"]
    wg = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wu = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wd = torch.randn(E, W, ff, device=dev).bfloat16() * 0.02
    for phase, q_lens, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx = context_of(q_lens, starts, slots[:len(q_lens)])
        n = ctx.n_tokens
        keys = [s + j + 1 for nq, s in zip(q_lens, starts) for j in range(nq)]
        seen = [min(k_, win) for k_ in keys]
        # window attention with capped scores and a sink, beside the dense attention over the same cache
        cols = (H + G) * d + G * dv
        proj = torch.randn(n, cols, device=dev)
        inv = torch.ones(d // 4, device=dev)
        bq, bk, bv = torch.zeros(H * d, device=dev), torch.zeros(G * d, device=dev), torch.zeros(G * dv, device=dev)
        note(f"{phase}/qk_prepare_store (bias, rotation, unit rms, store)",
             timed(lambda: ops.qk_prepare_store(ctx, proj, lane, H, G, d, dv, (bq, bk, bv), inv, d // 2, True, 1e-5)),
             n * cols * 6.0, like="rope_store_dv")
        qkv = torch.randn(n, cols, device=dev).bfloat16()
        inv2 = torch.ones(d // 2, device=dev)
        note(f"{phase}/rope_store_dv (Mufevik)", timed(lambda: ops.rope_store_dv(ctx, qkv, lane, H, G, d, dv, inv2, d)), n * cols * 4.0)
        lane.k.normal_(0, 0.5)
        q = torch.randn(n, H, d, device=dev).bfloat16()
        note(f"{phase}/sink_attention (window {win}, cap, sink)",
             timed(lambda: ops.sink_attention(ctx, q, lane, G, dv, d ** -0.5, win, 30.0, True)),
             nbytes=(len(q_lens) * min(context, win) * G * (d + dv) * 2.0) if phase == "decode" else 0.0,
             flops=2.0 * H * (d + dv) * sum(seen), like="attention")
        note(f"{phase}/sink_attention (no window: the keys of the dense kernel; cap, sink)",
             timed(lambda: ops.sink_attention(ctx, q, lane, G, dv, d ** -0.5, 0, 30.0, True)),
             nbytes=(sum(keys) * G * (d + dv) * 2.0) if phase == "decode" else 0.0,
             flops=2.0 * H * (d + dv) * sum(keys), like="attention")
        if d == dv:
            note(f"{phase}/attention (dense, {G} kv heads, no window)", timed(lambda: ops.attention(ctx, q, lane, G, d ** -0.5)),
                 nbytes=(sum(s + nq for nq, s in zip(q_lens, starts)) * G * 2 * d * 2.0) if phase == "decode" else 0.0,
                 flops=4.0 * H * d * sum(keys))
        # lightning attention, beside the recurrence with a decay per key channel
        width_in = 2 * LH * ld + 2 * LH * ldv
        lp = torch.randn(n, width_in, device=dev)
        note(f"{phase}/silu_columns", timed(lambda: ops.silu_columns(lp, 2 * LH * ld + LH * ldv)), n * (2 * LH * ld + LH * ldv) * 8.0,
             like="add_rmsnorm")
        ql, kl, vl = lp[:, :LH * ld], lp[:, LH * ld:2 * LH * ld], lp[:, 2 * LH * ld:2 * LH * ld + LH * ldv]
        dec = (torch.rand(LH, device=dev) * 0.1 + 0.9).unsqueeze(0).expand(n, LH)
        lstate = torch.zeros(n_slots, LH, ld, ldv, device=dev)
        rec_bytes = len(q_lens) * LH * ld * ldv * 8.0 + n * (2 * LH * ld + 2 * LH * ldv) * 4.0
        note(f"{phase}/linear_recurrence (one decay per head)",
             timed(lambda: ops.linear_recurrence(ctx, ql, kl, vl, dec, None, lstate, LH, LH, ld, ldv, 1.0)),
             nbytes=rec_bytes, flops=4.0 * n * LH * ld * ldv, like="linear_recurrence (decay per channel)")
        al2 = torch.rand(n, LH * ld, device=dev) * 0.1 + 0.9
        qc, kc, vc = (t.contiguous() for t in (ql, kl, vl))
        note(f"{phase}/linear_recurrence (decay per channel, Mufevik)",
             timed(lambda: ops.linear_recurrence(ctx, qc, kc, vc, al2, None, lstate, LH, LH, ld, ldv, ld ** -0.5, vector_decay=True)),
             nbytes=rec_bytes + n * LH * ld * 4.0, flops=4.0 * n * LH * ld * ldv)
        o = torch.randn(n, LH, ldv, device=dev)
        gate = lp[:, 2 * LH * ld + LH * ldv:]
        wall, wv = torch.ones(LH * ldv, device=dev), torch.ones(ldv, device=dev)
        note(f"{phase}/gated_group_norm (all heads, sigmoid gate)", timed(lambda: ops.gated_group_norm(o, gate, wall, 1e-5, LH, "sigmoid")),
             n * LH * ldv * 10.0, like="gated_head_norm")
        note(f"{phase}/gated_head_norm (Mufevik)", timed(lambda: ops.gated_head_norm(o, gate, wv, 1e-5)), n * LH * ldv * 10.0)
        # the residual and norm, and routed experts
        x1 = torch.randn(n, W, device=dev)
        y = torch.randn(n, W, device=dev).bfloat16()
        wn = torch.ones(W, device=dev)
        note(f"{phase}/add_rmsnorm (32-bit residual)", timed(lambda: ops.add_rmsnorm(x1, y, 1.0, wn, 1e-5)), n * W * 12.0)
        logits = torch.randn(n, E, device=dev)
        rb = torch.zeros(E, device=dev)
        note(f"{phase}/moe_route (largest logits, softmax over the chosen)",
             timed(lambda: ops.moe_route(logits, None, E, top, 1, 1, bias=rb, top_first=True)), n * E * 4.0, like="moe_route")
        logits1 = torch.randn(n, E + 1, device=dev)
        note(f"{phase}/moe_route (Mufevik: scores, groups, correction)",
             timed(lambda: ops.moe_route(logits1, rb, E, top, z["groups"], z["keep"], E)), n * (E + 1) * 4.0)
        chosen, weights, _ = ops.moe_route(logits, None, E, top, 1, 1, bias=rb, top_first=True)
        used = int(torch.unique(chosen).numel())
        note(f"{phase}/moe_experts (the kernels Mufevik uses)", timed(lambda: ops.moe_experts(y, chosen, wg, wu, wd)),
             nbytes=used * 3.0 * ff * W * 2.0 + n * top * (W + ff) * 4.0, flops=6.0 * n * top * ff * W)
        pairs = ops.moe_experts(y, chosen, wg, wu, wd)
        note(f"{phase}/moe_combine", timed(lambda: ops.moe_combine(pairs, weights, None, None)), n * W * 2.0 * (top + 1))
    return out


def workload_kipizen(steps: int, warmup: int, size: str, batch: int) -> int:
    """Kipizen at one of MUFEVIK_SIZES beside Mufevik at the same sizes (the closest design): decode steps of ``batch``
    sequences ending at a context of 4,096 tokens under a CUDA graph, a prompt of 2,048 tokens, and every kernel of the
    design alone beside its like."""
    import torch

    z, pk, context = MUFEVIK_SIZES[size], peaks(), CONTEXT
    cfg, model, cache, stepper = build_kipizen(z, batch * (context + 64) + 128, batch, context)
    pre_ms = time_prefill_any(stepper, cfg.vocab)
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    del model, cache, stepper
    torch.cuda.empty_cache()
    mcfg, mmodel, mcache, mstepper = build_mufevik(z, batch * (context + 64) + 128, batch, context)
    m_pre = time_prefill_any(mstepper, mcfg.vocab)
    m_ms, _, m_launches, m_cache = time_decode(mstepper, batch, steps, warmup, mcfg.vocab, False, context=context)
    m_weights = mmodel.weight_bytes_per_step()
    m_achieved = (m_weights + m_cache) / (m_ms * 1e-3) / 1e9
    del mmodel, mcache, mstepper
    torch.cuda.empty_cache()
    kernels = kipizen_kernels(z, pk, context, batch)
    print(json.dumps({
        "workload": "kipizen", "metric": f"decode tokens/s (Kipizen {size} sizes, bf16, batch {batch}, context {context})",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 6",
        "config": dict(z, size=size, layers=len(cfg.layers), window=KIPIZEN_WINDOW, global_batch=batch, seq_len=context,
                       prefill_tokens=PREFILL_TOKENS, cuda_graph=True, peaks=pk["source"]),
        "prefill": {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "ms": pre_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "weight_bytes": weight_bytes, "cache_bytes": cache_bytes},
        "closest_model": {"model": f"Mufevik at the {size} sizes, {len(mcfg.layers)} layers",
                          "decode_tokens_s": batch * 1000.0 / m_ms, "ms_per_step": m_ms, "prefill_tokens_s": PREFILL_TOKENS / (m_pre * 1e-3),
                          "prefill_ms": m_pre, "roofline_frac": m_achieved / pk["hbm_gbs"], "weight_bytes": m_weights,
                          "cache_bytes": m_cache, "gpu_launches": m_launches},
        "kernels": kernels, "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


# Lukelorn at the sizes of MUFEVIK_SIZES beside Kipizen at the same sizes (the closest design: window attention with capped
# scores and a sink, a matrix-state recurrence, routed experts): eight parallel layers (delta rule with a decay per key
# channel, window attention that keeps first tokens, the same layer's tensors once more with a cache of its own, latent
# attention with a rotated key part, ...); random weights N(0, 0.02), vectors N(0, 0.02) around their neutral value.
LUKELORN_WINDOW, LUKELORN_KEEP = 1024, 64
LUKELORN_LATENT = {"1k": dict(q_rank=384, kv_rank=192, rot_dim=32), "2k": dict(q_rank=768, kv_rank=448, rot_dim=64)}


def lukelorn_config(z: dict, lat: dict) -> dict:
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"]}}
    dense = {"kind": "dense", "ff": z["ff"] * z["top"]}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                     "softcap": 30.0, "mask": {"size": LUKELORN_WINDOW, "keep_first": LUKELORN_KEEP},
                     "rot": {"dims": z["dim"], "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    delta = {"type": "channel_delta", "mlp": moe,
             "mixer": {"heads": z["delta_heads"], "kv_heads": z["delta_qk_heads"], "dim": z["delta_dim"], "vdim": z["delta_vdim"],
                       "conv": z["conv"], "decay_rank": 32, "gate_rank": 32}}
    latent = {"type": "latent_attention", "mlp": dense,
              "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": lat["rot_dim"], "vdim": z["vdim"], "q_rank": lat["q_rank"],
                        "kv_rank": lat["kv_rank"], "scale": (z["dim"] + lat["rot_dim"]) ** -0.5, "mask": {"size": LUKELORN_WINDOW},
                        "rot": {"dims": lat["rot_dim"], "base": 10000.0}}}
    return {"architecture": "Lukelorn", "vocab": z["vocab"], "width": z["width"], "residual_mult": 0.5, "norm": {"eps": 1e-5},
            "layers": [delta, att, dict(att, weights_of=1), latent, delta, att, dict(att, weights_of=5), latent]}


def build_lukelorn(z: dict, lat: dict, max_tokens: int, max_batch: int, context: int):
    import torch
    from cpmcu_b200.engine import Stepper
    from cpmcu_b200.engine.storage import make_storage
    from cpmcu_b200.loading import build_model
    from cpmcu_b200.registry import architecture
    from cpmcu_b200.weights import random_tensors

    arch = architecture("Lukelorn")
    cfg = arch.config_class.from_dict(lukelorn_config(z, lat))
    model = build_model(arch, cfg, torch.bfloat16, "cuda:0")
    storage = make_storage(model, PREFILL_TOKENS, max_batch, max_tokens=max_tokens, max_seq_tokens=context + 64, n_slots=max_batch + 2)
    tensors = random_tensors(model.weight_specs(), 7, torch.bfloat16, std=0.02, norm_mean=1.0, device="cuda:0")
    for name, t in tensors.items():
        if name.endswith(("norm1", "final.norm", ".sink")):
            t.sub_(1.0)                                   # stored around zero
        elif name.endswith((".conv", ".A_log", ".dt_bias")):
            t.mul_(0.3)
    model.load_weights(tensors)
    del tensors
    torch.cuda.empty_cache()
    return cfg, model, storage.cache, Stepper(model, storage.cache, chunk_tokens=PREFILL_TOKENS, graph_prompts=True)


def lukelorn_kernels(z: dict, lat: dict, pk: dict, context: int, batch: int) -> dict:
    """Every kernel of the design alone, at the size's shapes, beside the like kernel of the closest models (Kipizen's
    window attention and its preparation, Mufevik's delta rule with a decay per head, Reravik's latent attention over a
    row of equal size, the gated experts): a prompt of 2,048 tokens and a decode step of ``batch`` sequences at
    ``context`` tokens.  CUDA events around one launch after a flush of L2 (a 512 MB buffer is written), median of five;
    bytes and FLOPs are the algorithmic ones (attention: the keys a window holds and the kept first tokens)."""
    import torch
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds, QUERY_TILE_TOKENS, StepContext

    ops = Ops(torch.bfloat16)
    dev = "cuda:0"
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    W, H, G, d, dv = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    T, win, keep = PREFILL_TOKENS, LUKELORN_WINDOW, LUKELORN_KEEP
    i32 = dict(dtype=torch.int32, device=dev)

    def timed(fn):
        ts = []
        for _ in range(6):
            flush.fill_(1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts[1:])

    def context_of(q_lens, starts, slots):
        pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
        seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
        cu = torch.tensor([0] + [sum(q_lens[:i + 1]) for i in range(len(q_lens))], **i32)
        kv = [s + n for n, s in zip(q_lens, starts)]
        ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                          q_lens=list(q_lens), kv_lens=kv, slots=list(slots), max_q_len=max(q_lens), max_kv_len=max(kv),
                          token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                          kv_len_dev=torch.tensor(kv, **i32), slot_dev=torch.tensor(list(slots), **i32))
        ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
        tr = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
        ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(tr, **i32), len(ts))
        return ctx

    out = {}

    def note(name, ms, nbytes=0.0, flops=0.0, like=None):
        row = {"us": ms * 1e3}
        if nbytes:
            row["gbs"] = nbytes / (ms * 1e-3) / 1e9
            row["frac_hbm"] = row["gbs"] / pk["hbm_gbs"]
        if flops:
            row["tflops"] = flops / (ms * 1e-3) / 1e12
            row["frac_bf16"] = row["tflops"] / pk["bf16_tflops"]
        if like:
            row["like"] = like
        out[name] = row

    n_slots = batch + 2
    R, QR, dr = lat["kv_rank"], lat["q_rank"], lat["rot_dim"]
    row = R + dr
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0),
                   CacheNeeds(kv_heads=1, head_dim=row, values=False)], max_tokens=(batch + 1) * (context + 64),
                  dtype=torch.bfloat16, device=dev, n_slots=n_slots)
    slots = [cache.open_sequence() for _ in range(batch)]
    for s_ in slots:
        cache.reserve(s_, context)
    cache.sync()
    lane, llane = cache.lane(0), cache.lane(1)
    lane.k.normal_(0, 0.5)
    lane.v.normal_(0, 0.5)
    llane.k.normal_(0, 0.5)
    E, top, ff = z["experts"], z["top"], z["ff"]
    DH, DG, dd, ddv, K = z["delta_heads"], z["delta_qk_heads"], z["delta_dim"], z["delta_vdim"], z["conv"]
    wg = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wu = torch.randn(E, ff, W, device=dev).bfloat16() * 0.02
    wd = torch.randn(E, W, ff, device=dev).bfloat16() * 0.02
    for phase, q_lens, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [context - 1] * batch)):
        ctx = context_of(q_lens, starts, slots[:len(q_lens)])
        n = ctx.n_tokens
        keys = [s + j + 1 for nq, s in zip(q_lens, starts) for j in range(nq)]
        seen = [min(k_, win + keep) for k_ in keys]
        seen_plain = [min(k_, win) for k_ in keys]
        # window attention: the preparation (adjacent pairs, no bias, no unit length) and the attention with kept first
        # tokens, learned sinks and the gate in its last step, beside the forms Kipizen runs
        cols = (H + G) * d + G * dv
        proj = torch.randn(n, cols + H, device=dev)
        inv = torch.ones(d // 2, device=dev)
        note(f"{phase}/qk_prepare_store (rotation of adjacent pairs, store)",
             timed(lambda: ops.qk_prepare_store(ctx, proj, lane, H, G, d, dv, (None, None, None), inv, d, False, 0.0, adjacent=True,
                                                extra_cols=H)), n * cols * 6.0, like="qk_prepare_store (Kipizen)")
        projk = torch.randn(n, cols, device=dev)
        bq, bk, bv = torch.zeros(H * d, device=dev), torch.zeros(G * d, device=dev), torch.zeros(G * dv, device=dev)
        inv4 = torch.ones(d // 4, device=dev)
        note(f"{phase}/qk_prepare_store (Kipizen: bias, rotation of half a head, unit rms, store)",
             timed(lambda: ops.qk_prepare_store(ctx, projk, lane, H, G, d, dv, (bq, bk, bv), inv4, d // 2, True, 1e-5)), n * cols * 6.0)
        lane.k.normal_(0, 0.5)
        q = torch.randn(n, H, d, device=dev).bfloat16()
        sinks = torch.randn(H, device=dev)
        gate = proj[:, cols:]
        note(f"{phase}/sink_attention (window {win}, {keep} kept first tokens, cap, learned sinks, gate)",
             timed(lambda: ops.sink_attention(ctx, q, lane, G, dv, d ** -0.5, win, 30.0, True, keep_first=keep, sinks=sinks, gate=gate)),
             nbytes=(len(q_lens) * min(context, win + keep) * G * (d + dv) * 2.0) if phase == "decode" else 0.0,
             flops=2.0 * H * (d + dv) * sum(seen), like="sink_attention (Kipizen)")
        note(f"{phase}/sink_attention (Kipizen: window {win}, cap, sink of score 0)",
             timed(lambda: ops.sink_attention(ctx, q, lane, G, dv, d ** -0.5, win, 30.0, True)),
             nbytes=(len(q_lens) * min(context, win) * G * (d + dv) * 2.0) if phase == "decode" else 0.0,
             flops=2.0 * H * (d + dv) * sum(seen_plain))
        # the delta rule with a decay per key channel beside Mufevik's with a decay per head
        C = 2 * DG * dd + DH * ddv
        dproj = torch.randn(n, C + 2 * DH + 64, device=dev)
        taps = torch.randn(C, K, device=dev) * 0.3
        cstate = torch.zeros(n_slots, max(K - 1, 1), C, device=dev)
        al, db, dbc = torch.zeros(DH, device=dev), torch.zeros(DH, device=dev), torch.zeros(DH * dd, device=dev)
        note(f"{phase}/conv_prepare (no decay)",
             timed(lambda: ops.conv_prepare(ctx, dproj, taps, cstate, al, db, C, 0, DH, DG, dd, ddv, 1e-6, head_decay=False)),
             n * C * 8.0, like="conv_prepare (Mufevik)")
        note(f"{phase}/conv_prepare (Mufevik: with the decay per head)",
             timed(lambda: ops.conv_prepare(ctx, dproj, taps, cstate, al, db, C, C + DH, DH, DG, dd, ddv, 1e-6)), n * C * 8.0)
        zlog = torch.randn(n, DH * dd, device=dev)
        note(f"{phase}/channel_decay", timed(lambda: ops.channel_decay(zlog, al, dbc, DH, dd)), n * DH * dd * 8.0, like="sigmoid_power (Mufevik)")
        note(f"{phase}/sigmoid_power (Mufevik)", timed(lambda: ops.sigmoid_power(zlog, dbc, 8.0)), n * DH * dd * 8.0)
        qd, kd, vd_, beta, hdecay = ops.conv_prepare(ctx, dproj, taps, cstate, al, db, C, C + DH, DH, DG, dd, ddv, 1e-6)
        cdecay = torch.rand(n, DH * dd, device=dev) * 0.1 + 0.9
        dstate = torch.zeros(n_slots, DH, dd, ddv, device=dev)
        rec_bytes = len(q_lens) * DH * dd * ddv * 8.0 + n * (2 * DG * dd + DH * ddv + DH * ddv) * 4.0
        note(f"{phase}/linear_recurrence (delta rule, decay per key channel)",
             timed(lambda: ops.linear_recurrence(ctx, qd, kd, vd_, cdecay, beta, dstate, DH, DG, dd, ddv, dd ** -0.5, vector_decay=True)),
             nbytes=rec_bytes + n * DH * dd * 4.0, flops=6.0 * n * DH * dd * ddv, like="linear_recurrence (Mufevik)")
        note(f"{phase}/linear_recurrence (Mufevik: delta rule, decay per head)",
             timed(lambda: ops.linear_recurrence(ctx, qd, kd, vd_, hdecay, beta, dstate, DH, DG, dd, ddv, dd ** -0.5)),
             nbytes=rec_bytes, flops=6.0 * n * DH * dd * ddv)
        o = torch.randn(n, DH, ddv, device=dev)
        og = torch.randn(n, DH * ddv, device=dev)
        wv = torch.ones(ddv, device=dev)
        note(f"{phase}/gated_head_norm (sigmoid gate)", timed(lambda: ops.gated_head_norm(o, og, wv, 1e-5, "sigmoid")),
             n * DH * ddv * 10.0, like="gated_head_norm (Mufevik)")
        note(f"{phase}/gated_head_norm (Mufevik)", timed(lambda: ops.gated_head_norm(o, og, wv, 1e-5)), n * DH * ddv * 10.0)
        # latent attention with a rotated key part beside Reravik's over a row of equal size
        down = torch.randn(n, QR + row + H, device=dev)
        gq, gkv, invr = torch.ones(QR, device=dev), torch.ones(R, device=dev), torch.ones(max(dr // 2, 1), device=dev)
        note(f"{phase}/latent_norm_store (with the rotated key part)",
             timed(lambda: ops.latent_norm_store(ctx, down, gq, gkv, llane, QR, R, 1e-5, rot_dim=dr, inv_freq=invr, adjacent=True)),
             n * (QR + row) * 6.0, like="latent_norm_store (Reravik)")
        note(f"{phase}/latent_norm_store (Reravik: a row of {row} values)",
             timed(lambda: ops.latent_norm_store(ctx, down, gq, gkv, llane, QR, row, 1e-5)), n * (QR + row) * 6.0)
        llane.k.normal_(0, 0.5)
        qf = torch.randn(n, H * (d + dr), device=dev)
        note(f"{phase}/rotate_heads", timed(lambda: ops.rotate_heads(ctx, qf, H, d, dr, invr, True)), n * H * (d + dr) * 6.0,
             like="rope_store_dv (Mufevik)")
        qkv = torch.randn(n, cols, device=dev).bfloat16()
        note(f"{phase}/rope_store_dv (Mufevik)", timed(lambda: ops.rope_store_dv(ctx, qkv, lane, H, G, d, dv, inv, d)), n * cols * 4.0)
        lane.k.normal_(0, 0.5)
        q_lat = torch.randn(n, H, row, device=dev)
        lkeys = [min(k_, win) for k_ in keys]
        note(f"{phase}/latent_attention (row {row} = rank {R} + rotated {dr}, window {win})",
             timed(lambda: ops.latent_attention(ctx, q_lat, llane, (d + dr) ** -0.5, win, out_compute_dtype=True)),
             nbytes=(len(q_lens) * min(context, win) * row * 2.0) if phase == "decode" else 0.0,
             flops=4.0 * H * row * sum(lkeys), like="the same kernel (Reravik's rows hold the latent alone)")
        oh = torch.randn(n, H * dv, device=dev).bfloat16()
        note(f"{phase}/head_gate", timed(lambda: ops.head_gate(oh, down[:, QR + row:], H)), n * H * dv * 4.0, like="silu_columns (Kipizen)")
        sc = torch.randn(n, H * dv, device=dev)
        note(f"{phase}/silu_columns (Kipizen)", timed(lambda: ops.silu_columns(sc, H * dv)), n * H * dv * 8.0)
        # the residual and norm, and the experts
        x1 = torch.randn(n, W, device=dev)
        y = torch.randn(n, W, device=dev).bfloat16()
        wn = torch.ones(W, device=dev)
        y2 = torch.randn(n, W, device=dev).bfloat16()
        note(f"{phase}/add_rmsnorm (32-bit residual, the two sublayers' outputs added in one pass)",
             timed(lambda: ops.add_rmsnorm(x1, y, 0.5, wn, 1e-5, delta2=y2)), n * W * 14.0, like="add_rmsnorm (Kipizen)")
        note(f"{phase}/add_rmsnorm (Kipizen: one output added)", timed(lambda: ops.add_rmsnorm(x1, y, 1.0, wn, 1e-5)), n * W * 12.0)
        logits = torch.randn(n, E, device=dev)
        rb = torch.zeros(E, device=dev)
        note(f"{phase}/moe_route (sigmoid scores)", timed(lambda: ops.moe_route(logits, None, E, top, 1, 1, sigmoid=True)), n * E * 4.0,
             like="moe_route (Kipizen)")
        note(f"{phase}/moe_route (Kipizen: largest logits, softmax over the chosen)",
             timed(lambda: ops.moe_route(logits, None, E, top, 1, 1, bias=rb, top_first=True)), n * E * 4.0)
        chosen, weights, _ = ops.moe_route(logits, None, E, top, 1, 1, sigmoid=True)
        used = int(torch.unique(chosen).numel())
        note(f"{phase}/moe_experts (up, relu squared, down; the weight on the input)",
             timed(lambda: ops.moe_experts(y, chosen, None, wu, wd, input_scale=weights)),
             nbytes=used * 2.0 * ff * W * 2.0 + n * top * (W + ff) * 4.0, flops=4.0 * n * top * ff * W, like="moe_experts (Kipizen)")
        note(f"{phase}/moe_experts (Kipizen: gate, up, down)", timed(lambda: ops.moe_experts(y, chosen, wg, wu, wd)),
             nbytes=used * 3.0 * ff * W * 2.0 + n * top * (W + ff) * 4.0, flops=6.0 * n * top * ff * W)
        pairs = ops.moe_experts(y, chosen, None, wu, wd, input_scale=weights)
        note(f"{phase}/moe_combine (plain sum)", timed(lambda: ops.moe_combine(pairs, None, None, None, top=top)), n * W * 2.0 * (top + 1),
             like="moe_combine (Kipizen)")
        note(f"{phase}/moe_combine (Kipizen: weighted)", timed(lambda: ops.moe_combine(pairs, weights, None, None)), n * W * 2.0 * (top + 1))
    return out


def workload_lukelorn(steps: int, warmup: int, size: str, batch: int) -> int:
    """Lukelorn at one of MUFEVIK_SIZES beside Kipizen at the same sizes (the closest design): decode steps of ``batch``
    sequences ending at a context of 4,096 tokens under a CUDA graph, a prompt of 2,048 tokens, and every kernel of the
    design alone beside its like."""
    import torch

    z, lat, pk, context = MUFEVIK_SIZES[size], LUKELORN_LATENT[size], peaks(), CONTEXT
    cfg, model, cache, stepper = build_lukelorn(z, lat, batch * (context + 64) + 128, batch, context)
    pre_ms = time_prefill_any(stepper, cfg.vocab)
    ms, clocks, launches, cache_bytes = time_decode(stepper, batch, steps, warmup, cfg.vocab, True, context=context)
    weight_bytes = model.weight_bytes_per_step()
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
    del model, cache, stepper
    torch.cuda.empty_cache()
    kcfg, kmodel, kcache, kstepper = build_kipizen(z, batch * (context + 64) + 128, batch, context)
    k_pre = time_prefill_any(kstepper, kcfg.vocab)
    k_ms, _, k_launches, k_cache = time_decode(kstepper, batch, steps, warmup, kcfg.vocab, False, context=context)
    k_weights = kmodel.weight_bytes_per_step()
    k_achieved = (k_weights + k_cache) / (k_ms * 1e-3) / 1e9
    del kmodel, kcache, kstepper
    torch.cuda.empty_cache()
    kernels = lukelorn_kernels(z, lat, pk, context, batch)
    print(json.dumps({
        "workload": "lukelorn", "metric": f"decode tokens/s (Lukelorn {size} sizes, bf16, batch {batch}, context {context})",
        "value": batch * 1000.0 / ms, "unit": "tokens/s", "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 7",
        "config": dict(z, **lat, size=size, layers=len(cfg.layers), window=LUKELORN_WINDOW, keep_first=LUKELORN_KEEP,
                       global_batch=batch, seq_len=context, prefill_tokens=PREFILL_TOKENS, cuda_graph=True, peaks=pk["source"]),
        "prefill": {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "ms": pre_ms},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "weight_bytes": weight_bytes, "cache_bytes": cache_bytes},
        "closest_model": {"model": f"Kipizen at the {size} sizes, {len(kcfg.layers)} layers",
                          "decode_tokens_s": batch * 1000.0 / k_ms, "ms_per_step": k_ms, "prefill_tokens_s": PREFILL_TOKENS / (k_pre * 1e-3),
                          "prefill_ms": k_pre, "roofline_frac": k_achieved / pk["hbm_gbs"], "weight_bytes": k_weights,
                          "cache_bytes": k_cache, "gpu_launches": k_launches},
        "kernels": kernels, "clocks": clocks, "gpu_launches": launches,
    }))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="layers built (the full model has 32)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--workload", default="dense8b", choices=["dense8b", "half_b", "sparse8b", "reravik", "mufevik", "kipizen", "lukelorn"],
                    help="dense8b: the headline line (8B sizes, batch 8, context 4096); half_b: 0.5B sizes, batch 64, prompts "
                         "uniform in [64, 2048] chunked at 512, decode at context 8192 (256 steps by default); sparse8b: 8B "
                         "sizes with InfLLM-v2, prompts of 16384 and 30000 tokens chunked at 2048, then decode steps; reravik: the Reravik "
                         "design at --size beside MiniCPM4 of equal sizes, and its kernels alone; mufevik: the same for the Mufevik design "
                         "(sizes 1k and 2k); kipizen: the Kipizen design beside Mufevik at the same sizes (1k and 2k), and its kernels alone; "
                         "lukelorn: the Lukelorn design beside Kipizen at the same sizes (1k and 2k), and its kernels alone")
    ap.add_argument("--size", default="2k", choices=sorted(RERAVIK_SIZES), help="--workload reravik / mufevik: which layer sizes")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the e2e run")
    ap.add_argument("--kernel", default=None, help="time one kernel alone: skinny_gemm, decode_attention, prefill_attention (tcgen05), prefill_attention_mma, gemm_tcgen05; or run eager steps of a 2-layer model for a launch list: decode_step, prefill_step")
    ap.add_argument("--ctx", type=int, default=CONTEXT, help="--kernel: cached tokens per sequence (or prompt tokens)")
    ap.add_argument("--rows", type=int, default=8, help="--kernel skinny_gemm / gemm_tcgen05: rows of the activation")
    ap.add_argument("--n", type=int, default=4096, help="--kernel skinny_gemm: output features")
    ap.add_argument("--k", type=int, default=4096, help="--kernel skinny_gemm: input features")
    ap.add_argument("--reps", type=int, default=5, help="--kernel: graph replays that are timed")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a.steps, a.warmup)
    if a.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    if a.kernel in ("decode_step", "prefill_step"):
        return step_launches(a.kernel, a.batch, a.ctx, a.layers if a.layers != FULL_LAYERS else 2, a.reps, a.workload)
    if a.workload == "half_b":
        return workload_half_b(a.steps if a.steps != 128 else 256, max(3, a.warmup))
    if a.workload == "sparse8b":
        return workload_sparse8b(a.steps, a.warmup, a.layers)
    if a.workload == "reravik":
        return workload_reravik(a.steps, max(3, a.warmup), a.size, a.batch)
    if a.workload == "mufevik":
        if a.size not in MUFEVIK_SIZES:
            print(f"bench.py: --workload mufevik takes --size {' or '.join(sorted(MUFEVIK_SIZES))}")
            return 2
        return workload_mufevik(a.steps, max(3, a.warmup), a.size, a.batch)
    if a.workload == "kipizen":
        if a.size not in MUFEVIK_SIZES:
            print(f"bench.py: --workload kipizen takes --size {' or '.join(sorted(MUFEVIK_SIZES))}")
            return 2
        return workload_kipizen(a.steps, max(3, a.warmup), a.size, a.batch)
    if a.workload == "lukelorn":
        if a.size not in MUFEVIK_SIZES:
            print(f"bench.py: --workload lukelorn takes --size {' or '.join(sorted(MUFEVIK_SIZES))}")
            return 2
        return workload_lukelorn(a.steps, max(3, a.warmup), a.size, a.batch)
    if a.kernel:
        return kernel_bench(a.kernel, a.batch, a.ctx, a.rows, a.n, a.k, a.reps)
    a.warmup = max(3, a.warmup)
    import torch
    from cpmcu_b200.ops import library

    pk = peaks()
    max_batch = a.batch if a.no_points else max(64, a.batch)
    cfg, model, cache, stepper = build_engine(a.layers, max_batch * (CONTEXT + 64) + 128, max_batch)
    weight_bytes = model.weight_bytes_per_step()

    ms, clocks, launches, cache_bytes = time_decode(stepper, a.batch, a.steps, a.warmup, cfg.vocab_size, True)
    value = a.batch * 1000.0 / ms
    achieved = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9

    pre_ms = time_prefill(stepper, cfg)
    flops = prefill_flops(cfg, a.layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}
    if "bf16_tflops_sustained" in pk:       # the step is 32 layers long: the peak under the power cap, beside the burst peak
        prefill["frac_sustained"] = flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12)

    points, e2e = {}, None
    if not a.no_points:
        for b in (1, 64):
            pms, _, _, _ = time_decode(stepper, b, min(a.steps, 64), a.warmup, cfg.vocab_size)
            points[f"decode_b{b}"] = b * 1000.0 / pms
        e2e = time_e2e(cfg, stepper, a.steps, a.batch)

    line = {
        "metric": "decode tokens/s (MiniCPM4-8B sizes, bf16, batch 8, context 4096)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random weights N(0,0.02) seed 2",
        "impl": "ours",
        "config": {
            "model": "MiniCPM4-8B sizes", "layers": a.layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
            "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": a.batch,
            "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "rope": "longrope", "attention": "dense", "l2": "inputs larger than L2 (weights read per step)",
            "peaks": pk["source"], "cuda_graph": True,
        },
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clocks,
        "gpu_launches": launches,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
