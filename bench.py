"""Headline measurement: decode tokens per second of the Qwen3-8B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A *step* is one decode step: every live request advances by one token (model
forward over the paged cache, greedy sampling on the device, one copy of the
tokens back).  The default run has the layer sizes of Qwen3-8B with seeded
random bfloat16 weights, a batch of 8 and a context that ends at 4,096 tokens.
It prints ONE JSON line:

  value      decoded tokens per second at the default batch, timed with CUDA events
  e2e        the same through ``LLM.generate`` (host token ids in, host token ids out)
  prefill    one 2,048-token prompt in one step: tokens/s, ms, fraction of the bf16 peak
  roofline   bytes the decode step must read (weights once + live cache) / its time
  points     decode tokens per second at batch 1 and 64
  clocks     SM clocks and throttle reasons sampled during the timed regions

The engine runs on one GPU only: for ``--gpus N`` with N > 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 40960,
}
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40,
                 intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600)
SIZES = {"8b": ("Qwen3-8B", QWEN3_8B), "14b": ("Qwen3-14B", QWEN3_14B), "32b": ("Qwen3-32B", QWEN3_32B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PROMPT_PORTION = PREFILL_TOKENS
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in the background, sampling clocks and throttle reasons (reading only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.file = None

    def start(self) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def bench_config(model_name: str, raw: dict, layers_of_model: int, batch: int, ctx: int, pf_tokens: int,
                 peaks_source: str) -> dict:
    """The ``config`` record of the bench line: every size, flat.  Both arms (this engine and the
    reference) print the same record for the same run."""
    return {
        "model": f"{model_name} layer sizes", "layers": raw["num_hidden_layers"], "layers_of_model": layers_of_model,
        "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"],
        "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
        "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "rope_theta": raw["rope_theta"],
        "rms_norm_eps": raw["rms_norm_eps"], "tied_head": bool(raw.get("tie_word_embeddings", False)),
        "global_batch": batch, "seq_len": ctx, "prefill_tokens": pf_tokens, "kv_block": 16,
        "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read every step)",
        "peaks": peaks_source,
    }


def weight_bytes(core) -> int:
    """Bytes of every weight a decode step reads once, as the model's parts report them (the
    embedding table is read by row only and reports nothing)."""
    return core.model.step_weight_bytes()


def step_flops(cfg, n_layers: int, tokens: int, ctx_start: int = 0) -> float:
    """Multiply-adds of a step of ``tokens`` new tokens of one request, counted as 2 flops."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    per_layer = 2.0 * tokens * (h * (hq + 2 * hkv) * d + hq * d * h + 3 * h * inter)
    # causal attention: token i sees ctx_start + i + 1 keys; QK^T and PV
    keys = tokens * ctx_start + tokens * (tokens + 1) / 2
    per_layer += 2.0 * 2.0 * keys * hq * d
    return n_layers * per_layer + 2.0 * 1 * h * cfg["vocab_size"]


def fill_context(core, req_ids, length: int, vocab: int, seed: int) -> None:
    """Put ``length`` random tokens of every request into the cache, in prompts and prompt
    portions of ``PROMPT_PORTION`` tokens a step (2,048 unless ``--prompt-tokens`` says otherwise)."""
    import torch
    from tokamak_b200.engine.step import StepEntry
    gen = torch.Generator().manual_seed(seed)
    for rid in req_ids:
        toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
        for s in range(0, length, PROMPT_PORTION):
            core.step.run([StepEntry(rid, toks[s:s + PROMPT_PORTION], [])], check=False)
    core.step.check_errors()


def time_decode(core, batch: int, steps: int, warmup: int, ctx_end: int, vocab: int, sampling=None):
    """Device time of ``steps`` decode steps of ``batch`` requests whose context ends at ``ctx_end``.

    The steps run as generation runs them: each request's token, position and sampling state
    are in its slot record on the device, the step is replayed from a CUDA graph, and it is
    launched one ahead, before the host has read the step before it; every step's tokens still
    come back to the host.  Afterwards the same requests are rewound and the same steps run
    again kernel by kernel, without graphs and without launching ahead: the tokens must be the
    same, or the timed path computed something else than the plain path."""
    import torch
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    step = core.step
    req_ids = [f"b{batch}_{i}" for i in range(batch)]
    start_len = ctx_end - (steps + warmup + 1)
    for rid in req_ids:
        # greedy, or (temperature, top_k, top_p) with a seed per request
        step.admit(rid, SamplingRow() if sampling is None else
                   SamplingRow(temperature=sampling[0], top_k=int(sampling[1]), top_p=sampling[2], seed=1 + len(rid)))
    fill_context(core, req_ids, start_len - 1, vocab, seed=batch)
    last = [1 + i for i in range(batch)]
    # the last prompt token of every request, sampled: from here on the records carry the requests
    first = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, last)])
    entries = [StepEntry(r, None, [0]) for r in req_ids]
    produced = [first]

    flight = step.launch_and_sample(entries)

    def one_step():
        nonlocal flight
        ahead = step.launch_and_sample(entries)
        produced.append(step.collect(flight))
        flight = ahead

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES + step.graph_launches
    h2d0, d2h0 = step.buffers.h2d_bytes, step.buffers.d2h_bytes
    t_host = time.perf_counter()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    produced.append(step.collect(flight))
    ms = begin.elapsed_time(end)
    wall = time.perf_counter() - t_host
    launches = ops.LAUNCHES + step.graph_launches - launches0
    h2d, d2h = step.buffers.h2d_bytes - h2d0, step.buffers.d2h_bytes - d2h0
    kv_bytes = batch * (ctx_end - steps / 2.0) * core.cache.bytes_per_token()

    # the check: rewind every request to where the records took over and decode again, plainly
    replays = step.graph_replays
    for rid in req_ids:
        if sampling is None:
            step.restart(rid)
        else:           # a restarted request keeps its generator's count, as after a preemption: begin anew instead
            step.free(rid)
            step.admit(rid, SamplingRow(temperature=sampling[0], top_k=int(sampling[1]), top_p=sampling[2],
                                        seed=1 + len(rid)))
    fill_context(core, req_ids, start_len - 1, vocab, seed=batch)
    graphs, step.use_graphs = step.use_graphs, False
    toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, last)])
    checked = toks == produced[0]
    for want in produced[1:]:
        toks = step.run_and_sample([StepEntry(r, [t], [0]) for r, t in zip(req_ids, toks)])
        checked = checked and toks == want
    step.use_graphs = graphs
    assert step.graph_replays == replays
    for r in req_ids:
        step.free(r)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
            "kv_bytes": kv_bytes, "wall_ms_per_step": wall * 1e3 / steps, "checked": checked,
            "graph_replays": replays, "h2d_bytes_per_step": h2d / steps, "d2h_bytes_per_step": d2h / steps}


def time_prefill(core, vocab: int, tokens: int = PREFILL_TOKENS, repeats: int = 3):
    import torch
    from tokamak_b200.engine.step import StepEntry
    gen = torch.Generator().manual_seed(99)
    times = []
    for i in range(repeats + 1):
        toks = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
        rid = f"prefill{i}"
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        core.step.run([StepEntry(rid, toks, [tokens - 1])], check=False)
        end.record()
        torch.cuda.synchronize()
        core.step.free(rid)
        if i > 0:
            times.append(begin.elapsed_time(end))
    core.step.check_errors()
    return statistics.median(times)


def time_e2e(core, batch: int, steps: int, warmup: int, ctx_end: int, vocab: int):
    """Decode tokens per second through ``LLM.generate``: host token ids in and out."""
    import torch
    from tokamak_b200 import LLM, SamplingParams
    # a budget that takes every prompt in one step, so that all requests decode together
    llm = LLM("<random>", _core=core, max_batch_size=batch, max_num_batched_tokens=batch * ctx_end,
              block_size=core.page_size)
    gen = torch.Generator().manual_seed(7)
    # the prompts of all requests are prefilled in one burst under the power cap, and the first
    # two dozen decode steps after it run at clocks that are still recovering (5.4, 4.7, 4.2 ms,
    # then 3.8 ms per step at batch 8): they count as warm-up here
    warmup = max(warmup, 32)
    new_tokens = steps + warmup + 1
    prompt_len = ctx_end - new_tokens
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in range(batch)]
    params = SamplingParams(temperature=0.0, max_new_tokens=new_tokens, ignore_eos=True)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert all(len(o.output_token_ids) == new_tokens for o in outs)
    times = llm.last_stats["decode_step_times"]
    assert len(times) >= steps + warmup, "the requests did not decode together"
    full = times[-steps:]                         # the last K decode steps, all at full batch
    tok_s = batch * len(full) / sum(full)
    # bytes copied to the device in those steps, counted from the copies the step function made: a
    # decode step's description lives in the slot records on the device, so what is copied is the
    # block-table entries of new pages (a new page every 16 tokens of a request) and, when the set
    # of running requests changes, the list of their slots
    h2d = sum(llm.last_stats["decode_step_h2d_bytes"][-steps:]) / len(full)
    d2h = 4 * (4 + batch)
    return {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": round(h2d, 1), "d2h_bytes_per_step": d2h,
            "ms_per_step": 1e3 * sum(full) / len(full), "warmup_steps": warmup}


QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960,
}


def throughput_requests(num_requests: int, max_new_cap: int, seed: int, vocab: int):
    """The requests of the reference's throughput benchmark (benchmarks/workload.py:23-48): prompt
    lengths log-normal(5.0, 0.7) clipped to 16..512, new tokens 8 + exponential(mean 120) capped,
    random token ids folded below the first special token.  The draws are made in the
    reference's order, so that the default arguments give its 4,915 prompt and 2,901 output tokens."""
    import random
    rng = random.Random(seed)
    prompts, new_tokens = [], []
    for _ in range(num_requests):
        length = int(min(max(rng.lognormvariate(5.0, 0.7), 16), 512))
        new_tokens.append(min(int(rng.expovariate(1 / 120)) + 8, max_new_cap))
        prompts.append([rng.randrange(vocab) % 151_643 for _ in range(length)])
    return prompts, new_tokens


def throughput_workload(sizes: str, num_requests: int, max_new_cap: int, batch: int, pool_tokens: int,
                        seed: int) -> dict:
    """Output tokens per second of ``LLM.generate`` over the reference's 32-request workload
    (benchmarks/benchmark_throughput.py:31-68: continuous batching, EOS ignored, greedy)."""
    import torch
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.engine.core import random_core
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else QWEN3_8B)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=1024, page_size=16,
                       pool_tokens=pool_tokens, max_slots=batch, max_step_tokens=2048)
    llm = LLM("<random>", _core=core, max_batch_size=batch, max_num_batched_tokens=2048, block_size=16)
    prompts, new_tokens = throughput_requests(num_requests, max_new_cap, seed, raw["vocab_size"])
    params = [SamplingParams(temperature=0.0, max_new_tokens=n, ignore_eos=True) for n in new_tokens]
    llm.generate(prompt_token_ids=prompts, sampling_params=params)          # warm-up: graphs, allocator
    runs = []                  # the median of three runs, as the reference reports (benchmarks/README.md:3-5)
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
        torch.cuda.synchronize()
        runs.append((time.perf_counter() - t0, outs, dict(llm.last_stats)))
    runs.sort(key=lambda r: r[0])
    wall, outs, stats = runs[1]
    n_out = sum(len(o.output_token_ids) for o in outs)
    ttft = sorted(o.ttft_s for o in outs)
    lat = sorted(o.latency_s for o in outs)
    return {"workload": "throughput (reference's 32 seeded requests)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "requests": num_requests, "prompt_tokens": sum(len(p) for p in prompts), "output_tokens": n_out,
            "max_batch_size": batch, "kv_pool_tokens": pool_tokens, "output_tok_s": round(n_out / wall, 1),
            "wall_s": round(wall, 3), "wall_s_runs": [round(r[0], 3) for r in runs], "ttft_mean_s": round(sum(ttft) / len(ttft), 4),
            "ttft_p99_s": round(ttft[-1], 4), "latency_mean_s": round(sum(lat) / len(lat), 4),
            "steps": stats["steps"], "mixed_steps": stats["mixed_steps"],
            "preemptions": stats["preemptions"], "dtype": "bf16", "data": "synthetic"}


def mixed_workload(sizes: str, num_requests: int, new_tokens: int, chunk: int, seed: int) -> dict:
    """A mixed batch through ``LLM.generate``: ``num_requests`` requests with prompt lengths uniform
    in 128..4,096, all submitted at once, prompts computed in portions of ``chunk`` tokens beside the
    decode tokens of the requests that already run, ``new_tokens`` greedy tokens each, context limit
    8,192.  Every request runs from the start (a pool for all of them), so all but the first steps
    are mixed steps until the last prompt is done."""
    import random
    import torch
    from tokamak_b200 import LLM, SamplingParams
    from tokamak_b200.engine.core import random_core
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else SIZES[sizes][1])
    rng = random.Random(seed)
    lengths = [rng.randint(128, 4096) for _ in range(num_requests)]
    prompts = [[rng.randrange(raw["vocab_size"]) for _ in range(n)] for n in lengths]
    pool = sum(-(-(n + new_tokens) // 16) * 16 for n in lengths)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=8192, page_size=16,
                       pool_tokens=max(pool, 8192), max_slots=num_requests,
                       max_step_tokens=chunk + num_requests)
    llm = LLM("<random>", _core=core, max_batch_size=num_requests, max_num_batched_tokens=chunk + num_requests,
              prefill_chunk=chunk, block_size=16)
    params = SamplingParams(temperature=0.0, max_new_tokens=new_tokens, ignore_eos=True)
    llm.generate(prompt_token_ids=prompts, sampling_params=params)          # warm-up
    runs = []
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
        torch.cuda.synchronize()
        runs.append((time.perf_counter() - t0, outs, dict(llm.last_stats)))
    runs.sort(key=lambda r: r[0])
    wall, outs, stats = runs[1]
    n_out = sum(len(o.output_token_ids) for o in outs)
    ttft = sorted(o.ttft_s for o in outs)
    return {"workload": "mixed batch (prompt portions beside decode tokens)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "requests": num_requests, "prompt_tokens": sum(lengths), "output_tokens": n_out,
            "prefill_chunk": chunk, "max_seq_len": 8192, "kv_pool_tokens": max(pool, 8192),
            "total_tok_s": round((sum(lengths) + n_out) / wall, 1), "output_tok_s": round(n_out / wall, 1),
            "wall_s": round(wall, 3), "wall_s_runs": [round(r[0], 3) for r in runs],
            "ttft_mean_s": round(sum(ttft) / len(ttft), 4), "ttft_max_s": round(ttft[-1], 4),
            "steps": stats["steps"], "mixed_steps": stats["mixed_steps"], "preemptions": stats["preemptions"],
            "dtype": "bf16", "data": "synthetic"}


def latency_workload(sizes: str, prompt_tokens: int, new_tokens: int, iters: int, seed: int) -> dict:
    """Single-sequence latency as the reference measures it (benchmarks/benchmark_latency.py:63-97,
    119-133): one seeded random prompt, time to the first token (prefill, argmax on the host side
    of a sync), then greedy steps one by one with the token read back every step; medians of
    ``iters`` runs after a warm-up."""
    import torch
    from tokamak_b200.engine.core import random_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    raw = dict(QWEN3_0_6B if sizes == "0.6b" else SIZES[sizes][1])
    total = prompt_tokens + new_tokens
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=total, page_size=16,
                       pool_tokens=2 * total, max_slots=2, max_step_tokens=max(prompt_tokens, 64))
    gen = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, raw["vocab_size"], (prompt_tokens,), generator=gen).tolist()

    def run_once(i: int) -> tuple[float, float]:
        rid = f"lat{i}"
        core.step.admit(rid, SamplingRow())
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        token = core.step.run_and_sample([StepEntry(rid, prompt, [prompt_tokens - 1])])[0]
        t1 = time.perf_counter()
        for _ in range(new_tokens):
            token = core.step.run_and_sample([StepEntry(rid, None, [0])])[0]
        t2 = time.perf_counter()
        core.step.free(rid)
        return (t1 - t0) * 1e3, new_tokens / (t2 - t1)

    run_once(-1)
    runs = [run_once(i) for i in range(iters)]
    prefill_ms = statistics.median(r[0] for r in runs)
    tok_s = statistics.median(r[1] for r in runs)
    return {"workload": "latency (reference's single-sequence measurement)", "sizes": f"Qwen3-{sizes.upper()} layer sizes",
            "prompt_tokens": prompt_tokens, "new_tokens": new_tokens, "prefill_ms": round(prefill_ms, 3),
            "prefill_tok_s": round(prompt_tokens / (prefill_ms / 1e3), 1), "decode_tok_s": round(tok_s, 1),
            "inter_token_ms": round(1e3 / tok_s, 3), "iters": iters, "dtype": "bf16", "data": "synthetic"}


def kernel_case(name: str, batch: int, ctx: int, iters: int, peaks: dict, portion: int = 0, sizes: str = "8b",
                sampling=None) -> dict:
    """One kernel alone on inputs larger than L2, timed with CUDA events: achieved bytes or flops
    per second against the peak.  Also the small case that ncu captures are made on."""
    import torch
    from tokamak_b200.csrc import ops
    dev = "cuda"
    cfg = SIZES[sizes][1] if sizes in SIZES else QWEN3_8B
    hq, hkv, d, page = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], 16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    flops = 0.0
    if name in ("attention_decode", "attention_decode_split", "attention_prefill", "attention_prefill_mma"):
        pages_per_req = -(-ctx // page)
        num_pages = batch * pages_per_req
        kc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
        vc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
        table = torch.randperm(num_pages, device=dev, generator=gen).to(torch.int32).view(batch, pages_per_req)
        slots = i32(list(range(batch)))
        if name in ("attention_decode", "attention_decode_split"):
            q = torch.randn((batch, hq, d), device=dev, generator=gen).bfloat16()
            out = torch.empty_like(q)
            items, tok_req = i32(list(range(batch))), i32(list(range(batch)))
            positions = i32([ctx - 1] * batch)
            if name == "attention_decode":          # the kernel the engine uses: key tiles dealt out evenly
                blocks = ops.decode_balanced_blocks(q.device, batch, hkv, ctx)
                run = lambda: ops.attention_decode_balanced(q, out, kc, vc, items, positions, tok_req, slots, table,
                                                            err, scale=d ** -0.5, window=None, blocks=blocks)
            else:                                   # the same number of splits for every (token, kv head)
                n_splits = ops.decode_splits(batch, hkv, ctx)
                scratch = torch.empty(batch * hq * n_splits * (d + 2), dtype=torch.float32, device=dev)
                run = lambda: ops.attention_decode(q, out, kc, vc, items, positions, tok_req, slots, table, err,
                                                   scale=d ** -0.5, window=None, n_splits=n_splits, scratch=scratch)
            nbytes = 2 * kc.numel() * 2 + 2 * q.numel() * 2
        else:
            qn = min(portion or ctx, ctx)         # query tokens of every request: the end of its context
            q = torch.randn((batch * qn, hq, d), device=dev, generator=gen).bfloat16()
            out = torch.empty_like(q)
            q_start, q_len, kv_len = [r * qn for r in range(batch)], [qn] * batch, [ctx] * batch
            if name == "attention_prefill_mma":
                tiles = [(r, t) for t in reversed(range(-(-qn // 64))) for r in range(batch)]
                tiles_t = i32([x for rt in tiles for x in rt])
                args = (i32(q_start), i32(q_len), i32(kv_len))
                run = lambda: ops.attention_prefill(q, out, kc, vc, tiles_t, *args, slots, table, err,
                                                    scale=d ** -0.5, window=None)
            else:
                records, n_parts, n_split = ops.prefill_tc_records(q_start, q_len, kv_len, list(range(batch)),
                                                                    heads=hq, sms=ops.sm_count(q.device))
                items = ops.PrefillItems(torch.from_numpy(records).to(dev), n_parts, n_split)
                run = lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=None)
            nbytes = 2 * kc.numel() * 2 + 2 * q.numel() * 2
            flops = batch * 2.0 * 2.0 * (qn * (ctx - qn) + qn * (qn + 1) / 2) * hq * d
    elif name == "rope_kv":
        # q/k norm + rotation + cache write for `batch` tokens of one request (prefill shape)
        n = batch
        pages = -(-n // page)
        kc = torch.zeros((pages, hkv, page, d), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        qkv = torch.randn((n, (hq + 2 * hkv) * d), device=dev, generator=gen).bfloat16()
        q_out = torch.empty((n, hq, d), dtype=torch.bfloat16, device=dev)
        positions = torch.arange(n, dtype=torch.int32, device=dev)
        tok_req = torch.zeros(n, dtype=torch.int32, device=dev)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        wq, wk = torch.ones(d, device=dev), torch.ones(d, device=dev)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(positions, inv_freq)
        slot0, len_n = i32([0]), i32([n])      # made once: a tensor from a host list is a blocking copy
        run = lambda: ops.rope_kv(qkv, q_out, kc, vc, positions, tok_req, slot0, table, wq, wk, rot, err,
                                  n_q_heads=hq, n_kv_heads=hkv, head_dim=d, rotary_dim=d, eps=1e-6,
                                  req_q_len=len_n, req_kv_len=len_n)
        nbytes = qkv.numel() * 2 + q_out.numel() * 2 + 2 * n * hkv * d * 2
    elif name == "sampling":
        # one token per row of float32 logits at the model's vocabulary; --sampling gives temperature,top_k,top_p
        n, vocab = batch, cfg["vocab_size"]
        t_, k_, p_ = sampling if sampling is not None else (0.8, 0, 0.95)
        logits = torch.randn((n, vocab), device=dev, generator=gen) * 3
        out_tok = torch.zeros(n, dtype=torch.int32, device=dev)
        temp = torch.full((n,), float(t_), device=dev)
        top_k = torch.full((n,), int(k_), dtype=torch.int32, device=dev)
        top_p = torch.full((n,), float(p_), device=dev)
        seeds = torch.arange(n, dtype=torch.int64, device=dev)
        counters = torch.zeros(n, dtype=torch.int32, device=dev)
        run = lambda: ops.sample(logits, temp, top_k, top_p, seeds, counters, out_tok)
        nbytes = n * vocab * 4          # one reading of the row; a top-k or top-p threshold reads it four times more each
    elif name == "rmsnorm":
        n, h = batch, cfg["hidden_size"]
        resid = torch.randn((n, h), device=dev, generator=gen)
        delta = torch.randn((n, h), device=dev, generator=gen).bfloat16()
        w = torch.ones(h, device=dev)
        out = torch.empty((n, h), dtype=torch.bfloat16, device=dev)
        run = lambda: ops.add_rmsnorm(resid, delta, w, out, 1e-6)
        nbytes = n * h * (4 + 2 + 4 + 2)
    elif name == "gemm_tc_decode":
        # the engine's own decode product: gate_up of one layer on tcgen05, weight as the row operand
        w = torch.randn((2 * cfg["intermediate_size"], cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        ws = [w.clone() for _ in range(4)]
        x = torch.randn((batch, cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        splits, stages, cluster = ops.swapped_gemm_plan(w.shape[0], w.shape[1], batch)
        out = torch.empty((splits // cluster if cluster > 1 else splits, batch, w.shape[0]),
                          dtype=torch.float32, device=dev)
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(ws)
            ops.gemm_tc_swapped(ws[turn[0]], x, err, splits, out=out, max_stages=stages, cluster=cluster)
        nbytes = w.numel() * 2
    elif name == "gemm_decode":
        # the library product the decode step uses, for comparison: gate_up of one layer
        w = torch.randn((2 * cfg["intermediate_size"], cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        ws = [w.clone() for _ in range(4)]          # rotate over copies so that L2 holds none of them
        x = torch.randn((batch, cfg["hidden_size"]), device=dev, generator=gen).bfloat16()
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(ws)
            torch.mm(x, ws[turn[0]].t())
        nbytes = w.numel() * 2
    elif name in ("products_chain", "products_separate"):
        # the four products between two attentions of a decode step (output, gate/up, down, the next
        # q|k|v, each with its fused epilogue) for `batch` tokens: as one persistent kernel, or one by one
        h, inter = cfg["hidden_size"], cfg["intermediate_size"]
        mk = lambda *shape, s=1.0: (torch.randn(*shape, device=dev, generator=gen) * s).bfloat16()
        sets = [dict(o=mk(h, hq * d, s=0.02), gu=mk(2 * inter, h, s=0.02), dn=mk(h, inter, s=0.02),
                     qkv=mk((hq + 2 * hkv) * d, h, s=0.02)) for _ in range(3)]      # rotated: none stays in L2
        x0 = mk(batch, hq * d)
        n1, n2 = torch.ones(h, device=dev), torch.ones(h, device=dev)
        qn, kn = torch.ones(d, device=dev), torch.ones(d, device=dev)
        resid = torch.zeros(batch, h, device=dev)
        pages = 4
        kc = torch.zeros((pages, hkv, page, d), dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        q = torch.zeros((batch, hq, d), dtype=torch.bfloat16, device=dev)
        positions = torch.arange(batch, dtype=torch.int32, device=dev) % (pages * page)
        tok_req, slot0 = torch.zeros(batch, dtype=torch.int32, device=dev), i32([0])
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(positions, inv_freq)
        plan = lambda w: ops.swapped_gemm_plan(w.shape[0], w.shape[1], batch)
        turn = [0]
        def run():
            turn[0] = (turn[0] + 1) % len(sets)
            w = sets[turn[0]]
            c = ops.ProductChain(batch, err) if name == "products_chain" else None
            resid.zero_()
            s_, st, cl = plan(w["o"])
            xb1, ss1 = ops.gemm_tc_swapped(w["o"], x0, err, s_, max_stages=st, cluster=cl, residual_norm=(resid, n1), chain=c)
            s_, st, cl = plan(w["gu"])
            act = ops.gemm_tc_swapped(w["gu"], xb1, err, s_, max_stages=st, cluster=cl, swiglu=True,
                                      colscale=(ss1, h, 1e-6), chain=c)
            s_, st, cl = plan(w["dn"])
            xb2, ss2 = ops.gemm_tc_swapped(w["dn"], act, err, s_, max_stages=st, cluster=cl, residual_norm=(resid, n2), chain=c)
            s_, st, cl = plan(w["qkv"])
            ops.gemm_qkv_rope(w["qkv"], xb2, err, s_, q, kc, vc, positions, tok_req, slot0, table, qn, kn, rot,
                              n_q_heads=hq, n_kv_heads=hkv, eps=1e-6, max_stages=st, colscale=(ss2, h, 1e-6), chain=c)
            ops.flush_chains()
        nbytes = sum(t.numel() * 2 for t in sets[0].values())
    elif name in ("gemm_pair_swiglu", "gemm_prefill_library"):
        # the prefill gate/up product of one layer over ctx tokens with the activation: the engine's
        # kernel on pairs of SMs with the activation in its epilogue, or the library product followed
        # by the activation kernel
        inter, hidden = cfg["intermediate_size"], cfg["hidden_size"]
        w = (torch.randn((2 * inter, hidden), device=dev, generator=gen) * 0.02).bfloat16()
        x = torch.randn((ctx, hidden), device=dev, generator=gen).bfloat16()
        act = torch.empty((ctx, inter), device=dev, dtype=torch.bfloat16)
        if name == "gemm_pair_swiglu":
            run = lambda: ops.gemm_pair(x, w, err, swiglu=True)
        else:
            def run():
                ops.swiglu(torch.mm(x, w.t()), act, block=ops.SWIGLU_TILE_BLOCK)
        nbytes = (w.numel() + x.numel() + act.numel()) * 2
        flops = 2.0 * ctx * 2 * inter * hidden
    else:
        raise SystemExit(f"unknown kernel case {name!r}")
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        run()
    end.record()
    torch.cuda.synchronize()
    us = begin.elapsed_time(end) * 1e3 / iters
    gbs = nbytes / (us * 1e-6) / 1e9
    res = {"kernel": name, "batch": batch, "ctx": ctx, "us": round(us, 2), "bytes": nbytes,
           "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4), "peaks": peaks["source"]}
    if flops:
        tf = flops / (us * 1e-6) / 1e12
        res.update({"TFLOP/s": round(tf, 1), "bf16_frac": round(tf / peaks["bf16_tflops"], 4)})
    assert err.tolist()[0] == 0
    return res


def prefill_attention_timeline(batch: int, ctx: int, portion: int, sizes: str) -> int:
    """Time stamps of the roles of the persistent prefill attention kernel on a few SMs (the library must
    have been built with TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE): when the producer published an item, when
    the softmax warps of query tile 0 / 1 started it, ended its key tiles, saw the last product and had
    written their rows, and the stamps of one block's thread per role within the key tiles."""
    import torch
    from tokamak_b200.csrc import ops
    cfg = SIZES[sizes][1] if sizes in SIZES else QWEN3_8B
    hq, hkv, d, page = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], 16
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    pages_per_req = -(-ctx // page)
    num_pages = batch * pages_per_req
    kc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
    vc = torch.randn((num_pages, hkv, page, d), device=dev, generator=gen).bfloat16()
    table = torch.randperm(num_pages, device=dev, generator=gen).to(torch.int32).view(batch, pages_per_req)
    qn = min(portion or ctx, ctx)
    q = torch.randn((batch * qn, hq, d), device=dev, generator=gen).bfloat16()
    out = torch.empty_like(q)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    records, n_parts, n_split = ops.prefill_tc_records([r * qn for r in range(batch)], [qn] * batch, [ctx] * batch,
                                                        list(range(batch)), heads=hq, sms=ops.sm_count(q.device))
    items = ops.PrefillItems(torch.from_numpy(records).to(dev), n_parts, n_split)
    run = lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=None)
    for _ in range(3):
        run()
    buf = ops.timeline_start(1 << 16)
    torch.cuda.synchronize()
    run()
    torch.cuda.synchronize()
    buf[0] = (buf.numel() - 1) // 2          # the roles' own ranges lie at the buffer's end
    every = [r for r in ops.timeline_read(buf) if r[0] > 0]
    recs = [r for r in every if r[1] == 30]
    clocks = [0] * 9
    for _, kernel, phase, _, value in every:
        if kernel == 32 and phase < 9:
            clocks[phase] += value
    if err.tolist()[0] != 0 or not recs:
        print("error word", err.tolist(), "records", len(recs))
        return 1
    t0 = recs[0][0]
    lengths = [int(r[5] - r[4]) for r in records]
    what = {1: "published", 10: "tile 0 starts", 11: "tile 1 starts", 20: "tile 0 keys done", 21: "tile 1 keys done",
            30: "tile 0 last product", 31: "tile 1 last product", 40: "tile 0 written", 41: "tile 1 written",
            50: "tile 0 parts added up", 51: "tile 1 parts added up", 60: "issuer 0 has item", 61: "issuer 1 has item"}
    coarse = [r for r in recs if r[2] < 70]
    by_sm: dict = {}
    for t, _, ph, sm, val in coarse:
        by_sm.setdefault(sm, []).append(((t - t0) / 1e3, ph, val))
    ends = sorted(max(x[0] for x in v) for v in by_sm.values())
    print(f"{batch} x {qn} tokens at the end of {ctx}, {hq} heads: {len(records)} records, {n_split} blocks of tokens cut; "
          f"blocks end after {ends[0]:.1f} / {ends[len(ends) // 2]:.1f} / {ends[-1]:.1f} us (first / median / last)")
    for sm in sorted(by_sm)[1:3]:
        print(f"SM {sm}")
        for t, ph, val in by_sm[sm]:
            n_rec = val // hq
            tiles = lengths[n_rec] if n_rec < len(lengths) else 0
            print(f"  {t:8.2f} us  item {val:5d} ({tiles:3d} key tiles)  {what.get(ph, ph)}")
    if clocks[8]:
        parts = ["waiting for S", "S loaded", "maximum", "exponentials, sum, conversion, store issued", "store arrived",
                 "fence and arrival", "loop", "between items"]
        print(f"one softmax thread of each query tile of block 0, clocks per key tile ({clocks[8]} key tiles):")
        for name, c in zip(parts, clocks):
            print(f"  {c / clocks[8]:7.1f}  {name}")
    fine = {70: "scores seen", 74: "probabilities given", 82: "S issued", 84: "probabilities seen", 86: "O += P V issued"}
    print("one block, within its key tiles (the stamps of this block cost it a few percent)")
    for t, _, ph, sm, val in [r for r in recs if r[2] >= 70][:64]:
        print(f"  {(t - t0) / 1e3:8.2f} us  tile {ph & 1}  {fine.get(ph - (ph & 1), ph):20s} key tile {val}")
    return 0


def tcgen05_probe() -> int:
    """Two tables of what the hardware gives the tcgen05 kernels (csrc/tcgen05_probe.cu): the cost of
    issuing a tcgen05.mma by shape, operand source and number of issuing threads, and the clocks one
    softmax warp of the prefill attention kernel needs for a 64-key tile in several forms of its loop."""
    from tokamak_b200.csrc import ops
    print("tcgen05.mma M 128 x N x K 16, bfloat16, 96 in a row: clocks per product until issued / until done")
    modes = {0: "one thread, A and B in shared memory", 1: "one thread, A in tensor memory",
             2: "two threads, A and B in shared memory", 3: "two threads, A in tensor memory",
             4: "one thread, 8 x (N, shared) then 4 x (N 128, A in tensor memory)"}
    for mode, name in modes.items():
        for n in (16, 64, 128, 256):
            if n > 128 and mode in (2, 3, 4) or mode == 4 and n == 16:
                continue
            for _ in range(2):
                rows = ops.probe_mma_issue(mode, n)
            cells = " | ".join(f"{r['issue_clk']:6.1f} / {r['done_clk']:6.1f} clk ({r['done_ns']:5.1f} ns)" for r in rows)
            print(f"  {name:66s} N {n:3d}: {cells}")
    print("one softmax warp, 64 keys: clocks per tile (load, maximum, exponentials + conversion + store, store arrived, fence)")
    forms = {0: "as the kernel has it", 1: "four chains for the maximum", 2: "second half loaded under the first maximum",
             3: "four chains and the split load", 4: "1 exponential in 4 by polynomial", 5: "2 in 4 by polynomial",
             6: "all by polynomial"}
    for variant, name in forms.items():
        for wg in (1, 2):
            for _ in range(2):
                r = ops.probe_softmax_tile(variant, wg)
            print(f"  {name:44s} {wg} warp(s) per scheduler: {r['tile']:7.1f}  ({r['load']:.0f}, {r['maximum']:.0f}, "
                  f"{r['exponentials_store']:.0f}, {r['store_arrived']:.0f}, {r['fence']:.0f})")
    return 0


def decode_timeline(batch: int, layers: int, ctx: int) -> int:
    """Lay the blocks of every kernel of two decode steps out on one time axis (the library must have
    been built with time stamps: TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE, see csrc/timeline.cuh).
    Prints, per kernel instance, when its blocks started, were released by the kernel before, finished
    their products and ended, in microseconds from the first stamp."""
    import torch
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.core import random_core
    from tokamak_b200.engine.step import SamplingRow, StepEntry
    raw = dict(QWEN3_8B, num_hidden_layers=layers)
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=ctx, page_size=16,
                       pool_tokens=batch * ctx, max_slots=batch, max_step_tokens=2048)
    step = core.step
    ids = [f"r{i}" for i in range(batch)]
    for r in ids:
        step.admit(r, SamplingRow())
    fill_context(core, ids, ctx - 40, raw["vocab_size"], seed=1)
    step.run_and_sample([StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)])
    entries = [StepEntry(r, None, [0]) for r in ids]
    for _ in range(6):
        step.run_and_sample(entries)
    buf = ops.timeline_start(1 << 18)
    first, second = step.launch_and_sample(entries), step.launch_and_sample(entries)
    step.collect(first); step.collect(second)
    recs = ops.timeline_read(buf)
    names = {1: "begin", 2: "attention", 3: "sample", 4: "embed", 10: "product", 11: "product+swiglu",
             12: "product+residual", 13: "q|k|v+rope", 20: "chain"}
    t0 = recs[0][0]
    by_kernel: dict = {}
    for t, k, ph, sm, blk in recs:
        by_kernel.setdefault(k, []).append((t - t0, ph))
    instances = []
    for k, rows in by_kernel.items():
        if k not in names:
            continue
        cur, last_start = None, None
        for t, ph in sorted(rows):
            if ph == 0 and (last_start is None or t - last_start > 4000):     # a gap of 4 us: another launch
                cur = {"k": k, "ph": {}}
                instances.append(cur)
            if ph == 0:
                last_start = t
            if cur is not None:
                cur["ph"].setdefault(ph, []).append(t)
    instances.sort(key=lambda i: min(i["ph"][0]))
    rng = lambda v: f"{min(v) / 1e3:7.1f}-{max(v) / 1e3:7.1f}" if v else " " * 15
    print(f"batch {batch}, {layers} layers of Qwen3-8B sizes, context {ctx}: two decode steps, us from the first stamp")
    print(f"{'kernel':17s} {'blocks':>6s} {'started':>15s} {'released':>15s} {'products done':>15s} {'ended':>15s}")
    for i in instances:
        ph = i["ph"]
        done = ph.get(2, []) if i["k"] != 20 else [t for q in ph if 31 <= q < 40 for t in ph[q]]
        print(f"{names[i['k']]:17s} {len(ph[0]):6d} {rng(ph.get(0))} {rng(ph.get(1))} {rng(done)} {rng(ph.get(4))}")
    return 0



# ------------------------------------------------------------------------------------------------
# --design ketalix: the Ketalix design beside a Qwen3 model of equal layer sizes

KETALIX_SIZES = {
    # width, query / key-value heads of 128 (keys and values), feed-forward, window; the gla layers have
    # width / 256 heads with keys of 128 and values of 256 (q, k: width / 2; v, gate: width)
    "2b": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, window=1024, vocab=65536, layers=8),
    "8b": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=12288, window=1024, vocab=151936, layers=8),
}


def ketalix_config(s: dict) -> dict:
    """Attention and gla layers in turn, every layer with a feed-forward."""
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
            "scale": s["dim"] ** -0.5 * 8.0, "softcap": 30.0, "mask": {"size": s["window"]},
            "rot": {"base": 1e6, "dims": s["dim"]}, "v_mix": True}
    gla = {"heads": s["width"] // 256, "dim": 128, "vdim": 256, "tau": 16.0, "rank": 16}
    mlp = {"kind": "dense", "ff": s["ff"]}
    layers = [{"type": "attention" if i % 2 == 0 else "gla", "mixer": attn if i % 2 == 0 else gla, "mlp": mlp}
              for i in range(s["layers"])]
    return {"architecture": "Ketalix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "layers": layers}


def qwen3_twin(s: dict) -> dict:
    """A Qwen3 configuration of the same widths, head counts, feed-forward, depth and window."""
    return dict(QWEN3_8B, num_hidden_layers=s["layers"], hidden_size=s["width"], num_attention_heads=s["heads"],
                num_key_value_heads=s["kv_heads"], head_dim=s["dim"], intermediate_size=s["ff"],
                vocab_size=s["vocab"], use_sliding_window=True, sliding_window=s["window"], max_window_layers=0)


def _time_us(run, iters: int = 20, graph: bool = False) -> float:
    """Microseconds a call of ``run`` takes on the device.  ``graph``: the calls are captured into one CUDA
    graph and replayed, as the engine replays the kernels of a step of single tokens, so that the host's
    time to launch does not count."""
    import torch
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                run()
        g.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        g.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) * 1e3 / iters
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        run()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) * 1e3 / iters


def ketalix_kernels(s: dict, tokens: int, batch: int, ctx: int, peaks: dict) -> list[dict]:
    """Every kernel of the design alone, beside the like kernel of the Qwen3 path at the same shape:
    time, achieved bytes or flops per second, and the fraction of the measured peak."""
    import torch
    from tokamak_b200.csrc import ops
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    hq, hkv, d, page, win, width, ff = s["heads"], s["kv_heads"], s["dim"], 16, s["window"], s["width"], s["ff"]
    bf = lambda *shape: torch.randn(shape, device=dev, generator=gen).bfloat16()
    rows = []

    def row(kernel, like, us, us_like, nbytes=0, flops=0.0, note=""):
        r = {"kernel": kernel, "like": like, "us": round(us, 1), "like_us": round(us_like, 1) if us_like else None}
        for name, t in (("", us), ("like_", us_like)):
            if not t:
                continue
            if flops:
                r[name + "bf16_frac"] = round(flops / (t * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)
            elif nbytes:
                r[name + "hbm_frac"] = round(nbytes / (t * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)
        if note:
            r["note"] = note
        rows.append(r)

    sinks = torch.randn(hq, device=dev, generator=gen)
    # ---- attention over a prompt of `tokens` tokens, and over `batch` single tokens at context `ctx`
    pages_pf = -(-tokens // page)
    kc, vc = bf(pages_pf, hkv, page, d), bf(pages_pf, hkv, page, d)
    table = torch.randperm(pages_pf, device=dev, generator=gen).to(torch.int32).view(1, pages_pf)
    q = bf(tokens, hq, d)
    out = torch.empty_like(q)
    rec, n_parts, n_split = ops.prefill_tc_records([0], [tokens], [tokens], [0], heads=hq, sms=ops.sm_count(q.device))
    items = ops.PrefillItems(torch.from_numpy(rec).to(dev), n_parts, n_split)
    pf = lambda **kw: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=win, **kw)
    keys = sum(min(i + 1, win) for i in range(tokens))
    row("attention, prompt (cap + sink)", "attention, prompt", _time_us(lambda: pf(softcap=30.0, sinks=sinks)),
        _time_us(pf), flops=4.0 * keys * hq * d,
        note="three exponential-unit operations a score (tanh by exp and reciprocal, then exp) against one")
    pages_req = -(-ctx // page)
    kc, vc = bf(batch * pages_req, hkv, page, d), bf(batch * pages_req, hkv, page, d)
    table = torch.randperm(batch * pages_req, device=dev, generator=gen).to(torch.int32).view(batch, pages_req)
    qd = bf(batch, hq, d)
    outd = torch.empty_like(qd)
    it, pos = i32(list(range(batch))), i32([ctx - 1] * batch)
    n_splits = ops.decode_splits(batch, hkv, min(ctx, win))
    scratch = torch.empty(batch * hq * n_splits * (d + 2), dtype=torch.float32, device=dev)
    dec = lambda **kw: ops.attention_decode(qd, outd, kc, vc, it, pos, it, it, table, err, scale=d ** -0.5,
                                            window=win, n_splits=n_splits, scratch=scratch, **kw)
    row("attention, single tokens (cap + sink)", "attention, single tokens",
        _time_us(lambda: dec(softcap=30.0, sinks=sinks)), _time_us(dec),
        nbytes=batch * 2 * hkv * min(ctx, win) * d * 2 + 2 * qd.numel() * 2)
    # ---- rotation, norm of q and k, page write
    qkv = bf(tokens, (hq + 2 * hkv) * d)
    kc, vc = torch.zeros((pages_pf, hkv, page, d), dtype=torch.bfloat16, device=dev), torch.zeros((pages_pf, hkv, page, d), dtype=torch.bfloat16, device=dev)
    positions, zeros = torch.arange(tokens, dtype=torch.int32, device=dev), torch.zeros(tokens, dtype=torch.int32, device=dev)
    table = torch.arange(pages_pf, dtype=torch.int32, device=dev).view(1, pages_pf)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
    rot = ops.rope_table(positions, inv_freq)
    ones, slot0, len_n = torch.ones(d, device=dev), i32([0]), i32([tokens])
    vf, lam = torch.randn(tokens, hkv * d, device=dev, generator=gen), torch.full((1,), 0.3, device=dev)
    pairs = lambda: ops.qkv_pairs(qkv, q, kc, vc, positions, zeros, slot0, table, rot, err, n_q_heads=hq,
                                  n_kv_heads=hkv, rotary_dim=d, unit_norm_eps=1e-6, v_first_in=vf, v_lambda=lam,
                                  req_q_len=len_n, req_kv_len=len_n)
    halves = lambda: ops.rope_kv(qkv, q, kc, vc, positions, zeros, slot0, table, ones, ones, rot, err, n_q_heads=hq,
                                 n_kv_heads=hkv, head_dim=d, rotary_dim=d, eps=1e-6, req_q_len=len_n, req_kv_len=len_n)
    nb = qkv.numel() * 2 + q.numel() * 2 + 2 * tokens * hkv * d * 2
    row("pair rotation + unit norm + value blend + page write", "half rotation + weighted norm + page write",
        _time_us(pairs), _time_us(halves), nbytes=nb + vf.numel() * 4)
    # ---- norms around a sublayer
    resid, branch = torch.randn(tokens, width, device=dev, generator=gen), bf(tokens, width)
    w1, w2, w3 = (torch.ones(width, device=dev) for _ in range(3))
    normed = torch.empty(tokens, width, dtype=torch.bfloat16, device=dev)
    row("output norm + layer scale + residual + input norm", "residual + input norm",
        _time_us(lambda: ops.branch_norm_add(resid, branch, w1, w2, 1e-6, w3, normed, 1e-6)),
        _time_us(lambda: ops.add_rmsnorm(resid, branch, w3, normed, 1e-6)), nbytes=tokens * width * (2 + 8 + 2))
    # ---- the gated unit's activation
    gu, act = bf(tokens, 2 * ff), torch.empty(tokens, ff, dtype=torch.bfloat16, device=dev)
    row("gelu gate", "silu gate (the unfused kernel)",
        _time_us(lambda: ops.swiglu(gu, act, block=ops.SWIGLU_TILE_BLOCK, activation="gelu_tanh")),
        _time_us(lambda: ops.swiglu(gu, act, block=ops.SWIGLU_TILE_BLOCK)), nbytes=3 * tokens * ff * 2,
        note="the kernel of its own, for float32 and for sizes that are no multiple of 64: both models' "
             "bfloat16 products apply the gate in their epilogues (next row)")
    wgu = bf(2 * ff, width) * (width ** -0.5)
    xin = bf(tokens, width)
    if ops.pair_gemm_takes(tokens, 2 * ff, width, fused=True):
        row("gate/up product with the gelu gate in its epilogue", "the same with the silu gate",
            _time_us(lambda: ops.gemm_pair(xin, wgu, err, swiglu=True, activation="gelu_tanh")),
            _time_us(lambda: ops.gemm_pair(xin, wgu, err, swiglu=True)), flops=2.0 * tokens * 2 * ff * width)
    # ---- gated linear attention
    gh, gk, gv, rank = width // 256, 128, 256, 16
    rowlen = 2 * gh * gk + 2 * gh * gv + rank
    for name, n, n_req in (("prompt", tokens, 1), ("single tokens", batch, batch)):
        proj = bf(n, rowlen) * 0.5
        w2a, bias = bf(gh * gk, rank) * 0.1, torch.randn(gh * gk, device=dev, generator=gen)
        state = torch.zeros(max(n_req, 1), gh, gk, gv, device=dev)
        starts, lens = i32([i * (n // n_req) for i in range(n_req)]), i32([n // n_req] * n_req)
        slots = i32(list(range(n_req)))
        prepare = lambda: ops.gla_prepare(proj, 0, gh * gk, 2 * gh * gk, 2 * gh * gk + 2 * gh * gv, w2a, bias, heads=gh,
                                          key_dim=gk, value_dim=gv, tau=16.0, q_scale=gk ** -0.5)
        prep = prepare()
        scan = lambda: ops.gla_scan(prep, state, starts, lens, slots, err)
        o = scan()
        us = _time_us(scan)
        state_bytes = 2 * n_req * gh * gk * gv * 4
        in_bytes = prep.numel() * 4 + n * gh * gv * 4
        r = {"kernel": f"gla recurrence, {name}", "like": None, "us": round(us, 1),
             "hbm_frac": round((state_bytes + in_bytes) / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
             "fp32_tflops": round(4.0 * n * gh * gk * gv / (us * 1e-6) / 1e12, 2),
             "note": "float32 on the CUDA cores, token by token: bound by the length of the chain of tokens in "
                     "a prompt, by the state's bytes for single tokens"}
        rows.append(r)
        nw = torch.ones(gv, device=dev)
        row(f"gla float32 inputs (scaled q, k, decays, v), {name}", None, _time_us(prepare), 0.0,
            nbytes=n * (2 * gh * gk + gh * gv + rank) * 2 + prep.numel() * 4)
        row(f"gla output norm + gate, {name}", None,
            _time_us(lambda: ops.gla_out(o, proj, 2 * gh * gk + gh * gv, nw, 1e-6, torch.bfloat16)), 0.0,
            nbytes=n * gh * gv * (4 + 2 + 2))
    assert err.tolist()[0] == 0
    return rows


# ------------------------------------------------------------------------------------------------
# --design logivik: the Logivik design beside a Ketalix model of equal layer sizes (the engine's
# other design with paged attention layers and recurrent layers in turn)

def logivik_config(s: dict) -> dict:
    """Windowed latent attention, delta rule, latent attention with a rotated part, delta rule, and again;
    every layer with a feed-forward.  Latents of 512 (+ 64 rotated), heads of 128; the delta layers have
    width / 256 heads with keys of 128 and values of 256 (the state of Ketalix's recurrent layers)."""
    d, h, w = s["dim"], s["heads"], s["width"]
    win = {"heads": h, "dim": d, "vdim": d, "kv_rank": 512, "q_rank": 3 * w // 4, "scale": d ** -0.5,
           "mask": {"size": s["window"]}}
    rot = {"heads": h, "dim": d, "rot_dim": 64, "vdim": d, "kv_rank": 512, "scale": (d + 64) ** -0.5,
           "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    delta = {"heads": w // 256, "kv_heads": max(1, w // 512), "dim": 128, "vdim": 256, "conv": 4}
    mlp = {"kind": "dense", "ff": s["ff"]}
    order = [("latent_attention_2", win), ("delta", delta), ("latent_attention", rot), ("delta", delta)]
    layers = [{"type": order[i % 4][0], "mixer": order[i % 4][1], "mlp": mlp} for i in range(s["layers"])]
    return {"architecture": "Logivik", "vocab": s["vocab"], "width": w, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "layers": layers}


def logivik_kernels(s: dict, tokens: int, batch: int, ctx: int, peaks: dict) -> list[dict]:
    """Every kernel of the design alone, beside the like kernel of the Ketalix path at the same shape:
    time, achieved bytes or flops per second, and the fraction of the measured peak."""
    import torch
    from types import SimpleNamespace
    from tokamak_b200.csrc import ops
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    hq, hkv, d, page, win, width = s["heads"], s["kv_heads"], s["dim"], 16, s["window"], s["width"]
    rank, rot = 512, 64
    bf = lambda *shape: torch.randn(shape, device=dev, generator=gen).bfloat16()
    rows = []

    def row(kernel, like, us, us_like, nbytes=0, flops=0.0, like_bytes=0, like_flops=0.0, note=""):
        r = {"kernel": kernel, "like": like, "us": round(us, 1), "like_us": round(us_like, 1) if us_like else None}
        for name, t, fl, nb in (("", us, flops, nbytes), ("like_", us_like, like_flops or flops, like_bytes or nbytes)):
            if not t:
                continue
            if fl:
                r[name + "bf16_frac"] = round(fl / (t * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)
            elif nb:
                r[name + "hbm_frac"] = round(nb / (t * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)
        if note:
            r["note"] = note
        rows.append(r)

    sinks = torch.randn(hq, device=dev, generator=gen)
    # ---- attention over a prompt of `tokens` tokens
    pages_pf = -(-tokens // page)
    table = torch.randperm(pages_pf, device=dev, generator=gen).to(torch.int32).view(1, pages_pf)
    positions, zeros = torch.arange(tokens, dtype=torch.int32, device=dev), torch.zeros(tokens, dtype=torch.int32, device=dev)
    step_pf = SimpleNamespace(positions=positions, tok_req=zeros, req_q_start=i32([0]), req_q_len=i32([tokens]),
                              req_kv_len=i32([tokens]), req_slot=i32([0]), err=err)
    tiles = i32([x for t in reversed(range(-(-tokens // 64))) for x in (0, t)])
    kc, vc = bf(pages_pf, hkv, page, d), bf(pages_pf, hkv, page, d)
    q = bf(tokens, hq, d)
    out = torch.empty_like(q)
    rec, n_parts, n_split = ops.prefill_tc_records([0], [tokens], [tokens], [0], heads=hq, sms=ops.sm_count(q.device))
    items = ops.PrefillItems(torch.from_numpy(rec).to(dev), n_parts, n_split)
    like_pf = lambda w: _time_us(lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5,
                                                                  window=w, softcap=30.0, sinks=sinks))
    for name, dr, w, sk in (("latent attention, prompt (rotated part, sink)", rot, None, sinks),
                            ("latent attention, prompt (window)", 0, win, None)):
        cache = bf(pages_pf, 1, page, rank + dr) * 0.3
        ql = torch.randn(tokens, hq, rank + dr, device=dev, generator=gen) * 0.1
        ol = torch.empty(tokens, hq, rank, dtype=torch.bfloat16, device=dev)
        keys = sum(min(i + 1, w or tokens) for i in range(tokens))
        us = _time_us(lambda: ops.attention_latent(ql, ol, cache, rank, step_pf, table, scale=0.07, window=w, sinks=sk,
                                                   tiles=tiles), iters=5)
        row(name, "attention, prompt (cap + sink), same window", us, like_pf(w),
            flops=2.0 * keys * hq * (2 * rank + dr), like_flops=4.0 * keys * hq * d,
            note="scores and sums in the latent space: 2 x 512 (+ 64) multiply-adds a key and head against 2 x 128, "
                 "on mma.sync with both column halves forming the scores")
    # ---- attention of `batch` single tokens at context `ctx`
    pages_req = -(-ctx // page)
    table_d = torch.randperm(batch * pages_req, device=dev, generator=gen).to(torch.int32).view(batch, pages_req)
    it, pos = i32(list(range(batch))), i32([ctx - 1] * batch)
    step_d = SimpleNamespace(positions=pos, tok_req=it, req_q_start=it, req_q_len=i32([1] * batch),
                             req_kv_len=i32([ctx] * batch), req_slot=it, err=err)
    kc, vc = bf(batch * pages_req, hkv, page, d), bf(batch * pages_req, hkv, page, d)
    qd = bf(batch, hq, d)
    outd = torch.empty_like(qd)

    def like_dec(w):
        n_splits = ops.decode_splits(batch, hkv, min(ctx, w or ctx))
        scratch = torch.empty(batch * hq * n_splits * (d + 2), dtype=torch.float32, device=dev)
        return _time_us(lambda: ops.attention_decode(qd, outd, kc, vc, it, pos, it, it, table_d, err, scale=d ** -0.5,
                                                     window=w, n_splits=n_splits, scratch=scratch, softcap=30.0, sinks=sinks),
                        graph=True)
    for name, dr, w, sk in (("latent attention, single tokens (rotated part, sink)", rot, None, sinks),
                            ("latent attention, single tokens (window)", 0, win, None)):
        cache = bf(batch * pages_req, 1, page, rank + dr) * 0.3
        ql = torch.randn(batch, hq, rank + dr, device=dev, generator=gen) * 0.1
        ol = torch.empty(batch, hq, rank, dtype=torch.bfloat16, device=dev)
        n_splits = ops.latent_decode_splits(ql.device, batch, ctx, w)
        us = _time_us(lambda: ops.attention_latent(ql, ol, cache, rank, step_d, table_d, scale=0.07, window=w, sinks=sk,
                                                   items=it, n_splits=n_splits), graph=True)
        seen = min(ctx, w or ctx)
        row(name, "attention, single tokens (cap + sink), same window", us, like_dec(w),
            nbytes=batch * seen * (rank + dr) * 2, like_bytes=batch * 2 * hkv * seen * d * 2)
    # ---- what stands between the input projection and attention
    cols = hq * (d + rot) + rank + rot + hq * d
    proj = bf(tokens, cols)
    cache = torch.zeros(pages_pf, 1, page, rank + rot, dtype=torch.bfloat16, device=dev)
    table_w = torch.arange(pages_pf, dtype=torch.int32, device=dev).view(1, pages_pf)
    freq = (1.0 / (1e6 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev)
    rope = ops.rope_table(positions, freq, 1.1)
    q_abs = torch.randn(hq, tokens, rank, device=dev, generator=gen)
    ones_r = torch.ones(rank, device=dev)
    prep = lambda: ops.latent_prepare(proj, cache, positions, zeros, i32([0]), table_w, err, kv_off=hq * (d + rot), rank=rank,
                                      rot=rot, kv_norm_w=ones_r, eps=1e-6, table=rope, q_abs=q_abs, q_off=0,
                                      q_head_cols=d + rot, q_rot_off=d)
    qkv = bf(tokens, (hq + 2 * hkv) * d)
    kc2, vc2 = (torch.zeros((pages_pf, hkv, page, d), dtype=torch.bfloat16, device=dev) for _ in range(2))
    qo = torch.empty(tokens, hq, d, dtype=torch.bfloat16, device=dev)
    rope_d = ops.rope_table(positions, (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev))
    len_n = i32([tokens])
    pairs = lambda: ops.qkv_pairs(qkv, qo, kc2, vc2, positions, zeros, i32([0]), table_w, rope_d, err, n_q_heads=hq,
                                  n_kv_heads=hkv, rotary_dim=d, unit_norm_eps=1e-6, req_q_len=len_n, req_kv_len=len_n)
    row("latent norm + rotated parts + cache write + query rows (float32)", "pair rotation + unit norm + page write",
        _time_us(prep), _time_us(pairs),
        nbytes=tokens * ((rank + rot + hq * rot) * 2 + (rank + rot) * 2 + hq * rank * 4 + hq * (rank + rot) * 4),
        like_bytes=qkv.numel() * 2 + qo.numel() * 2 + 2 * tokens * hkv * d * 2)
    o_h = bf(hq, tokens, d)
    row("heads back to token rows + sigmoid gate", None, _time_us(lambda: ops.heads_gate(o_h, proj, cols - hq * d)), 0.0,
        nbytes=3 * tokens * hq * d * 2)
    # ---- the norm behind a sublayer
    resid, branch = torch.randn(tokens, width, device=dev, generator=gen), bf(tokens, width)
    w1, w2, w3 = (torch.ones(width, device=dev) for _ in range(3))
    normed = torch.empty(tokens, width, dtype=torch.bfloat16, device=dev)
    row("output norm + residual, the stream handed on unnormalised", "output norm + layer scale + residual + input norm",
        _time_us(lambda: ops.branch_norm_add(resid, branch, w1, None, 1e-6, None, normed, 0.0)),
        _time_us(lambda: ops.branch_norm_add(resid, branch, w1, w2, 1e-6, w3, normed, 1e-6)), nbytes=tokens * width * (2 + 8 + 2))
    # ---- the recurrences
    gh, gkh, gk, gv, taps, rk = width // 256, max(1, width // 512), 128, 256, 4, 16
    rowlen = 2 * gkh * gk + 2 * gh * gv + 2 * gh
    rowlen_g = 2 * gh * gk + 2 * gh * gv + rk
    for name, n, n_req in (("prompt", tokens, 1), ("single tokens", batch, batch)):
        projd, projg = bf(n, rowlen) * 0.5, bf(n, rowlen_g) * 0.5
        conv = torch.randn(2 * gkh * gk + gh * gv, taps, device=dev, generator=gen) * 0.5
        a_log, dt_b = torch.randn(gh, device=dev, generator=gen) * 0.5, torch.randn(gh, device=dev, generator=gen) * 0.5
        floats, _ = ops.delta_record_floats(gh, gkh, gk, gv, taps)
        records = torch.zeros(n_req, floats, device=dev)
        per = n // n_req
        starts, lens, slots = i32([i * per for i in range(n_req)]), i32([per] * n_req), i32(list(range(n_req)))
        tok_req = torch.arange(n, dtype=torch.int32, device=dev) // per
        offs = dict(q_off=0, k_off=gkh * gk, v_off=2 * gkh * gk, b_off=2 * gkh * gk + 2 * gh * gv, a_off=2 * gkh * gk + 2 * gh * gv + gh)
        dprep = lambda: ops.delta_prepare(projd, conv, a_log, dt_b, records, tok_req, starts, lens, slots, err,
                                          dtype=torch.bfloat16, heads=gh, kv_heads=gkh, key_dim=gk, value_dim=gv,
                                          unit_eps=1e-6, q_scale=gk ** -0.5, **offs)
        qf, kf, vf, bt, gg = dprep()
        dscan = lambda: ops.delta_scan(qf, kf, vf, bt, gg, records, starts, lens, slots, err)
        w2a, bias = bf(gh * gk, rk) * 0.1, torch.randn(gh * gk, device=dev, generator=gen)
        state = torch.zeros(n_req, gh, gk, gv, device=dev)
        gprep = lambda: ops.gla_prepare(projg, 0, gh * gk, 2 * gh * gk, 2 * gh * gk + 2 * gh * gv, w2a, bias, heads=gh,
                                        key_dim=gk, value_dim=gv, tau=16.0, q_scale=gk ** -0.5)
        gp = gprep()
        gscan = lambda: ops.gla_scan(gp, state, starts, lens, slots, err)
        single = n_req > 1          # kernels of a step of single tokens are timed as the engine runs them: from a graph
        us, us_like = _time_us(dscan, graph=single), _time_us(gscan, graph=single)
        state_bytes = 2 * n_req * gh * gk * gv * 4
        r = {"kernel": f"delta rule recurrence, {name}", "like": f"gla recurrence, {name}", "us": round(us, 1),
             "like_us": round(us_like, 1),
             "hbm_frac": round((state_bytes + n * (2 * gkh * gk + 2 * gh * gv + 2 * gh) * 4) / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
             "like_hbm_frac": round((state_bytes + gp.numel() * 4 + n * gh * gv * 4) / (us_like * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
             "fp32_tflops": round(8.0 * n * gh * gk * gv / (us * 1e-6) / 1e12, 2),
             "like_fp32_tflops": round(4.0 * n * gh * gk * gv / (us_like * 1e-6) / 1e12, 2),
             "note": "float32 on the CUDA cores, token by token; the delta rule reads the state twice a token "
                     "(S^T k before the write, S^T q after it): 8 flops a state element against 4"}
        rows.append(r)
        row(f"delta rule float32 inputs (convolution, silu, unit norm, beta, decay), {name}",
            f"gla float32 inputs (scaled q, k, decays, v), {name}", _time_us(dprep, graph=single),
            _time_us(gprep, graph=single),
            nbytes=n * (2 * gkh * gk + gh * gv + 2 * gh) * (2 + 4), like_bytes=n * (2 * gh * gk + gh * gv + rk) * 2 + gp.numel() * 4)
    assert err.tolist()[0] == 0
    return rows


# ------------------------------------------------------------------------------------------------
# --design tarivik: the Tarivik design beside a Ketalix model of equal layer sizes (the engine's
# closest other design: paged attention layers and recurrent layers on the same recurrence kernel in turn)

def tarivik_config(s: dict) -> dict:
    """Parallel (chunked attention beside a state-space half), HGRN2, parallel, mLSTM, and again; every layer with
    a mixture of 8 experts of which 2 are used, together as wide as the twin's feed-forward.  Attention heads
    as the twin's, chunks as long as its window; the state-space half has width / 64 heads of 64 channels and a
    state of 128 rows; the other recurrent layers have the twin's state (width / 256 heads, 128 x 256)."""
    w, d = s["width"], s["dim"]
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
            "mask": {"size": s["window"]}}
    right = {"heads": w // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 4}
    par = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.6}
    rec = {"heads": w // 256, "dim": 128, "vdim": 256}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"] // 2},
           "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}}
    order = [("parallel", par), ("hgrn2", rec), ("parallel", par), ("mlstm", dict(rec, gate_cap=15.0))]
    layers = [{"type": order[i % 4][0], "mixer": order[i % 4][1], "mlp": mlp} for i in range(s["layers"])]
    return {"architecture": "Tarivik", "vocab": s["vocab"], "width": w, "max_positions": 32768,
            "norm": {"eps": 1e-5, "groups": 8}, "canon": {"taps": 4}, "layers": layers}


def tarivik_kernels(s: dict, tokens: int, batch: int, ctx: int, peaks: dict) -> list[dict]:
    """Every kernel of the design alone, beside the like kernel of the Ketalix path at the same shape:
    time, achieved bytes or flops per second, and the fraction of the measured peak."""
    import torch
    from types import SimpleNamespace
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.attention import paged_attention
    from tokamak_b200.cache.device import KVView
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    hq, hkv, d, page, chunk, width = s["heads"], s["kv_heads"], s["dim"], 16, s["window"], s["width"]
    ffe, experts, top = s["ff"] // 2, 8, 2
    bf = lambda *shape: torch.randn(shape, device=dev, generator=gen).bfloat16()
    f32 = lambda *shape: torch.randn(shape, device=dev, generator=gen)
    rows = []

    def row(kernel, like, us, us_like, nbytes=0, flops=0.0, like_bytes=0, like_flops=0.0, note=""):
        r = {"kernel": kernel, "like": like, "us": round(us, 1), "like_us": round(us_like, 1) if us_like else None}
        for name, t, fl, nb in (("", us, flops, nbytes), ("like_", us_like, like_flops or flops, like_bytes or nbytes)):
            if not t:
                continue
            if fl:
                r[name + "bf16_frac"] = round(fl / (t * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)
            elif nb:
                r[name + "hbm_frac"] = round(nb / (t * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)
        if note:
            r["note"] = note
        rows.append(r)

    def step_of(n, n_req, start):
        per = n // n_req
        none = i32([])
        rec, n_parts, n_split = ops.prefill_tc_records([r * per for r in range(n_req)], [per] * n_req, [start + per] * n_req,
                                                       list(range(n_req)), heads=s["heads"], sms=ops.sm_count(torch.device(dev, 0)))
        return SimpleNamespace(
            decode_items=i32(list(range(n))) if per == 1 else none, prefill_items=none if per == 1 else i32(list(range(n))),
            prefill_tiles=none, prefill_tc=ops.PrefillItems(torch.from_numpy(rec).to(dev), n_parts, n_split),
            positions=i32([start + i for _ in range(n_req) for i in range(per)]),
            tok_req=i32([r for r in range(n_req) for _ in range(per)]), req_q_start=i32([r * per for r in range(n_req)]),
            req_q_len=i32([per] * n_req), req_kv_len=i32([start + per] * n_req), req_slot=i32(list(range(n_req))),
            err=err, max_q_len=per, n_tokens=n, n_reqs=n_req, scratch={}, host_q_start=[r * per for r in range(n_req)],
            host_q_len=[per] * n_req, host_kv_len=[start + per] * n_req, host_slot=list(range(n_req)),
            max_kv_len=start + per)

    sinks, slopes = f32(hq), torch.pow(2.0, -8.0 * torch.arange(1, hq + 1, device=dev) / hq).float()
    cases = (("prompt", tokens, 1, 0), ("single tokens", batch, batch, ctx - 1))
    # ---- chunked attention with distance bias and sinks; the twin's has a window, a cap and sinks
    for name, n, n_req, start in cases:
        single = n_req > 1
        step = step_of(n, n_req, start)
        pages_req = -(-(start + n // n_req) // page)
        kc, vc = bf(n_req * pages_req, hkv, page, d), bf(n_req * pages_req, hkv, page, d)
        table = torch.randperm(n_req * pages_req, device=dev, generator=gen).to(torch.int32).view(n_req, pages_req)
        q = bf(n, hq, d)
        out = torch.empty_like(q)
        view = KVView(kc, vc, table, page, None)
        if single:
            keys = n * ((start % chunk) + 1)
            like_keys = n * min(start + 1, chunk)
            n_splits = ops.decode_splits(n, hkv, min(ctx, chunk))
            scratch = torch.empty(n * hq * n_splits * (d + 2), dtype=torch.float32, device=dev)
            it = i32(list(range(n)))
            like = lambda: ops.attention_decode(q, out, kc, vc, it, step.positions, it, it, table, err, scale=d ** -0.5,
                                                window=chunk, n_splits=n_splits, scratch=scratch, softcap=30.0, sinks=sinks)
        else:
            keys = sum((i % chunk) + 1 for i in range(n))
            like_keys = sum(min(i + 1, chunk) for i in range(n))
            rec, n_parts, n_split = ops.prefill_tc_records([0], [n], [n], [0], heads=hq, sms=ops.sm_count(q.device))
            items = ops.PrefillItems(torch.from_numpy(rec).to(dev), n_parts, n_split)
            like = lambda: ops.attention_prefill_tc(q, out, kc, vc, items, table, err, scale=d ** -0.5, window=chunk,
                                                    softcap=30.0, sinks=sinks)
        mine = lambda: paged_attention(q, out, view, step, scale=d ** -0.5, window=None, sinks=sinks, chunk=chunk,
                                       slopes=slopes)
        mine()
        if single:
            row(f"chunked attention (distance bias, sink), {name}", "windowed attention (cap, sink), single tokens",
                _time_us(mine, graph=True), _time_us(like, graph=True), nbytes=2 * hkv * keys * d * 2 + 2 * q.numel() * 2,
                like_bytes=2 * hkv * like_keys * d * 2 + 2 * q.numel() * 2,
                note=f"the last token of a chunk would see {chunk} keys; at position {start} it sees {(start % chunk) + 1}")
        else:
            row(f"chunked attention (distance bias, sink), {name}", "windowed attention (cap, sink), prompt",
                _time_us(mine, iters=5), _time_us(like), flops=4.0 * keys * hq * d, like_flops=4.0 * like_keys * hq * d)
        # ---- biases, whole-row norms of q and k, page write
        proj = bf(n, (2 * hq + 2 * hkv) * d)
        qb, kb, vb = f32(hq * d), f32(hkv * d), f32(hkv * d)
        qn, kn = f32(hq * d), f32(hkv * d)
        rn = lambda: ops.qkv_rownorm(proj, q, kc, vc, step, table, q_off=0, k_off=hq * d, v_off=(hq + hkv) * d, q_bias=qb,
                                     k_bias=kb, v_bias=vb, q_norm=qn, k_norm=kn, eps=1e-6)
        qkv = bf(n, (hq + 2 * hkv) * d)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(step.positions, inv_freq)
        vf, lam = f32(n, hkv * d), torch.full((1,), 0.3, device=dev)
        pairs = lambda: ops.qkv_pairs(qkv, q, kc, vc, step.positions, step.tok_req, step.req_slot, table, rot, err,
                                      n_q_heads=hq, n_kv_heads=hkv, rotary_dim=d, unit_norm_eps=1e-6, v_first_in=vf,
                                      v_lambda=lam, req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)
        nb = 2 * (hq + 2 * hkv) * d * n * 2
        row(f"biases + norms over whole q and k + page write, {name}",
            f"pair rotation + unit norm + value blend + page write, {name}", _time_us(rn, graph=single),
            _time_us(pairs, graph=single), nbytes=nb, like_bytes=nb + vf.numel() * 4)
        att, gproj = bf(n, hq * d), bf(n, (2 * hq + 2 * hkv) * d)
        wide = torch.empty(n, hq * d + width, dtype=torch.bfloat16, device=dev)
        row(f"output gate + branch factor into the stacked rows, {name}", None,
            _time_us(lambda: ops.gate_scale(att, gproj, (hq + 2 * hkv) * d, out=wide[:, :hq * d], scale=0.8), graph=single),
            0.0, nbytes=3 * n * hq * d * 2)
        # ---- the block's seats: join with a norm in groups, then the input convolution on the stream
        resid, branch = f32(n, width), bf(n, width)
        w1 = torch.ones(width, device=dev)
        normed = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        row(f"output norm in groups + residual, {name}", f"output norm + layer scale + residual + input norm, {name}",
            _time_us(lambda: ops.branch_norm_add(resid, branch, w1, None, 1e-6, None, None, branch_groups=4), graph=single),
            _time_us(lambda: ops.branch_norm_add(resid, branch, w1, w1, 1e-6, w1, normed, 1e-6), graph=single),
            nbytes=n * width * (2 + 8), like_bytes=n * width * (2 + 8 + 2))
        taps4, tail = f32(width, 4) * 0.3, torch.zeros(n_req, 3, width, device=dev)
        row(f"input convolution on the float32 stream, {name}", None,
            _time_us(lambda: ops.short_conv(resid, taps4, tail, step, dtype=torch.bfloat16, add_input=True), graph=single),
            0.0, nbytes=n * width * (4 + 2) + (2 * tail.numel() * 4 if single else 0))
        # ---- mixture of experts against the twin's gated unit of the same active width
        h = bf(n, width)
        router, corr = f32(experts, width) * 0.05, f32(experts) * 0.05
        wg, wu = bf(experts, ffe, width) * width ** -0.5, bf(experts, ffe, width) * width ** -0.5
        wd = bf(experts, width, ffe) * ffe ** -0.5
        route = lambda: ops.moe_route(h, router, corr, top=top, n_groups=4, keep=2, padded=True)
        routing = route()
        row(f"router (scores, groups, choice, tiles), {name}", None, _time_us(route, graph=True), 0.0,
            nbytes=n * width * 2 + experts * width * 4)
        wgu_dense = bf(2 * top * ffe, width) * width ** -0.5
        wd_dense = bf(width, top * ffe) * (top * ffe) ** -0.5
        from tokamak_b200.parts.base import linear

        def dense():
            if ops.pair_gemm_takes(n, 2 * top * ffe, width, fused=True):
                a = ops.gemm_pair(h, wgu_dense, err, swiglu=True)
            else:
                gu = linear(h, wgu_dense, err=err)
                a = torch.empty(n, top * ffe, dtype=torch.bfloat16, device=dev)
                ops.swiglu(gu, a, block=ops.SWIGLU_TILE_BLOCK)
            y = linear(a, wd_dense, err=err)
            ops.flush_chains()
            return y
        used = len(set(routing.chosen.flatten().tolist()))
        wgu = ops.moe_stack_gate_up(wg, wu)
        if ops.moe_small_takes(n, top, width, ffe):       # as the part chooses
            moe = lambda: ops.moe_experts_small(h, routing, wgu, wd)
        else:
            moe = lambda: ops.moe_experts_tc(h, routing, wgu, wd, err)
        flops = 2.0 * n * top * 3 * ffe * width
        if single:
            row(f"experts (gate, up, down, weighted sum), {name}", "dense gated unit of the same active width",
                _time_us(moe, graph=True), _time_us(dense, graph=True),
                nbytes=used * 3 * ffe * width * 2, like_bytes=top * 3 * ffe * width * 2,
                note=f"{used} of {experts} experts are read by the {n} tokens")
        else:
            row(f"experts (gate, up, down, weighted sum), {name}", "dense gated unit of the same active width",
                _time_us(moe), _time_us(dense), flops=flops)
        # ---- the recurrent layers: inputs, recurrence, output stage, beside gated linear attention's
        gh, gk, gv, rk = width // 256, 128, 256, 16
        sh, sn, sv = width // 64, 128, 64
        gproj = bf(n, 2 * gh * gk + 2 * gh * gv + rk) * 0.5
        w2a, gbias = bf(gh * gk, rk) * 0.1, f32(gh * gk)
        gprep = lambda: ops.gla_prepare(gproj, 0, gh * gk, 2 * gh * gk, 2 * gh * gk + 2 * gh * gv, w2a, gbias, heads=gh,
                                        key_dim=gk, value_dim=gv, tau=16.0, q_scale=gk ** -0.5)
        gstate = torch.zeros(n_req, gh, gk, gv, device=dev)
        gp = gprep()
        gscan = lambda: ops.gla_scan(gp, gstate, step.req_q_start, step.req_q_len, step.req_slot, err)
        go = gscan()
        us_gscan, us_gprep = _time_us(gscan, graph=single), _time_us(gprep, graph=single)
        nw = torch.ones(gv, device=dev)
        us_gout = _time_us(lambda: ops.gla_out(go, gproj, 2 * gh * gk + gh * gv, nw, 1e-6, torch.bfloat16), graph=single)
        gla_in = n * (2 * gh * gk + gh * gv + rk) * 2 + gp.numel() * 4

        def scan_row(kind, prep, state, heads, dk, dv, like_us):
            scan = lambda: ops.gla_scan(prep, state, step.req_q_start, step.req_q_len, step.req_slot, err)
            o = scan()
            us = _time_us(scan, graph=single)
            r = {"kernel": f"{kind} recurrence, {name}", "like": f"gla recurrence, {name}", "us": round(us, 1),
                 "like_us": round(like_us, 1),
                 "hbm_frac": round((2 * state.numel() * 4 + prep.numel() * 4 + o.numel() * 4) / (us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
                 "like_hbm_frac": round((2 * gstate.numel() * 4 + gp.numel() * 4 + go.numel() * 4) / (like_us * 1e-6) / 1e9 / peaks["hbm_gbs"], 4),
                 "fp32_tflops": round(4.0 * n * heads * dk * dv / (us * 1e-6) / 1e12, 2),
                 "like_fp32_tflops": round(4.0 * n * gh * gk * gv / (like_us * 1e-6) / 1e12, 2),
                 "note": "the same kernel: float32 on the CUDA cores, token by token"}
            rows.append(r)
            return o
        # HGRN2
        hproj, fb, lower = bf(n, 2 * gh * gk + gh * gv) * 0.5, f32(gh * gk), torch.rand(gh * gk, device=dev, generator=gen) * 0.9
        hprep = lambda: ops.hgrn2_prepare(hproj, fb, lower, dtype=torch.bfloat16, q_off=0, f_off=gh * gk, v_off=2 * gh * gk,
                                          heads=gh, key_dim=gk, value_dim=gv)
        hp = hprep()
        row(f"hgrn2 float32 inputs (silu q, bounded gate, 1 - gate, v), {name}", f"gla float32 inputs, {name}",
            _time_us(hprep, graph=single), us_gprep, nbytes=hproj.numel() * 2 + hp.numel() * 4, like_bytes=gla_in)
        ho = scan_row("hgrn2", hp, torch.zeros(n_req, gh, gk, gv, device=dev), gh, gk, gv, us_gscan)
        row(f"hgrn2 output norm, {name}", f"gla output norm + gate, {name}",
            _time_us(lambda: ops.gla_out(ho, None, 0, nw, 1e-6, torch.bfloat16), graph=single), us_gout,
            nbytes=n * gh * gv * (4 + 2), like_bytes=n * gh * gv * (4 + 2 + 2))
        # mLSTM
        mproj = bf(n, 2 * gh * gk + 2 * gh * gv + 2 * gh) * 0.5
        ib, fbm, mstate = f32(gh), f32(gh) + 3.0, torch.zeros(n_req, gh, device=dev)
        mprep = lambda: ops.mlstm_prepare(mproj, ib, fbm, mstate, step, dtype=torch.bfloat16, q_off=0, k_off=gh * gk,
                                          v_off=2 * gh * gk, i_off=2 * gh * gk + 2 * gh * gv, f_off=2 * gh * gk + 2 * gh * gv + gh,
                                          heads=gh, key_dim=gk, value_dim=gv, cap=15.0, q_scale=gk ** -0.5)
        mp, mg = mprep()
        row(f"mlstm float32 inputs (gates, running maximum, scaled q, k, v | 1), {name}", f"gla float32 inputs, {name}",
            _time_us(mprep, graph=single, iters=5 if not single else 20), us_gprep,
            nbytes=n * (2 * gh * gk + gh * gv + 2 * gh) * 2 + mp.numel() * 4, like_bytes=gla_in)
        mo = scan_row("mlstm", mp, torch.zeros(n_req, gh, gk, gv + 1, device=dev), gh, gk, gv + 1, us_gscan)
        nwm = torch.ones(gh * gv, device=dev)
        row(f"mlstm normaliser + unit norm + gate, {name}", f"gla output norm + gate, {name}",
            _time_us(lambda: ops.mlstm_out(mo, mg, mproj, 2 * gh * gk + gh * gv, nwm, 1e-6, torch.bfloat16), graph=single),
            us_gout, nbytes=n * gh * gv * (4 + 2 + 2))
        # the state-space half
        inner, cch = sh * sv, sh * sv + 2 * sn
        sproj = bf(n, inner + cch + sh) * 0.5
        taps_s, cb, ctail = f32(cch, 4) * 0.3, f32(cch) * 0.1, torch.zeros(n_req, 3, cch, device=dev)
        sconv = lambda: ops.short_conv(sproj, taps_s, ctail, step, dtype=torch.bfloat16, in_off=inner, channels=cch,
                                       bias=cb, silu=True, out_f32=True)
        xbc = sconv()
        row(f"state-space convolution + silu, {name}", None, _time_us(sconv, graph=single), 0.0, nbytes=n * cch * (2 + 4))
        dtb, alog, skip = f32(sh) * 0.5, f32(sh) * 0.5 - 1.0, f32(sh)
        sprep = lambda: ops.ssd_prepare(xbc, sproj, inner + cch, dtb, alog, dtype=torch.bfloat16, heads=sh, groups=1,
                                        state=sn, value_dim=sv)
        sp = sprep()
        row(f"state-space float32 inputs (dt, decay, B, C, dt x), {name}", f"gla float32 inputs, {name}",
            _time_us(sprep, graph=single), us_gprep, nbytes=xbc.numel() * 4 + sp.numel() * 4, like_bytes=gla_in)
        so = scan_row("state-space", sp, torch.zeros(n_req, sh, sn, sv, device=dev), sh, sn, sv, us_gscan)
        nws = torch.ones(inner, device=dev)
        row(f"state-space skip + gate + norm in groups + branch factor, {name}", f"gla output norm + gate, {name}",
            _time_us(lambda: ops.ssd_out(so, xbc, sproj, 0, skip, nws, 2, 1e-6, torch.bfloat16, out=wide[:, hq * d:hq * d + inner] if inner <= width else None,
                                         out_scale=0.5), graph=single),
            us_gout, nbytes=n * inner * (4 + 4 + 2 + 2), like_bytes=n * gh * gv * (4 + 2 + 2))
    assert err.tolist()[0] == 0, err.tolist()
    return rows


# --design pukinex: the Pukinex design beside a Ketalix model of equal layer sizes (the engine's closest other
# design: attention layers with a cap and a sink, recurrent layers on the same recurrence kernel, dense feed-forwards)

def pukinex_config(s: dict) -> dict:
    """Parallel layers (attention with a bucketed distance bias beside retention) and attention layers in turn,
    every layer with an ungated feed-forward that holds as many weights as the twin's gated one (ff * 3 / 2); two
    copies of the residual stream.  Attention heads as the twin's; retention has the twin's recurrent state
    (width / 256 heads, 128 x 256)."""
    w, d = s["width"], s["dim"]
    att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5 * 8.0, "softcap": 40.0,
           "rot": {"base": 1e4, "dims": d // 2, "scaling": {"factor": 4.0}}}
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5, "bias_max": 2048,
            "bias_buckets": 32, "q_temp": {"coef": 0.3, "every": 512}}
    heads = w // 256
    right = {"heads": heads, "dim": 128, "vdim": 256, "decay": [1.0 - 2.0 ** (-4 - (h % 5)) for h in range(heads)],
             "rot": {"base": 1e5, "dims": 128}}
    par = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.4}
    mlp = {"kind": "dense", "ff": s["ff"] * 3 // 2}
    layers = [{"type": "parallel" if i % 2 == 0 else "attention", "mixer": par if i % 2 == 0 else att, "mlp": mlp}
              for i in range(s["layers"])]
    return {"architecture": "Pukinex", "vocab": s["vocab"], "width": w, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "residual_mult": 0.8, "streams": 2, "logit_scale": 0.5, "logit_softcap": 25.0, "layers": layers}


def pukinex_kernels(s: dict, tokens: int, batch: int, ctx: int, peaks: dict) -> list[dict]:
    """Every kernel of the design alone, beside the like kernel of the Ketalix path at the same shape:
    time, achieved bytes or flops per second, and the fraction of the measured peak."""
    import torch
    from types import SimpleNamespace
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.attention import bucketed_distance_table, paged_attention
    from tokamak_b200.parts.base import linear
    from tokamak_b200.cache.device import KVView
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    hq, hkv, d, page, width = s["heads"], s["kv_heads"], s["dim"], 16, s["width"]
    ff, ff_twin = s["ff"] * 3 // 2, s["ff"]
    bf = lambda *shape: torch.randn(shape, device=dev, generator=gen).bfloat16()
    f32 = lambda *shape: torch.randn(shape, device=dev, generator=gen)
    rows = []

    def row(kernel, like, us, us_like, nbytes=0, flops=0.0, like_bytes=0, like_flops=0.0, note=""):
        r = {"kernel": kernel, "like": like, "us": round(us, 1), "like_us": round(us_like, 1) if us_like else None}
        for name, t, fl, nb in (("", us, flops, nbytes), ("like_", us_like, like_flops or flops, like_bytes or nbytes)):
            if not t:
                continue
            if fl:
                r[name + "bf16_frac"] = round(fl / (t * 1e-6) / 1e12 / peaks["bf16_tflops"], 4)
            elif nb:
                r[name + "hbm_frac"] = round(nb / (t * 1e-6) / 1e9 / peaks["hbm_gbs"], 4)
        if note:
            r["note"] = note
        rows.append(r)

    def step_of(n, n_req, start):
        per = n // n_req
        none = i32([])
        rec, n_parts, n_split = ops.prefill_tc_records([r * per for r in range(n_req)], [per] * n_req, [start + per] * n_req,
                                                       list(range(n_req)), heads=s["heads"], sms=ops.sm_count(torch.device(dev, 0)))
        return SimpleNamespace(
            decode_items=i32(list(range(n))) if per == 1 else none, prefill_items=none if per == 1 else i32(list(range(n))),
            prefill_tiles=none, prefill_tc=ops.PrefillItems(torch.from_numpy(rec).to(dev), n_parts, n_split),
            positions=i32([start + i for _ in range(n_req) for i in range(per)]),
            tok_req=i32([r for r in range(n_req) for _ in range(per)]), req_q_start=i32([r * per for r in range(n_req)]),
            req_q_len=i32([per] * n_req), req_kv_len=i32([start + per] * n_req), req_slot=i32(list(range(n_req))),
            err=err, max_q_len=per, n_tokens=n, n_reqs=n_req, scratch={}, max_kv_len=start + per)

    rel = f32(32, hq)
    dist = bucketed_distance_table(rel, 2048)
    unit, sinks = torch.zeros(hq, device=dev), f32(hq)
    cases = (("prompt", tokens, 1, 0), ("single tokens", batch, batch, ctx - 1))
    for name, n, n_req, start in cases:
        single = n_req > 1
        step = step_of(n, n_req, start)
        pages_req = -(-(start + n // n_req) // page)
        kc, vc = bf(n_req * pages_req, hkv, page, d), bf(n_req * pages_req, hkv, page, d)
        table = torch.randperm(n_req * pages_req, device=dev, generator=gen).to(torch.int32).view(n_req, pages_req)
        q = bf(n, hq, d)
        out = torch.empty_like(q)
        view = KVView(kc, vc, table, page, None)
        keys = n * (start + 1) if single else n * (n + 1) // 2
        # ---- attention with the bucketed distance bias and one in the denominator; the twin's has a cap and a sink
        mine = lambda: paged_attention(q, out, view, step, scale=d ** -0.5, window=None, sinks=unit, dist_bias=dist)
        like = lambda: paged_attention(q, out, view, step, scale=d ** -0.5, window=None, sinks=sinks, softcap=30.0)
        mine(); like()
        if single:
            row(f"attention (bucketed distance bias, unit sink), {name}", f"attention (cap, sink), {name}",
                _time_us(mine, graph=True), _time_us(like, graph=True), nbytes=2 * hkv * keys * d * 2 + 2 * q.numel() * 2)
        else:
            row(f"attention (bucketed distance bias, unit sink), {name}", f"attention (cap, sink), {name}",
                _time_us(mine, iters=5), _time_us(like, iters=5), flops=4.0 * keys * hq * d)
        # ---- q, k, v head by head: the left halves' form, the attention layers' form; the twin's pair rotation
        projl = bf(n, (2 * hq + 2 * hkv) * d)
        qb, kb, vb, qn, kn = f32(hq * d), f32(hkv * d), f32(hkv * d), f32(d), f32(d)
        left = lambda: ops.qkv_heads(projl, q, kc, vc, step, table, q_off=0, k_off=hq * d, v_off=(hq + hkv) * d, q_bias=qb,
                                     k_bias=kb, v_bias=vb, head_norm_eps=1e-5, q_norm=qn, k_norm=kn, temp_coef=0.3, temp_every=512)
        inv_half = (1.0 / (1e4 ** (torch.arange(0, d // 2, 2, dtype=torch.float32) / (d // 2))) / 4.0).to(dev)
        rot_half = ops.rope_table(step.positions, inv_half)
        proja = bf(n, (hq + hkv) * d + hq)
        attn = lambda: ops.qkv_heads(proja, q, kc, vc, step, table, q_off=0, k_off=hq * d, v_off=None, table=rot_half,
                                     rotary_dim=d // 2)
        qkv = bf(n, (hq + 2 * hkv) * d)
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(dev)
        rot = ops.rope_table(step.positions, inv_freq)
        vf, lam = f32(n, hkv * d), torch.full((1,), 0.3, device=dev)
        pairs = lambda: ops.qkv_pairs(qkv, q, kc, vc, step.positions, step.tok_req, step.req_slot, table, rot, err,
                                      n_q_heads=hq, n_kv_heads=hkv, rotary_dim=d, unit_norm_eps=1e-6, v_first_in=vf,
                                      v_lambda=lam, req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)
        nb = 2 * (hq + 2 * hkv) * d * n * 2
        us_pairs = _time_us(pairs, graph=single)
        row(f"biases + head norms + temperature + page write, {name}", f"pair rotation + unit norm + value blend + page write, {name}",
            _time_us(left, graph=single), us_pairs, nbytes=nb, like_bytes=nb + vf.numel() * 4)
        row(f"pair rotation on half a head + values from keys + page write, {name}",
            f"pair rotation + unit norm + value blend + page write, {name}", _time_us(attn, graph=single), us_pairs,
            nbytes=(2 * hq + 3 * hkv) * d * n * 2, like_bytes=nb + vf.numel() * 4)
        # ---- gates: per channel into the stacked rows (left half), per head (attention layers)
        att_rows = bf(n, hq * d)
        wide = torch.empty(n, hq * d + width, dtype=torch.bfloat16, device=dev)
        row(f"channel gate + branch factor into the stacked rows, {name}", None,
            _time_us(lambda: ops.gate_scale(att_rows, projl, 0, out=wide[:, :hq * d], scale=0.7),
                     graph=single), 0.0, nbytes=3 * n * hq * d * 2)
        row(f"head gate, {name}", None,
            _time_us(lambda: ops.gate_scale(att_rows, proja, (hq + hkv) * d, gate_group=d), graph=single), 0.0,
            nbytes=2 * n * hq * d * 2)
        # ---- the block's seats: write to two copies of the stream + read + layer norm; the twin's norm kernel
        streams, branch = f32(2, n, width), bf(n, width)
        mixm, wr, rd = f32(2, 2), f32(2), f32(2)
        w1, b1 = torch.ones(width, device=dev), torch.zeros(width, device=dev)
        resid = f32(n, width)
        normed = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
        row(f"write to 2 copies + read + layer norm, {name}", f"output norm + layer scale + residual + input norm, {name}",
            _time_us(lambda: ops.hyper_mix_norm(streams, branch, mix=mixm * 0.1, write=wr, read=rd, mult=0.8, norm_w=w1, norm_b=b1,
                                                eps=1e-5, dtype=torch.bfloat16), graph=single),
            _time_us(lambda: ops.branch_norm_add(resid, branch, w1, w1, 1e-6, w1, normed, 1e-6), graph=single),
            nbytes=n * width * (2 + 16 + 2), like_bytes=n * width * (2 + 8 + 2))
        # ---- the ungated feed-forward beside the twin's gated one of equal weights
        h = bf(n, width)
        w_up, w_down = bf(ff, width) * width ** -0.5, bf(width, ff) * ff ** -0.5
        wgu, wd = bf(2 * ff_twin, width) * width ** -0.5, bf(width, ff_twin) * ff_twin ** -0.5

        def mlp():         # as the part chooses
            if n <= 64:
                splits, stages, cluster = ops.swapped_gemm_plan(ff, width, n)
                a = ops.gemm_tc_swapped(w_up, h, err, splits, max_stages=stages, cluster=cluster, unary="relu2")
            elif ops.pair_gemm_takes(n, ff, width, fused=True):
                a = ops.gemm_pair(h, w_up, err, unary="relu2")
            else:
                a = ops.unary_act(linear(h, w_up, err=err), torch.bfloat16, "relu2")
            y = linear(a, w_down, err=err)
            ops.flush_chains()
            return y

        def gated():
            if n <= 64:
                splits, stages, cluster = ops.swapped_gemm_plan(2 * ff_twin, width, n)
                a = ops.gemm_tc_swapped(wgu, h, err, splits, max_stages=stages, cluster=cluster, swiglu=True, activation="gelu_tanh")
            elif ops.pair_gemm_takes(n, 2 * ff_twin, width, fused=True):
                a = ops.gemm_pair(h, wgu, err, swiglu=True, activation="gelu_tanh")
            else:
                gu = linear(h, wgu, err=err)
                a = torch.empty(n, ff_twin, dtype=torch.bfloat16, device=dev)
                ops.swiglu(gu, a, block=ops.SWIGLU_TILE_BLOCK, activation="gelu_tanh")
            y = linear(a, wd, err=err)
            ops.flush_chains()
            return y
        if single:
            row(f"feed-forward (up with relu squared in its epilogue, down), {name}", f"gated feed-forward of equal weights, {name}",
                _time_us(mlp, graph=True), _time_us(gated, graph=True), nbytes=2 * ff * width * 2, like_bytes=3 * ff_twin * width * 2)
        else:
            row(f"feed-forward (up with relu squared in its epilogue, down), {name}", f"gated feed-forward of equal weights, {name}",
                _time_us(mlp), _time_us(gated), flops=4.0 * n * ff * width, like_flops=6.0 * n * ff_twin * width)
        up_sums = linear(h, w_up, err=err)
        gu_twin, act_twin = bf(n, 2 * ff_twin), torch.empty(n, ff_twin, dtype=torch.bfloat16, device=dev)
        row(f"relu squared (the kernel of its own), {name}", f"gelu gate (the kernel of its own), {name}",
            _time_us(lambda: ops.unary_act(up_sums, torch.bfloat16, "relu2"), graph=single),
            _time_us(lambda: ops.swiglu(gu_twin, act_twin, block=ops.SWIGLU_TILE_BLOCK, activation="gelu_tanh"), graph=single),
            nbytes=up_sums.numel() * up_sums.element_size() + n * ff * 2, like_bytes=n * ff_twin * 3 * 2)
        # ---- retention beside gated linear attention: inputs, recurrence (the same kernel), output stage
        gh, gk, gv, rk = width // 256, 128, 256, 16
        gproj = bf(n, 2 * gh * gk + 2 * gh * gv + rk) * 0.5
        w2a, gbias = bf(gh * gk, rk) * 0.1, f32(gh * gk)
        gprep = lambda: ops.gla_prepare(gproj, 0, gh * gk, 2 * gh * gk, 2 * gh * gk + 2 * gh * gv, w2a, gbias, heads=gh,
                                        key_dim=gk, value_dim=gv, tau=16.0, q_scale=gk ** -0.5)
        gstate = torch.zeros(n_req, gh, gk, gv, device=dev)
        gp = gprep()
        gscan = lambda: ops.gla_scan(gp, gstate, step.req_q_start, step.req_q_len, step.req_slot, err)
        go = gscan()
        us_gscan, us_gprep = _time_us(gscan, graph=single), _time_us(gprep, graph=single)
        nw = torch.ones(gv, device=dev)
        us_gout = _time_us(lambda: ops.gla_out(go, gproj, 2 * gh * gk + gh * gv, nw, 1e-6, torch.bfloat16), graph=single)
        gla_in = n * (2 * gh * gk + gh * gv + rk) * 2 + gp.numel() * 4
        rproj = bf(n, 2 * gh * gk + 2 * gh * gv) * 0.5
        decay = torch.tensor([1.0 - 2.0 ** (-4 - (i % 5)) for i in range(gh)], device=dev)
        inv_r = (1.0 / (1e5 ** (torch.arange(0, gk, 2, dtype=torch.float32) / gk))).to(dev)
        rtab = ops.rope_table(step.positions, inv_r)
        rprep = lambda: ops.retention_prepare(rproj, decay, rtab, dtype=torch.bfloat16, q_off=0, k_off=gh * gk, v_off=2 * gh * gk,
                                              heads=gh, key_dim=gk, value_dim=gv, rotary_dim=gk, halves=True, k_scale=gk ** -0.5)
        rp = rprep()
        row(f"retention float32 inputs (rotation, scale, decay), {name}", f"gla float32 inputs, {name}",
            _time_us(rprep, graph=single), us_gprep, nbytes=n * (2 * gh * gk + gh * gv) * 2 + rp.numel() * 4, like_bytes=gla_in)
        rstate = torch.zeros(n_req, gh, gk, gv, device=dev)
        rscan = lambda: ops.gla_scan(rp, rstate, step.req_q_start, step.req_q_len, step.req_slot, err)
        ro = rscan()
        us_rscan = _time_us(rscan, graph=single)
        rows.append({"kernel": f"retention recurrence, {name}", "like": f"gla recurrence, {name}", "us": round(us_rscan, 1),
                     "like_us": round(us_gscan, 1),
                     "fp32_tflops": round(4.0 * n * gh * gk * gv / (us_rscan * 1e-6) / 1e12, 2),
                     "like_fp32_tflops": round(4.0 * n * gh * gk * gv / (us_gscan * 1e-6) / 1e12, 2),
                     "note": "the same kernel: float32 on the CUDA cores, token by token"})
        row(f"retention unit norm + silu gate + branch factor into the stacked rows, {name}", f"gla output norm + gate, {name}",
            _time_us(lambda: ops.gla_out(ro, rproj, 2 * gh * gk + gh * gv, None, 1e-5, torch.bfloat16,
                                         out=wide[:, hq * d:hq * d + gh * gv] if gh * gv <= width else None, out_scale=0.4),
                     graph=single), us_gout, nbytes=n * gh * gv * (4 + 2 + 2))
        # ---- scaled and capped logits (float32, in place)
        if single:
            logits = f32(n, s["vocab"])
            row(f"logit scale + cap, {name}", None, _time_us(lambda: ops.logits_scale_cap(logits, 0.5, 25.0), graph=True), 0.0,
                nbytes=2 * logits.numel() * 4)
    assert err.tolist()[0] == 0, err.tolist()
    return rows


DESIGNS = {
    "ketalix": dict(name="Ketalix", config=ketalix_config, twin=("qwen3_twin", qwen3_twin), kernels=ketalix_kernels),
    "logivik": dict(name="Logivik", config=logivik_config, twin=("ketalix_twin", ketalix_config), kernels=logivik_kernels),
    "tarivik": dict(name="Tarivik", config=tarivik_config, twin=("ketalix_twin", ketalix_config), kernels=tarivik_kernels),
    "pukinex": dict(name="Pukinex", config=pukinex_config, twin=("ketalix_twin", ketalix_config), kernels=pukinex_kernels),
}


def design_compare(args) -> int:
    """Prefill and decode throughput of a design beside the engine's closest other model of equal layer
    sizes (random weights), and the design's kernels alone beside their like kernels."""
    import torch
    from tokamak_b200.engine.core import random_core
    design = DESIGNS[args.design]
    s = KETALIX_SIZES[args.design_sizes]
    peaks = load_peaks()
    ctx, pf_tokens, batch = args.seq_len, args.prefill_tokens, args.batch
    global PROMPT_PORTION
    PROMPT_PORTION = args.prompt_tokens or pf_tokens
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    models = {}
    twin_name, twin_config = design["twin"]
    for name, raw, vocab in ((args.design, design["config"](s), s["vocab"]), (twin_name, twin_config(s), s["vocab"])):
        core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=max(ctx, pf_tokens), page_size=16,
                           pool_tokens=max(batch * ctx, pf_tokens + 64), max_slots=batch,
                           max_step_tokens=max(pf_tokens, batch * ctx))
        dec = time_decode(core, batch, args.steps, args.warmup, ctx, vocab)
        one = time_decode(core, 1, args.steps, args.warmup, ctx, vocab)
        pf_ms = time_prefill(core, vocab, pf_tokens)
        models[name] = {
            "decode_tok_s": round(dec["tok_s"], 1), "decode_ms_per_step": round(dec["ms_per_step"], 4),
            "decode_b1_tok_s": round(one["tok_s"], 1), "prefill_tok_s": round(pf_tokens / (pf_ms / 1e3), 1),
            "prefill_ms": round(pf_ms, 3), "checked": bool(dec["checked"] and one["checked"]),
            "graph_replays": dec["graph_replays"], "launches": dec["launches"],
            "weight_gb": round(weight_bytes(core) / 1e9, 3),
            "decode_hbm_frac": round((weight_bytes(core) + dec["kv_bytes"]) / (dec["ms_per_step"] / 1e3) / 1e9
                                     / peaks["hbm_gbs"], 4)}
        del core
        torch.cuda.empty_cache()
    kernels = design["kernels"](s, pf_tokens, batch, ctx, peaks)
    clocks = sampler.stop()
    print(json.dumps({"design": design["name"], "sizes": {**s, "name": args.design_sizes}, "batch": batch, "seq_len": ctx,
                      "prefill_tokens": pf_tokens, "steps": args.steps, "warmup": args.warmup, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random token ids", "models": models,
                      "kernels": kernels, "peaks": peaks, "clocks": clocks}))
    return 0 if all(m["checked"] for m in models.values()) else 1


def reference_main(args) -> int:
    """``--impl reference``: the unmodified reference from ``baseline/_ref`` on the same metric, or
    one line that says why it cannot run.  Everything it does is in ``baseline/reference_arm.py``."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm
    why = reference_arm.available()
    if why is None and args.gpus != 1:
        why = "the reference runs on one GPU only"
    if why is None and args.sizes not in SIZES:
        why = "--sizes 0.6b is for --workload throughput only"
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    model_name, sizes = SIZES[args.sizes]
    raw = dict(sizes)
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    try:
        config = bench_config(model_name, raw, sizes["num_hidden_layers"], args.batch, args.seq_len,
                              args.prefill_tokens, load_peaks()["source"])
        line = reference_arm.run(raw, model_name, args.batch, args.seq_len, args.prefill_tokens, max(1, args.steps),
                                 max(3, args.warmup), points=() if args.skip_points else tuple(args.points),
                                 clock_sampler=ClockSampler(0), config=config)
    except Exception as err:    # the reference's failure is reported, never hidden behind our numbers
        print(json.dumps({"impl": "reference", "unavailable": f"{type(err).__name__}: {str(err)[:300]}"}))
        return 0
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the 36 of Qwen3-8B")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out the further batch sizes")
    ap.add_argument("--points", type=lambda v: [int(x) for x in v.split(",") if x], default=[1, 64],
                    help="further decode batch sizes to time, comma-separated (default 1,64)")
    ap.add_argument("--sampling", default=None,
                    type=lambda v: tuple(float(x) for x in v.split(",")) if v else None,
                    help="temperature,top_k,top_p of the timed decode steps of the main batch (default: greedy), "
                         "e.g. 0.8,0,0.95; the points and the end-to-end run stay greedy")
    ap.add_argument("--kernel", default=None, help="time one kernel alone instead: attention_decode, attention_decode_split, "
                    "attention_prefill (tcgen05), attention_prefill_mma, rope_kv, rmsnorm, sampling (--batch rows, --sampling T,K,P), gemm_tc_decode, gemm_decode (library), "
                    "gemm_pair_swiglu, gemm_prefill_library (--ctx tokens), products_chain / products_separate (the four products "
                    "between two attentions of a decode step, as one kernel or one by one); attention_prefill_timeline prints the time stamps of the persistent prefill attention kernel's roles; tcgen05_probe prints what issuing a tcgen05.mma costs by shape and what a softmax warp needs for a key tile; decode_timeline prints when the blocks of every "
                    "kernel of a decode step run (needs a library built with TOKAMAK_B200_NVCC_FLAGS=-DTK_TIMELINE)")
    ap.add_argument("--ctx", type=int, default=CONTEXT, help="context length of a --kernel case")
    ap.add_argument("--workload", default=None, choices=["throughput", "latency", "mixed"],
                    help="run the reference's throughput workload through LLM.generate, or its single-sequence "
                         "latency measurement (512 prompt tokens, 128 greedy steps), or a mixed batch of 32 "
                         "requests (prompts of 128 to 4,096 tokens in portions of 512 beside decode tokens, 256 "
                         "new tokens each; --sizes 14b is the configuration it is named for), instead")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="portion size of --workload mixed")
    ap.add_argument("--portion", type=int, default=0,
                    help="query tokens per request of the attention_prefill kernel cases (the end of a context "
                         "of --ctx tokens; default: the whole context)")
    ap.add_argument("--sizes", default="8b", choices=["0.6b", "8b", "14b", "32b"],
                    help="layer sizes: of --workload (0.6b, 8b), or of the decode/prefill run (8b, the metric's "
                         "own, 14b, 32b)")
    ap.add_argument("--design", default=None, choices=["ketalix", "logivik", "tarivik", "pukinex"],
                    help="measure another design instead: its prefill and decode throughput beside the engine's closest "
                         "other model of equal layer sizes (Ketalix beside Qwen3, Logivik beside Ketalix), and its kernels "
                         "alone beside their like kernels (--design-sizes)")
    ap.add_argument("--design-sizes", default="2b", choices=sorted(KETALIX_SIZES))
    ap.add_argument("--num-requests", type=int, default=32)
    ap.add_argument("--max-new-cap", type=int, default=256)
    ap.add_argument("--kv-pool-tokens", type=int, default=16384)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=CONTEXT, help="context length at which the decode steps run")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt")
    ap.add_argument("--prompt-tokens", type=int, default=None,
                    help="length of the random prompts (and prompt portions) that fill the contexts before the "
                         "decode steps are timed (default: --prefill-tokens)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_main(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.design is not None:
        args.warmup, args.steps = warmup, steps
        return design_compare(args)
    if args.kernel == "decode_timeline":
        return decode_timeline(args.batch, args.layers or 3, args.ctx)
    if args.kernel == "tcgen05_probe":
        return tcgen05_probe()
    if args.kernel == "attention_prefill_timeline":
        return prefill_attention_timeline(args.batch, args.ctx, args.portion, args.sizes)
    if args.kernel:
        print(json.dumps(kernel_case(args.kernel, args.batch, args.ctx, steps, load_peaks(), args.portion, args.sizes,
                                     args.sampling)))
        return 0
    if args.workload == "latency":
        print(json.dumps(latency_workload(args.sizes, 512, 128, 3, args.seed)))
        return 0
    if args.workload == "mixed":
        print(json.dumps(mixed_workload(args.sizes, args.num_requests, args.max_new_cap, args.prefill_chunk,
                                        args.seed)))
        return 0
    if args.workload == "throughput":
        print(json.dumps(throughput_workload(args.sizes, args.num_requests, args.max_new_cap, args.batch,
                                             args.kv_pool_tokens, args.seed)))
        return 0

    import torch
    from tokamak_b200.engine.core import random_core

    if args.sizes not in SIZES:
        raise SystemExit("--sizes 0.6b is for --workload throughput only")
    model_name, sizes = SIZES[args.sizes]
    raw = dict(sizes)
    n_layers = args.layers or raw["num_hidden_layers"]
    raw["num_hidden_layers"] = n_layers
    vocab = raw["vocab_size"]
    peaks = load_peaks()
    ctx, pf_tokens = args.seq_len, args.prefill_tokens      # the defaults unless asked otherwise
    global PROMPT_PORTION
    PROMPT_PORTION = args.prompt_tokens or pf_tokens
    max_batch = max([args.batch, 1] + ([] if args.skip_points else list(args.points)))
    core = random_core(raw, seed=0, std=0.02, dtype="bfloat16", max_seq_len=max(ctx, pf_tokens), page_size=16,
                       pool_tokens=max(max_batch * ctx, pf_tokens + 64), max_slots=max_batch,
                       max_step_tokens=max(pf_tokens, args.batch * ctx))
    wbytes = weight_bytes(core)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    main_run = time_decode(core, args.batch, steps, warmup, ctx, vocab, args.sampling)
    prefill_ms = time_prefill(core, vocab, pf_tokens)
    points = {}
    checked = main_run["checked"]
    if not args.skip_points:
        for b in args.points:
            run = time_decode(core, b, steps, warmup, ctx, vocab)
            points[f"decode_b{b}"] = round(run["tok_s"], 1)
            checked = checked and run["checked"]
    e2e = time_e2e(core, args.batch, steps, warmup, ctx, vocab)
    clocks = sampler.stop()

    step_bytes = wbytes + main_run["kv_bytes"]
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    pf_flops = step_flops(raw, n_layers, pf_tokens)
    pf_frac = pf_flops / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12)
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name} layer sizes, context {ctx})",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "config": bench_config(model_name, raw, sizes["num_hidden_layers"], args.batch, ctx, pf_tokens,
                               peaks["source"]),
        "prompt_tokens": PROMPT_PORTION,
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(pf_tokens / (prefill_ms / 1e3), 1), "tokens": pf_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
        "host_ms_per_step": round(main_run["wall_ms_per_step"], 4),
        # every timed decode step's tokens equal those of the same steps run again kernel by kernel
        # (no CUDA graph, no step launched ahead, tokens fed by the host)
        "checked": checked,
        "device_step_h2d_bytes": round(main_run["h2d_bytes_per_step"], 1),
    }
    print(json.dumps(line))
    if not checked:
        print("bench.py: the timed decode steps produced other tokens than the same steps run "
              "kernel by kernel", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
