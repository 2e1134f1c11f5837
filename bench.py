#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the Qwen3-4B layer sizes with random weights (seeded normal(0, 0.02)),
bfloat16, 64 cache slots of 4,096 positions; 1,024-token prompts of seeded uniform
token ids are prefilled, then K decode steps are timed at batch 8 (``value``), and
at batch 1 and 64 (``points``); a 2,048-token prompt is prefilled (``prefill``). A
"step" is one decode step of the whole batch. One JSON line is printed.

* ``value``: decoded tokens per second, timed on the device with CUDA events around
  K steps that run without the host in between (captured step + selection kernel,
  which feeds the next step); the median of 5 such timed regions, with the clocks
  sampled during them. ``points`` and ``prefill`` carry clock records of their own.
* ``e2e``: the same through ``Engine.generate``: host token lists in, and every step's
  tokens (with the kernels' error word) read back to the host through pinned memory;
  at batch 8, and at batch 1 and 64 under ``e2e.points``.
* ``roofline``: bytes a decode step has to read (every weight once, the live
  requests' keys and values at the mean context of the timed steps) over its time,
  against the measured copy bandwidth.
* ``prefill.frac``: the step's flops over its time over the measured bfloat16 peak.

``--only workload_8b`` and ``--only workload_14b`` run the baseline's two larger
configurations (Qwen3-8B sizes: 8 prompts of 256 to 2,048 tokens, 128 greedy steps;
Qwen3-14B sizes: 16 prompts of 512 to 4,096 tokens, 128 steps at temperature 0.7)
through ``Engine.generate`` and print a short line of their own.

With --gpus above 1 it says that it runs on one GPU only and exits with 2.
--impl reference runs the unmodified reference from baseline/_ref (a copy of its
source tree: it is source-only, with no setup.py or pyproject.toml to install) on
the same workload through its own entry point and prints the same line; where that
copy, Triton or a CUDA device is missing it prints an ``unavailable`` line.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
PROMPT = 1024
PREFILL_TOKENS = 2048
SLOTS, CONTEXT = 64, 4096
REPEATS = 5  # timed regions per decode point; the median is reported
PREFILL_REPEATS = 15  # timed prefills (a quarter of a second: long enough for the clock sampler); the median is reported


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    out = {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "source": "fallback"}
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            if raw.get("hbm_gbs"):
                out["hbm_gbs"] = float(raw["hbm_gbs"])
            if raw.get("bf16_tflops"):
                out["bf16_tflops"] = float(raw["bf16_tflops"])
            out["source"] = "measured"
        except (ValueError, OSError):
            pass
    return out


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in text.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def timed_regions(steps_iter, warmup: int, steps: int, counter=None):
    """Consume a generator of decode steps: `warmup` untimed yields, then REPEATS regions of `steps`
    yields each, timed by the host's clock from the yield before a region to its last yield. Returns
    (median ms per step over the regions, mean of `counter`'s growth per step). As with the
    device-timed figure, the median keeps out the first region, which runs while the board's clocks
    still recover from the prompt step before it."""
    for _ in range(warmup):
        next(steps_iter)
    before = counter() if counter else 0
    times, total = [], 0
    for _ in range(REPEATS):
        t_start = time.perf_counter()
        n = 0
        for _ in steps_iter:
            n += 1
            if n == steps:
                break
        if n:
            times.append((time.perf_counter() - t_start) * 1000.0 / n)
            total += n
    for _ in steps_iter:  # nothing is left unless the generator yields more than asked
        pass
    grown = (counter() - before) / max(total, 1) if counter else 0.0
    return statistics.median(times), grown


def model_numbers(cfg, layers: int) -> dict:
    """Parameter bytes a decode step reads and flops per token of the linear layers."""
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    HQ, HKV, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    per_layer = (HQ + 2 * HKV) * D * H + H * HQ * D + 3 * I * H  # matrix elements
    norms = layers * (2 * H + 2 * D) + H
    head = V * H  # the output head; the embedding read is one row per token
    weight_bytes = 2 * (layers * per_layer + head + norms)
    kv_bytes_per_token = 2 * 2 * layers * HKV * D
    return {"per_layer": per_layer, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token,
            "head": head, "attn_dim": HQ * D}


WORKLOADS = {
    # the two larger configurations of the baseline: (preset, prompts, shortest, longest, steps, temperature, context)
    "workload_8b": ("qwen3_8b", 8, 256, 2048, 128, 0.0, 4096),
    "workload_14b": ("qwen3_14b", 16, 512, 4096, 128, 0.7, 8192),
}


def run_workload(args) -> dict:
    """One of the baseline's larger configurations end to end through ``Engine.generate``: an unequal batch
    of seeded prompts, then decode steps (greedy at the 8B sizes, temperature 0.7 at the 14B sizes), timed by
    the engine's own per-call statistics (host clock). Run twice; the second run is reported."""
    import torch

    from kernel_rush_kawk_b200 import Engine, Qwen3Config

    preset, n, shortest, longest, steps, temperature, context = WORKLOADS[args.only]
    base = Qwen3Config.preset(preset)
    layers = args.layers or base.num_hidden_layers
    cfg = Qwen3Config.from_dict({**base.to_dict(), "num_hidden_layers": layers})
    engine = Engine.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", max_slots=n, max_context=context,
                                max_tokens=n * context)
    gen = torch.Generator().manual_seed(4321)
    lengths = torch.randint(shortest, longest + 1, (n,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (k,), generator=gen).tolist() for k in lengths]
    for _ in range(2):
        produced = sum(1 for _ in engine.generate(prompts, steps, temperature=temperature, seed=7))
        torch.cuda.synchronize()
    st = engine.last_stats
    return {"only": args.only, "model": preset, "layers": layers, "layers_of_model": base.num_hidden_layers,
            "prompts": n, "prompt_tokens": st.prompt_tokens, "steps": produced, "temperature": temperature,
            "prefill_ms": round(st.prefill_ms, 2), "prefill_tokens_per_s": round(st.prefill_tokens_per_s, 1),
            "decode_ms_per_step": round(st.decode_ms_per_step, 4), "decode_tokens_per_s": round(st.decode_tokens_per_s, 1)}


def run_ours(args) -> dict:
    import torch

    from kernel_rush_kawk_b200 import Engine, Qwen3Config, StepEntry

    torch.cuda.set_device(0)
    base = Qwen3Config.preset("qwen3_4b")
    full_layers = base.num_hidden_layers
    layers = args.layers or full_layers
    cfg = Qwen3Config.from_dict({**base.to_dict(), "num_hidden_layers": layers})
    pk = peaks()
    t0 = time.time()
    engine = Engine.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", max_tokens=SLOTS * CONTEXT, max_slots=SLOTS,
                                max_context=CONTEXT)
    ops, cache, stepper = engine.ops, engine.cache, engine.stepper
    numbers = model_numbers(cfg, layers)
    gen = torch.Generator().manual_seed(1234)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def decode_point(batch: int, steps: int, warmup: int, repeats: int = REPEATS):
        """Prefill `batch` prompts, then time `steps` device-fed decode steps, `repeats` times over
        (the sequences grow on: each repeat starts where the one before ended; the mean context is
        that of all timed steps). Returns (tokens per second, median ms per step, launches per step,
        mean context, clock record)."""
        slots = [cache.alloc() for _ in range(batch)]
        sampler = ClockSampler()
        try:
            for i in range(0, batch, 8):  # prompts go in by eights to bound activation memory
                chunk = slots[i:i + 8]
                logits = engine.step([StepEntry(s, p, [PROMPT - 1]) for s, p in zip(chunk, prompts(len(chunk), PROMPT))])
                first = logits.argmax(dim=-1).tolist() if i == 0 else first + logits.argmax(dim=-1).tolist()
            toks = stepper.decode_on_device(slots, first, warmup)
            first = toks[-1].tolist()
            torch.cuda.synchronize()
            sampler.start()
            times, done = [], warmup
            before = ops.launches
            for _ in range(repeats):
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                toks = stepper.decode_on_device(slots, first, steps, first_step=done)
                end.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(end) / steps)
                first = toks[-1].tolist()
                done += steps
            clocks = sampler.stop()
            ms = statistics.median(times)
            graph_launches = stepper.graph_launches.get(batch, 0)
            launches = graph_launches + (ops.launches - before) / (steps * repeats)
            mean_ctx = PROMPT + warmup + (steps * repeats + 1) / 2
            return batch * 1000.0 / ms, ms, launches, mean_ctx, clocks
        finally:
            for s in slots:
                cache.free(s)

    def e2e_point(batch: int):
        """The same through ``Engine.generate``: host token lists in, host token lists out every step."""
        e2e_prompts = prompts(batch, PROMPT)
        it = engine.generate(e2e_prompts, args.warmup + REPEATS * args.steps)
        ms, copied = timed_regions(it, args.warmup, args.steps, stepper.h2d_total)
        return batch * 1000.0 / ms, ms, copied

    if args.only:  # one piece only, for profiling runs: prints a short line of its own
        if args.only == "prefill":
            prompt = prompts(1, PREFILL_TOKENS)[0]
            for _ in range(args.warmup + args.steps):
                slot = cache.alloc()
                torch.cuda.synchronize()
                t = time.perf_counter()
                engine.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
                torch.cuda.synchronize()
                ms = (time.perf_counter() - t) * 1e3
                cache.free(slot)
            return {"only": "prefill", "tokens": PREFILL_TOKENS, "ms_last": round(ms, 3), "layers": layers}
        b = int(args.only.split("_b")[1])
        v, ms_b, launches, _, _ = decode_point(b, args.steps, args.warmup, 1)
        return {"only": args.only, "value": round(v, 1), "ms_per_step": round(ms_b, 4), "launches_per_step": launches,
                "layers": layers}

    # -- headline: batch 8 -------------------------------------------------------
    value, ms_step, launches, mean_ctx, clocks = decode_point(8, args.steps, args.warmup)
    step_bytes = numbers["weight_bytes"] + 8 * mean_ctx * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # -- end to end through the entry point ---------------------------------------------
    # Each step's input is the step before's output, which the selection kernel hands on on the device; what
    # still travels from the host every step is the page table's growth (averaged here), and every step's
    # tokens travel back with the kernels' error word. The reference's loop does the same (engine.py:458-469).
    e2e_value, e2e_ms, e2e_h2d = e2e_point(8)
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": round(e2e_h2d, 1), "d2h_bytes_per_step": (8 + 1) * 4, "points": {},
           "inputs": "prompts as host token lists; a decode step's input is the step before's output, handed on on the device"}

    # -- the other batch sizes -------------------------------------------------------
    points, point_clocks = {}, {}
    for b in (1, 64):
        v, ms_b, _, ctx_b, ck = decode_point(b, args.steps, args.warmup)
        bytes_b = numbers["weight_bytes"] + b * ctx_b * numbers["kv_bytes_per_token"]
        points[f"decode_b{b}"] = round(v, 1)
        points[f"decode_b{b}_ms"] = round(ms_b, 4)
        points[f"decode_b{b}_hbm_frac"] = round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        point_clocks[f"decode_b{b}"] = ck
        e2e["points"][f"decode_b{b}"] = round(e2e_point(b)[0], 1)

    # -- prefill of 2,048 tokens ---------------------------------------------------------
    prompt = prompts(1, PREFILL_TOKENS)[0]
    times = []
    sampler = ClockSampler()
    sampler.start()
    for i in range(args.warmup + PREFILL_REPEATS):
        slot = cache.alloc()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        cache.free(slot)
        if i >= args.warmup:
            times.append(start.elapsed_time(end))
    point_clocks["prefill"] = sampler.stop()
    pre_ms = statistics.median(times)
    T = PREFILL_TOKENS
    flops = 2 * T * layers * numbers["per_layer"] + 2 * numbers["head"] + layers * 4 * numbers["attn_dim"] * T * (T + 1) / 2
    prefill = {"value": round(T * 1000.0 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    return {
        "metric": "decode tokens/s at batch 8 (Qwen3-4B shape, 1,024-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights normal(0, 0.02), seeded uniform token ids",
        "config": {"model": "qwen3-4b-shape", "layers": layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size, "q_heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab": cfg.vocab_size,
                   "tied_head": cfg.tie_word_embeddings, "global_batch": 8, "prompt_len": PROMPT,
                   "seq_len": CONTEXT, "slots": SLOTS, "parallelism": "1 GPU",
                   "l2": "inputs larger than L2: a step reads %.1f GB" % (step_bytes / 1e9),
                   "peaks": pk["source"], "hbm_peak_gbs": pk["hbm_gbs"], "bf16_peak_tflops": pk["bf16_tflops"]},
        "e2e": e2e, "gpu_launches": int(round(launches * args.steps)), "launches_per_step": round(launches, 1),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points, "clocks": clocks, "point_clocks": point_clocks, "repeats": REPEATS, "impl": "ours",
        "load_s": round(time.time() - t0, 1),
    }


def run_reference(args) -> dict:
    """The unmodified reference (a copy of its tree under baseline/_ref) on the same workload, through
    its own entry point: ``Engine(model_path).generate(input_ids, max_new_tokens)`` with equal-length
    prompts (engine/engine.py:480,590 of willzeng274/kernel-rush-kawk). Its own switches turn off the
    Transformers self-check and the token-recycling speculation (ENGINE_SELF_CHECK=0, ENGINE_RECYCLE=0,
    engine.py:490,502), which leaves plain greedy decoding by graph replay (GraphPlan.run, :438-469):
    the same work as this library's arm. Nothing of this package runs inside a timed region; it only
    writes the random model folder that the reference then loads."""
    import os
    import tempfile

    def unavailable(why: str) -> dict:
        return {"impl": "reference", "unavailable": why}

    ref_engine_dir = ROOT / "baseline" / "_ref" / "engine"
    if not (ref_engine_dir / "engine.py").is_file():
        return unavailable("no copy of the reference under baseline/_ref (it is source-only: a copy of its tree is its install)")
    if args.gpus != 1:
        return unavailable("the reference runs on one GPU only")
    try:
        import torch
        import triton  # noqa: F401  (the reference's kernels)
    except ImportError as exc:
        return unavailable(f"import failed: {exc}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    torch.cuda.set_device(0)

    from kernel_rush_kawk_b200 import Qwen3Config, write_model_folder

    base = Qwen3Config.preset("qwen3_4b")
    full_layers = base.num_hidden_layers
    layers = args.layers or full_layers
    cfg = Qwen3Config.from_dict({**base.to_dict(), "num_hidden_layers": layers})
    numbers = model_numbers(cfg, layers)
    pk = peaks()
    t0 = time.time()
    os.environ["ENGINE_SELF_CHECK"] = "0"
    os.environ["ENGINE_RECYCLE"] = "0"
    gen = torch.Generator().manual_seed(1234)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    with tempfile.TemporaryDirectory(prefix="krk_ref_model_") as tmp:
        folder = write_model_folder(Path(tmp) / "model", cfg, seed=0, std=0.02, device="cuda:0")
        torch.cuda.empty_cache()
        sys.path.insert(0, str(ref_engine_dir))
        try:
            import budget as ref_budget
            import engine as ref_engine  # baseline/_ref/engine/engine.py
            eng = ref_engine.Engine(str(folder))
        except Exception as exc:  # noqa: BLE001
            return unavailable(f"the reference failed to load: {exc!r}"[:300])
    if eng.fallback is not None or eng.model is None:
        return unavailable("the reference's own model failed to load here and it fell back to Transformers (see its log on stderr)")

    def plan_for(batch, length, new):
        ref_budget.start(ref_engine.PICKER_BUDGET_S)  # each shape gets the reference's whole tuning budget
        plan = eng._plan(batch, length, new)
        torch.cuda.synchronize()
        return plan

    def decode_point(batch: int):
        """(device-timed tokens/s, ms per step, end-to-end tokens/s, ms per step, clocks)."""
        total = args.warmup + REPEATS * args.steps
        ids = prompts(batch, PROMPT)
        for _ in eng.generate(ids, total):  # builds the plan, tunes, captures; one untimed sample
            pass
        if eng.fallback is not None:
            raise RuntimeError("the reference gave up on its own engine and fell back to Transformers")
        sampler = ClockSampler()
        sampler.start()
        e2e_ms, _ = timed_regions(eng.generate(ids, total), args.warmup, args.steps)
        # device-timed: the reference's captured decode step, replayed back to back
        plan = eng.plans[(batch, PROMPT)]
        plan.plan.ids.copy_(torch.tensor(ids, dtype=torch.int64))
        plan._step_prefill()
        for _ in range(args.warmup):
            plan._step_decode()
        times = []
        for _ in range(REPEATS):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(args.steps):
                plan._step_decode()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end) / args.steps)
        clocks = sampler.stop()
        ms = statistics.median(times)
        return batch * 1000.0 / ms, ms, batch * 1000.0 / e2e_ms, e2e_ms, clocks

    try:
        value, ms_step, e2e_value, e2e_ms, clocks = decode_point(8)
        mean_ctx = PROMPT + args.warmup + (args.steps * REPEATS + 1) / 2
        step_bytes = numbers["weight_bytes"] + 8 * mean_ctx * numbers["kv_bytes_per_token"]
        achieved = step_bytes / (ms_step * 1e-3) / 1e9
        points, e2e_points, point_clocks = {}, {}, {}
        for b in (1, 64):
            v, ms_b, ev, _, ck = decode_point(b)
            bytes_b = numbers["weight_bytes"] + b * mean_ctx * numbers["kv_bytes_per_token"]
            points[f"decode_b{b}"] = round(v, 1)
            points[f"decode_b{b}_hbm_frac"] = round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            e2e_points[f"decode_b{b}"] = round(ev, 1)
            point_clocks[f"decode_b{b}"] = ck
        plan = plan_for(1, PREFILL_TOKENS, 1)
        plan.plan.ids.copy_(torch.tensor(prompts(1, PREFILL_TOKENS), dtype=torch.int64))
        sampler = ClockSampler()
        sampler.start()
        times = []
        for i in range(args.warmup + PREFILL_REPEATS):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            plan._step_prefill()
            end.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(start.elapsed_time(end))
        point_clocks["prefill"] = sampler.stop()
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"the reference failed on this device: {exc!r}"[:300])
    pre_ms = statistics.median(times)
    T = PREFILL_TOKENS
    flops = 2 * T * layers * numbers["per_layer"] + 2 * numbers["head"] + layers * 4 * numbers["attn_dim"] * T * (T + 1) / 2
    prefill = {"value": round(T * 1000.0 / pre_ms, 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    return {
        "metric": "decode tokens/s at batch 8 (Qwen3-4B shape, 1,024-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights normal(0, 0.02), seeded uniform token ids",
        "config": {"model": "qwen3-4b-shape", "layers": layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size, "q_heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab": cfg.vocab_size,
                   "tied_head": cfg.tie_word_embeddings, "global_batch": 8, "prompt_len": PROMPT,
                   "parallelism": "1 GPU", "switches": "ENGINE_SELF_CHECK=0 ENGINE_RECYCLE=0",
                   "l2": "inputs larger than L2: a step reads %.1f GB" % (step_bytes / 1e9),
                   "peaks": pk["source"], "hbm_peak_gbs": pk["hbm_gbs"], "bf16_peak_tflops": pk["bf16_tflops"]},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8 * 8, "points": e2e_points},
        "gpu_launches": None, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points, "clocks": clocks, "point_clocks": point_clocks, "impl": "reference",
        "load_s": round(time.time() - t0, 1),
    }


def main() -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--only", default="", choices=["", "prefill", "decode_b1", "decode_b8", "decode_b16", "decode_b32", "decode_b64",
                                                  "workload_8b", "workload_14b"],
                   help="run one piece only (for profiling), or one of the baseline's larger configurations end to end")
    p.add_argument("--layers", type=int, default=0, help="run fewer layers than the model has (both numbers are reported)")
    args = p.parse_args()
    if args.impl == "reference":
        args.warmup = max(args.warmup, 3)
        print(json.dumps(run_reference(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py runs on one GPU only (this library has no multi-GPU path); got --gpus {args.gpus}")
        return 2
    args.warmup = max(args.warmup, 3)
    print(json.dumps(run_workload(args) if args.only in WORKLOADS else run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
