"""Measuring decode and prompt throughput of a model with random weights on one GPU.

The numbers the reference's benchmark reports per turn are context tokens, the time
to the first token and decode tokens a second = (tokens - 1) / (t_last - t_first)
(`cmd/enginebench/main.go:172-189`, `:315-336`; `bench/mlx.py:20-41`).  The same
two quantities are measured here on seeded synthetic tokens:

* decode: `batch` sequences are brought to the wanted context length by real prompt
  steps, then `warmup + steps` decode steps run; tokens stay on the device (the next
  token is picked there and fed to the next step) and the timed steps are bracketed by
  CUDA events.  Every step reads all weights and the cache of the live sequences, far
  more than the L2 holds, so nothing needs flushing between steps.
* end to end: the same through `Engine.generate`: per step the host sends the step's
  tables from pinned memory and reads the chosen tokens back.
* prompt: one step over a prompt of 2,048 tokens that returns the last logits.

Each comes with the fraction of its roofline: bytes that a decode step must read
(every weight once, and the cache of the live requests) over time against the HBM
copy bandwidth; the prompt step's floating-point operations over time against the
bfloat16 matrix peak.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_HERE)
# an earlier measurement on this kind of GPU: copy bandwidth, the library's bfloat16 product as a burst and sustained
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_config(name_or_path: str) -> dict:
    path = name_or_path if os.path.exists(name_or_path) else os.path.join(_HERE, "configs", name_or_path + ".json")
    with open(path) as f:
        return json.load(f)


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
               "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"])}
        return out, "measured"
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in a loop while a region is timed: SM clock and the reasons for slowing down."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------
# what a step must read and compute
# ---------------------------------------------------------------------------

def weight_bytes(model, itemsize: int = 2) -> int:
    """Bytes of every tensor a decode step reads once (the tied table counts once: the head reads all of
    it, the embedding a row per sequence)."""
    total = 0
    for spec in model.tensor_specs().values():
        n = 1
        for s in spec.shape:
            n *= s
        total += n * (4 if len(spec.shape) == 1 else itemsize)
    return total


def cache_bytes(model, lengths, itemsize: int = 2) -> int:
    """Bytes of cache that a decode step over sequences of these lengths reads: keys and values of every position
    a line keeps (a window of them for a windowed line), and every fixed-size state, whatever mixer asked for it."""
    from .cache.cache import KVNeed, StateNeed
    total = 0
    for needs in model.cache_line_needs():
        for need in (needs or {}).values():
            if isinstance(need, KVNeed):
                per_token = 2 * need.n_kv_heads * need.head_dim * itemsize
                total += sum(per_token * (min(n, need.window) if need.window else n) for n in lengths)
            elif isinstance(need, StateNeed):
                n = 1
                for d in need.shape:
                    n *= int(d)
                total += len(lengths) * n * torch.empty((), dtype=need.dtype).element_size()
    return total


def prefill_flops(model, n_tokens: int) -> float:
    """2 M N K of every product of a prompt step of n_tokens that asks for the last logits, plus what each
    layer's mixer says it computes beyond its products (attention: scores and weighted sums)."""
    flops = 0.0
    for name, spec in model.tensor_specs().items():
        if len(spec.shape) == 2 and name not in (getattr(model.embedding, "table_name", None),
                                                    getattr(model.head, "table_name", None)):       # (the head: below)
            flops += 2.0 * n_tokens * spec.shape[0] * spec.shape[1]
    for call in model.schedule:
        flops += float(model.blocks[call.layer].mixer.prompt_flops(n_tokens))
    flops += 2.0 * model.hidden * model.vocab          # the head, last position only
    return flops


# ---------------------------------------------------------------------------
# measurements
# ---------------------------------------------------------------------------

def _tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def uniform_lengths(n: int, lo: int, hi: int, seed: int) -> list[int]:
    """n seeded lengths, uniform in [lo, hi]."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def fill(engine, lengths, seed: int = 0) -> list[int]:
    """New sequences of these lengths, of seeded random tokens, by real prompt steps."""
    from .engine.step import StepEntry
    slots = [engine.alloc_slot() for _ in lengths]
    cur, cur_tok = [], 0
    batches = []
    for i, n in enumerate(lengths):
        if cur and cur_tok + n > engine.stepper.max_step_tokens:
            batches.append(cur)
            cur, cur_tok = [], 0
        cur.append(i)
        cur_tok += n
    batches.append(cur)
    for part in batches:
        engine.stepper.step([StepEntry(slots[i], _tokens(engine.model.vocab, lengths[i], seed + i), ()) for i in part])
    return slots


def measure_decode(engine, start_lengths, steps: int, warmup: int, sample_clocks: bool = False,
                   profile: bool = False, runs: int = 1) -> dict:
    """Decode tokens a second over sequences that hold `start_lengths` tokens before the first warm-up step
    (brought there by real prompt steps).  `runs` timed runs of exactly `steps` steps each, every one from the
    same lengths; the median run is reported (the reference's method: three runs, the median,
    `bench/mlx.py:41-46`).  `profile` opens the CUDA profiler range around the first two timed steps (for a
    profiler that was started with its capture off); the timing of such a run means nothing."""
    from .engine.step import StepEntry
    ops = engine.rt.ops
    batch = len(start_lengths)
    st = engine.stepper
    results = []
    clock_rows = None
    for run_no in range(max(1, runs)):
        slots = fill(engine, start_lengths)
        toks = st.token_buffer(batch)
        toks.copy_(torch.tensor(_tokens(engine.model.vocab, batch, 99), dtype=torch.int32))
        entries = [StepEntry(s, (0,), (0,)) for s in slots]
        history = torch.zeros((steps + warmup, batch), dtype=torch.int32, device=engine.rt.device)

        def one(i):
            logits = st.step(entries, copy=False, tokens_on_device=True)
            ops.argmax(logits, toks)                      # the next step's tokens, picked on the device
            history[i].copy_(toks)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.__enter__()
        e0.record()
        for i in range(steps):
            if profile and i == 0 and run_no == 0:
                torch.cuda.profiler.start()
            one(warmup + i)
            if profile and i == 1 and run_no == 0:
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
        e1.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.__exit__()
        results.append((e0.elapsed_time(e1), clocks, int(history.cpu().sum())))
        for s in slots:
            engine.free_slot(s)
    results.sort(key=lambda r: r[0])
    ms, clocks, checksum = results[len(results) // 2]
    per_step = st.launch_counter + 1                  # kernels of one replayed step, plus argmax
    mid = [n + warmup + steps // 2 for n in start_lengths]
    bytes_step = weight_bytes(engine.model) + cache_bytes(engine.model, mid)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "bytes_per_step": bytes_step,
            "gb_s": bytes_step / (ms / steps / 1e3) / 1e9, "gpu_launches": per_step * steps,
            "clocks": clocks.summary() if clocks else None, "tokens_checksum": checksum,
            "runs_ms_per_step": [round(r[0] / steps, 4) for r in results]}


def measure_e2e(engine, batch: int, context: int, steps: int, temp: float = 0.0, top_p: float = 1.0) -> dict:
    """The same through Engine.generate: token ids in from the host, token ids out to the host."""
    n_prompt = context - steps - 1
    prompts = [_tokens(engine.model.vocab, n_prompt, 1000 + i) for i in range(batch)]
    return measure_generate(engine, prompts, steps + 1, temp, top_p)


def measure_generate(engine, prompts, new_tokens: int, temp: float = 0.0, top_p: float = 1.0) -> dict:
    """Decode tokens a second of `Engine.generate` over these prompts, `new_tokens` each: the tokens after each
    request's first, over the time from the first token heard to the end (the reference's decode rate,
    `cmd/enginebench/main.go:172-189`), and the time to that first token."""
    t_first = [None]
    count = [0]

    def on_token(i, tok):
        if t_first[0] is None:
            torch.cuda.synchronize()
            t_first[0] = time.perf_counter()
        count[0] += 1

    # warm-up: the same call over the same lengths, so that every graph the timed call replays exists
    engine.generate(prompts, temp=temp, top_p=top_p, max_tokens=new_tokens, stop=())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, temp=temp, top_p=top_p, max_tokens=new_tokens, stop=(), on_token=on_token)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_first[0]
    return {"tok_s": (count[0] - len(prompts)) / dt, "h2d_bytes_per_step": engine.stepper.h2d_bytes,
            "d2h_bytes_per_step": 4 * len(prompts), "first_token_ms": (t_first[0] - t0) * 1e3}


def measure_prefill(engine, n_tokens: int, repeats: int = 5, warmup: int = 3, profile: bool = False) -> dict:
    from .engine.step import StepEntry
    times = []
    for r in range(warmup + repeats):
        slot = engine.alloc_slot()
        toks = _tokens(engine.model.vocab, n_tokens, 500 + r)
        torch.cuda.synchronize()
        last = profile and r == warmup + repeats - 1
        if last:
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.stepper.step([StepEntry(slot, toks, (n_tokens - 1,))])
        e1.record()
        torch.cuda.synchronize()
        if last:
            torch.cuda.profiler.stop()
        if r >= warmup:
            times.append(e0.elapsed_time(e1))
        engine.free_slot(slot)
    ms = float(np.median(times))
    return {"tok_s": n_tokens / (ms / 1e3), "ms": ms, "flops": prefill_flops(engine.model, n_tokens)}


def fp32_check(raw: dict, bf16_engine, n_tokens: int = 256, seed: int = 0) -> dict:
    """The logits at the end of a seeded prompt from the bfloat16 engine against a true 32-bit engine over the
    same weights: the largest difference as a fraction of the largest logit."""
    import janis_b200
    from .engine.step import StepEntry
    toks = _tokens(bf16_engine.model.vocab, n_tokens, 4242)
    slot = bf16_engine.alloc_slot()
    a = bf16_engine.step([StepEntry(slot, toks, (n_tokens - 1,))]).float().cpu()
    bf16_engine.free_slot(slot)
    ref = janis_b200.from_config(raw, seed=seed, dtype="float32", max_tokens=max(64, n_tokens), max_batch=1)
    slot = ref.alloc_slot()
    b = ref.step([StepEntry(slot, toks, (n_tokens - 1,))]).float().cpu()
    ref.close()
    return {"tokens": n_tokens, "max_err": round(float((a - b).abs().max()), 5),
            "scale": round(float(b.abs().max()), 3), "same_argmax": bool(a.argmax() == b.argmax())}


def _pretty(config: str) -> str:
    name = os.path.splitext(os.path.basename(config))[0]
    return "Gemma2-" + name[len("gemma2-"):].upper() if name.startswith("gemma2-") else name


def _frac(r: dict, pk: dict) -> float:
    return round(r["gb_s"] / pk["hbm_gbs"], 4)


def run(steps: int = 256, warmup: int = 8, batch: int = 8, context: int = 8192, config: str = "gemma2-2b",
        layers: int | None = None, points=(1, 64), prefill_tokens: int = 2048, e2e: bool = True,
        profile: str = "", runs: int = 3, workloads: bool = True, prompt_lengths=None) -> dict:
    """The whole benchmark; returns the record that bench.py prints as one JSON line.

    The headline is the median of `runs` runs of exactly `steps` decode steps at `batch` sequences whose cache
    reaches `context` tokens.  `points` adds decode at other batch sizes at the same context.  `workloads` adds
    the other measurements the configurations are quoted with: decode at batch 1, 8 and 64 from prompts of
    seeded lengths uniform in [128, 2048]; the 9B sizes generating 256 tokens each for an unequal batch of 8
    prompts of lengths uniform in [64, 4096] through `Engine.generate`; the 27B sizes' prompt step of 2,048
    tokens and decode at batch 1 and 16 from prompts of 1,024; each decode point with the fraction of the
    copy bandwidth that its own lengths give it; and the bfloat16 logits of the headline model against a true
    32-bit engine."""
    import janis_b200
    raw = load_config(config)
    full_layers = raw["num_hidden_layers"]
    if layers:
        raw = dict(raw, num_hidden_layers=int(layers))
    pk, pk_kind = peaks()
    max_batch = max([batch, *points, *((64,) if workloads else ())])
    room = max(context, prefill_tokens)                 # the prefill measurement needs its own length to fit
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=max_batch * room, max_batch=max_batch,
                                 max_context=room)
    start = context - steps - warmup
    if start < 1:
        raise ValueError("context too short for the steps asked")
    # (prompt_lengths = (lo, hi): the headline run decodes from prompts of seeded lengths uniform in [lo, hi] instead)
    starts = uniform_lengths(batch, prompt_lengths[0], prompt_lengths[1], 7 + batch) if prompt_lengths else [start] * batch
    main = measure_decode(eng, starts, steps, warmup, sample_clocks=True, profile=profile == "decode",
                          runs=1 if profile else runs)
    pre = measure_prefill(eng, prefill_tokens, profile=profile == "prefill")
    pts = {}
    for b in points:
        k = max(16, steps // 2)
        r = measure_decode(eng, [context - k - warmup] * b, k, warmup)
        pts[f"decode_b{b}"] = round(r["tok_s"], 1)
        pts[f"decode_b{b}_frac"] = _frac(r, pk)
    if workloads and not profile:
        for b in (1, 8, 64):                            # prompts of seeded lengths uniform in [128, 2048]
            r = measure_decode(eng, uniform_lengths(b, 128, 2048, 7 + b), 128, warmup, runs=3)
            pts[f"decode_b{b}_u2048"] = round(r["tok_s"], 1)
            pts[f"decode_b{b}_u2048_frac"] = _frac(r, pk)
    end = measure_e2e(eng, batch, context, steps) if e2e and not profile else None
    if end and workloads:                                # and with sampling instead of the highest logit
        pts["e2e_b%d_temp0.8_top_p0.95" % batch] = round(measure_e2e(eng, batch, context, steps, 0.8, 0.95)["tok_s"], 1)
    check = fp32_check(raw, eng) if workloads and not profile else None
    cfg = eng.config
    eng.close()
    del eng
    if workloads and not profile:
        pts.update(other_sizes(pk, warmup))
    rec = {
        "metric": "decode tok/s at batch %d (%s sizes, %s)" % (
            batch, _pretty(config), "prompts of %d to %d tokens" % tuple(prompt_lengths) if prompt_lengths else "context %d" % context),
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": config, "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "window": cfg.sliding_window, "global_batch": batch, "seq_len": context,
                   "context_len": context, "prefill_tokens": prefill_tokens, "weights": "random seed 0",
                   "parallelism": "single", "l2": "each step reads weights+cache >> L2",
                   "timed_runs": "median of %d" % (1 if profile else runs)},
        "clocks": main["clocks"], "gpu_launches": main["gpu_launches"], "runs_ms_per_step": main["runs_ms_per_step"],
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": prefill_tokens, "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(main["gb_s"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": _frac(main, pk), "peaks": pk_kind},
        "points": pts,
    }
    if end:
        rec["e2e"] = {"value": round(end["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": end["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": end["d2h_bytes_per_step"]}
    if check:
        rec["fp32_check"] = check
    return rec


def other_sizes(pk: dict, warmup: int = 8) -> dict:
    """The measurements quoted for the larger configurations (all of their layers, random weights):
    9B: an unequal batch of 8 prompts of seeded lengths uniform in [64, 4096], 256 tokens generated for each,
    through `Engine.generate` (host tokens in and out); 27B: the prompt step of 2,048 tokens, and decode at batch 1
    and 16 from prompts of 1,024 tokens."""
    import janis_b200
    out = {}
    raw = load_config("gemma2-9b")
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=8 * (4096 + 256 + 64), max_batch=8,
                                 max_context=8192)
    lens = uniform_lengths(8, 64, 4096, 5)
    prompts = [_tokens(eng.model.vocab, n, 3000 + i) for i, n in enumerate(lens)]
    g = measure_generate(eng, prompts, 256)
    out["gen_9b_b8_u4096_tok_s"] = round(g["tok_s"], 1)
    out["gen_9b_b8_u4096_first_token_ms"] = round(g["first_token_ms"], 1)
    mid = [n + 128 for n in lens]
    bytes_step = weight_bytes(eng.model) + cache_bytes(eng.model, mid)
    out["gen_9b_b8_u4096_frac"] = round(bytes_step * (g["tok_s"] / 8) / 1e9 / pk["hbm_gbs"], 4)
    eng.close()
    del eng
    raw = load_config("gemma2-27b")
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=16 * 2048, max_batch=16, max_context=8192)
    pre = measure_prefill(eng, 2048, repeats=3, warmup=2)
    out["prefill_27b_tok_s"] = round(pre["tok_s"], 1)
    out["prefill_27b_frac"] = round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
    for b in (1, 16):
        r = measure_decode(eng, [1024] * b, 64, warmup, runs=3)
        out[f"decode_27b_b{b}_p1024"] = round(r["tok_s"], 1)
        out[f"decode_27b_b{b}_p1024_frac"] = _frac(r, pk)
    eng.close()
    return out


# ---------------------------------------------------------------------------
# two designs side by side at equal layer sizes (`--compare sigalorn`)
# ---------------------------------------------------------------------------

class KernelTimer:
    """CUDA events around chosen functions of the kernels module while a step runs launch by launch: the device
    time of each, summed per name.  (Events between kernels keep a kernel's CTAs from arriving while its
    predecessor still runs, so a step timed this way is slower than the same step untimed; the shares are what
    is read.)"""

    def __init__(self, ops, names):
        self.ops, self.names = ops, [n for n in names if hasattr(ops, n)]
        self.events: dict[str, list] = {n: [] for n in self.names}
        self._orig = {}

    def __enter__(self):
        for n in self.names:
            orig = getattr(self.ops, n)
            self._orig[n] = orig

            def timed(*a, _orig=orig, _n=n, **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r = _orig(*a, **k)
                e1.record()
                self.events[_n].append((e0, e1))
                return r

            setattr(self.ops, n, timed)
        return self

    def __exit__(self, *exc):
        for n, orig in self._orig.items():
            setattr(self.ops, n, orig)
        return False

    def totals_us(self) -> dict:
        torch.cuda.synchronize()
        return {n: round(sum(a.elapsed_time(b) for a, b in ev) * 1e3, 1) for n, ev in self.events.items() if ev}


def sigalorn_like(gemma: dict, layers: int) -> dict:
    """A Sigalorn configuration with the layer sizes of a Gemma2 one: the same width, heads, head size (for keys
    and values), feed-forward width and vocabulary; attention blocks as long as Gemma2's window; layers alternate
    attention and gated linear attention (its key channels half the head size, at most 256), and the second
    attention layer of every four reads the keys and values of the first."""
    hd = int(gemma["head_dim"])
    att = {"heads": gemma["num_attention_heads"], "kv_heads": gemma["num_key_value_heads"], "dim": hd, "vdim": hd,
           "scale": hd ** -0.5, "rot": {"base": 10000.0, "dims": hd}, "mask": {"size": int(gemma.get("sliding_window", 4096))}}
    gla = {"heads": gemma["num_attention_heads"], "dim": min(256, hd // 2), "vdim": hd, "tau": 16.0, "rank": 64}
    mlp = {"kind": "dense", "ff": gemma["intermediate_size"]}
    out = []
    for i in range(layers):
        if i % 2:
            out.append({"type": "gla", "mixer": dict(gla), "mlp": dict(mlp)})
        elif i % 4 == 2:
            out.append({"type": "attention", "mixer": dict(att, kv_from=i - 2), "mlp": dict(mlp)})
        else:
            out.append({"type": "attention", "mixer": dict(att), "mlp": dict(mlp)})
    return {"architecture": "Sigalorn", "vocab": gemma["vocab_size"], "width": gemma["hidden_size"],
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "layers": out}


def nosolix_like(gemma: dict, layers: int) -> dict:
    """A Nosolix configuration with the layer sizes of a Gemma2 one: the same width, heads, head size (for keys and
    values), feed-forward width and vocabulary; layers alternate "parallel" (attention over Gemma2's window beside a
    state-space-duality mixer of twice the width in heads of 64 channels with 128 states) and "mamba1" (twice the
    width in channels, 16 states, step sizes through a rank of a sixteenth of the width); feed-forwards alternate
    dense and a mixture of 16 experts of a quarter of the dense width, 4 chosen from the best 2 of 4 groups, with a
    shared expert of that width: as many active feed-forward weights a token as the dense layer."""
    hd, W, ff = int(gemma["head_dim"]), int(gemma["hidden_size"]), int(gemma["intermediate_size"])
    left = {"heads": gemma["num_attention_heads"], "kv_heads": gemma["num_key_value_heads"], "dim": hd, "vdim": hd,
            "scale": hd ** -0.5, "mask": {"size": int(gemma.get("sliding_window", 4096))},
            "rot": {"base": 10000.0, "dims": hd, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": 2 * W // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}
    scan = {"inner": 2 * W, "state": 16, "dt_rank": max(8, W // 16), "conv": 4}
    e_ff = max(8, ff // 4 // 8 * 8)
    moe = {"kind": "moe", "expert": {"ff": e_ff, "limit": 7.0}, "shared": {"ff": e_ff, "limit": 7.0},
           "router": {"experts": 16, "top": 4, "scale": 1.0, "groups": {"count": 4, "keep": 2}}}
    out = []
    for i in range(layers):
        mixer = {"left": dict(left), "right": dict(right)} if i % 2 == 0 else dict(scan)
        mlp = {"kind": "dense", "ff": ff} if i % 4 < 2 else copy.deepcopy(moe)
        out.append({"type": "parallel" if i % 2 == 0 else "mamba1", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Nosolix", "vocab": gemma["vocab_size"], "width": W, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": out}


def vivazen_like(gemma: dict, layers: int) -> dict:
    """A Vivazen configuration with the layer sizes of a Gemma2 one: the same width, heads, head size (for keys and
    values), feed-forward width and vocabulary; layers alternate "attention" (Gemma2's heads and key/value heads, a
    filter of 4 taps, scores capped at 30, no window) and "latent_attention" (as many heads, each half the head size
    plain and a quarter rotated, values of half the head size, a compressed row as wide as one head, Gemma2's
    window); the last layer of every four runs the tensors of the one two before it."""
    hd, W, ff = int(gemma["head_dim"]), int(gemma["hidden_size"]), int(gemma["intermediate_size"])
    att = {"heads": gemma["num_attention_heads"], "kv_heads": gemma["num_key_value_heads"], "dim": hd, "vdim": hd,
           "scale": hd ** -0.5, "softcap": 30.0, "conv": 4}
    lat = {"heads": gemma["num_attention_heads"], "dim": hd // 2, "rot_dim": hd // 4, "vdim": hd // 2, "kv_rank": hd,
           "scale": (hd // 2 + hd // 4) ** -0.5, "mask": {"size": int(gemma.get("sliding_window", 4096))},
           "rot": {"base": 10000.0, "dims": hd // 4, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "dense", "ff": ff}
    out = []
    for i in range(layers):
        entry = {"type": "latent_attention" if i % 2 else "attention", "mixer": copy.deepcopy(lat if i % 2 else att), "mlp": dict(mlp)}
        if i % 4 == 3:
            entry["weights_of"] = i - 2
        out.append(entry)
    return {"architecture": "Vivazen", "vocab": gemma["vocab_size"], "width": W, "norm": {"eps": 1e-6, "groups": 8},
            "postln_alpha": 2.0, "layers": out}


def dekutar_like(gemma: dict, layers: int) -> dict:
    """A Dekutar configuration with the layer sizes of a Gemma2 one: the same width, heads, head size, and vocabulary; two
    copies of the stream; layers take turns as "latent_attention" (as many heads, each half the head size plain and a
    quarter rotated, values of half the head size, a compressed row as wide as one head, queries through a row of three
    heads' width), "attention" (Gemma2's heads and key/value heads, half the head turned, Gemma2's window with four kept
    first positions), "mlstm" (as many heads, key channels half the head size, at most 256, values of the head size) and
    "attention" again; every feed-forward is a mixture of 16 experts of a quarter of the dense width and 2 identity
    entries, 4 chosen, with a shared expert of that width: as many active feed-forward weights a token as the dense layer."""
    hd, W, ff = int(gemma["head_dim"]), int(gemma["hidden_size"]), int(gemma["intermediate_size"])
    H, G = gemma["num_attention_heads"], gemma["num_key_value_heads"]
    lat = {"heads": H, "dim": hd // 2, "rot_dim": hd // 4, "vdim": hd // 2, "kv_rank": hd, "q_rank": 3 * hd,
           "scale": (hd // 2 + hd // 4) ** -0.5, "rot": {"base": 10000.0, "dims": hd // 4}}
    att = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "rot": {"base": 10000.0, "dims": hd // 2},
           "mask": {"size": int(gemma.get("sliding_window", 4096)), "keep_first": 4}}
    mem = {"heads": H, "dim": min(256, hd // 2), "vdim": hd, "gate_cap": 10.0}
    e_ff = max(8, ff // 4 // 8 * 8)
    moe = {"kind": "moe", "expert": {"ff": e_ff}, "shared": {"ff": e_ff}, "router": {"experts": 16, "identity": 2, "top": 4}}
    kinds = (("latent_attention", lat), ("attention", att), ("mlstm", mem), ("attention", att))
    out = [{"type": kinds[i % 4][0], "mixer": copy.deepcopy(kinds[i % 4][1]), "mlp": copy.deepcopy(moe)} for i in range(layers)]
    return {"architecture": "Dekutar", "vocab": gemma["vocab_size"], "width": W, "streams": 2, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "logit_scale": 1.0, "layers": out}


_TIMED = {"sigalorn": ("talk_attention", "qkv_rotate_store", "gla_scan", "head_norm_gate", "bias_act", "add_rmsnorm", "rmsnorm"),
          "gemma2": ("attn_prefill", "attn_decode", "rope_store", "gemv_rope_store", "gated_act"),
          "nosolix": ("talk_attention", "qkv_rotate_store", "selective_scan", "causal_conv_silu", "gate_group_norm",
                      "moe_route", "moe_expert_act", "dyt_norm", "rmsnorm_accumulate", "sigmoid_gate", "bias_act"),
          "dekutar": ("talk_attention", "talk_attention_rows", "qk_rotate_norm_store", "latent_rotate_store", "head_linear", "mlstm_scan",
                      "head_norm_gate", "hc_update", "hc_read_norm", "hc_spread", "sigmoid_gate", "moe_route", "moe_expert_act",
                      "moe_identity_add", "rmsnorm"),
          "vivazen": ("talk_attention", "talk_attention_rows", "qkv_conv_norm_store", "latent_rotate_store", "head_linear", "group_norm", "round_rows",
                      "sigmoid_gate", "gated_act")}


def _leaf_mixers(mixer):
    branches = getattr(mixer, "branches", None)
    if not branches:
        yield mixer
        return
    for m in branches.values():
        yield from _leaf_mixers(m)


def _measure_design(raw: dict, kind: str, pk: dict, prefill_tokens: int, batch: int, context: int, steps: int,
                    warmup: int) -> dict:
    import janis_b200
    from .engine.step import StepEntry
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=batch * max(context, prefill_tokens) + 64,
                                 max_batch=batch, max_context=max(context, prefill_tokens))
    ops, model = eng.rt.ops, eng.model
    out = {"layers": len(model.schedule)}
    pre = measure_prefill(eng, prefill_tokens, repeats=3, warmup=2)
    out["prefill_tok_s"] = round(pre["tok_s"], 1)
    out["prefill_ms"] = round(pre["ms"], 3)
    out["prefill_frac_of_bf16_peak"] = round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
    dec = measure_decode(eng, [context - steps - warmup] * batch, steps, warmup)
    out["decode_tok_s"] = round(dec["tok_s"], 1)
    out["decode_ms_per_step"] = round(dec["ms_per_step"], 4)
    out["decode_frac_of_copy_bandwidth"] = _frac(dec, pk)
    # the kernels of one prompt step and of one decode step, launch by launch
    kernels = {}
    slot = eng.alloc_slot()
    with KernelTimer(ops, _TIMED[kind]) as kt:
        eng.stepper.step([StepEntry(slot, _tokens(model.vocab, prefill_tokens, 1), (prefill_tokens - 1,))])
    kernels["prefill_us"] = kt.totals_us()
    eng.free_slot(slot)
    slots = fill(eng, [context - 2] * batch)
    graphs, eng.stepper.use_graphs = eng.stepper.use_graphs, False
    entries = [StepEntry(s, (1,), (0,)) for s in slots]
    eng.stepper.step(entries)
    with KernelTimer(ops, _TIMED[kind]) as kt:
        eng.stepper.step(entries)
    kernels["decode_us"] = kt.totals_us()
    eng.stepper.use_graphs = graphs
    for s in slots:
        eng.free_slot(s)
    # what those kernels must compute or read, from the mixers' own account
    from .cache.cache import KVNeed, StateNeed
    att_flops = gla_flops = 0.0
    kv_bytes = state_bytes = 0
    for call in model.schedule:
        for mixer in _leaf_mixers(model.blocks[call.layer].mixer):
            for name, need in mixer.cache_needs().items():
                if isinstance(need, KVNeed):
                    att_flops += mixer.prompt_flops(prefill_tokens)
                    seen = min(context, need.window) if need.window else context
                    seen = min(seen, (context - 1) % mixer.block + 1) if getattr(mixer, "block", 0) else seen
                    seen = min(seen, mixer.window) if getattr(mixer, "window", 0) else seen
                    kv_bytes += batch * seen * need.n_kv_heads * (need.head_dim + need.value_dim) * 2
                elif isinstance(need, StateNeed) and name in ("state", "memory"):      # (a convolution's kept inputs are another kernel's)
                    gla_flops += mixer.prompt_flops(prefill_tokens)
                    state_bytes += 2 * batch * int(np.prod(need.shape)) * 4
                elif isinstance(need, StateNeed) and name in ("normaliser", "maximum"):   # the matrix memory's other parts
                    state_bytes += 2 * batch * int(np.prod(need.shape)) * 4
    att_name = "attn_prefill" if kind == "gemma2" else "talk_attention"
    dec_name = "attn_decode" if kind == "gemma2" else "talk_attention"
    if kernels["decode_us"].get("talk_attention_rows"):      # decode steps through the kernels that take single rows
        dec_name = "talk_attention_rows"
    scan_name = {"nosolix": "selective_scan", "dekutar": "mlstm_scan"}.get(kind, "gla_scan")
    roof = {}
    if kernels["prefill_us"].get(att_name):
        roof["attention_prefill_frac_of_bf16_peak"] = round(att_flops / (kernels["prefill_us"][att_name] * 1e-6) / (pk["bf16_tflops"] * 1e12), 5)
    dec_us = kernels["decode_us"].get(dec_name)
    if kind == "dekutar":       # its two attentions decode through different kernels: both kernels' time against both lines' bytes
        dec_us = (kernels["decode_us"].get("talk_attention") or 0.0) + (kernels["decode_us"].get("talk_attention_rows") or 0.0)
    if dec_us:
        roof["attention_decode_frac_of_copy_bandwidth"] = round(kv_bytes / (dec_us * 1e-6) / 1e9 / pk["hbm_gbs"], 5)
    if kernels["prefill_us"].get(scan_name):
        roof["recurrence_prefill_tflops_fp32"] = round(gla_flops / (kernels["prefill_us"][scan_name] * 1e-6) / 1e12, 3)
    if kernels["decode_us"].get(scan_name):
        roof["recurrence_decode_frac_of_copy_bandwidth"] = round(state_bytes / (kernels["decode_us"][scan_name] * 1e-6) / 1e9 / pk["hbm_gbs"], 5)
    # the elementwise kernels of a step against the bytes of the residual stream they pass over (one float32 read and
    # write and one activation written per norm): the norms' share, a number to set beside the other design's
    T = prefill_tokens
    for nm in ("dyt_norm", "add_rmsnorm", "group_norm"):
        if kernels["prefill_us"].get(nm):
            n_norm = sum(2 if getattr(model.blocks[c.layer], "feed_forward", None) is not None else 1 for c in model.schedule)
            roof[f"{nm}_prefill_frac_of_copy_bandwidth"] = round(n_norm * T * model.hidden * 10 / (kernels["prefill_us"][nm] * 1e-6) / 1e9 / pk["hbm_gbs"], 5)
    # the kernels between an attention's projection and its scores (rotate or filter, norm, write the cache line): the
    # projected rows read once and written once
    if kernels["prefill_us"].get("hc_update"):
        # the write of a sublayer's output into the copies of the stream with the next read: every copy read and written
        # as floats, the output read and the next input written in the activation type
        n_norm = sum(2 if getattr(model.blocks[c.layer], "feed_forward", None) is not None else 1 for c in model.schedule)
        copies = model.stream_width // model.hidden
        roof["hc_update_prefill_frac_of_copy_bandwidth"] = round(n_norm * T * model.hidden * (8 * copies + 4) / (kernels["prefill_us"]["hc_update"] * 1e-6) / 1e9 / pk["hbm_gbs"], 5)
    for nm in ("qkv_rotate_store", "qkv_conv_norm_store", "qk_rotate_norm_store"):
        if kernels["prefill_us"].get(nm):
            chans = 0
            for call in model.schedule:
                for mixer in _leaf_mixers(model.blocks[call.layer].mixer):
                    if hasattr(mixer, "n_kv_heads") and any(isinstance(n, KVNeed) for n in mixer.cache_needs().values()):
                        own = bool(getattr(mixer, "own_kv", True))
                        if (nm == "qk_rotate_norm_store") != bool(getattr(mixer, "values_from_keys", False)):
                            continue
                        chans += mixer.n_heads * mixer.key_dim + own * mixer.n_kv_heads * (mixer.key_dim + mixer.value_dim)
            for mode, rows_n in (("prefill", T), ("decode", batch)):
                if chans and kernels[f"{mode}_us"].get(nm):
                    roof[f"{nm}_{mode}_frac_of_copy_bandwidth"] = round(rows_n * chans * 4 / (kernels[f"{mode}_us"][nm] * 1e-6) / 1e9 / pk["hbm_gbs"], 5)
    out["kernels"] = kernels
    out["kernel_rooflines"] = roof
    eng.close()
    return out


def compare(sizes=("gemma2-2b", "gemma2-9b", "gemma2-27b"), layers: int = 4, prefill_tokens: int = 2048, batch: int = 8,
            context: int = 4096, steps: int = 64, warmup: int = 4, design: str = "sigalorn") -> dict:
    """Sigalorn beside Gemma2 at the layer sizes of the Gemma2 configurations, `layers` layers each, random
    weights: prompt tokens a second, decode tokens a second, and the device time of each design's own kernels in
    one prompt step and one decode step with what fraction of the roofline that is."""
    pk, pk_kind = peaks()
    rec = {"compare": f"{design} beside {'sigalorn' if design in ('nosolix', 'vivazen', 'dekutar') else 'gemma2'}", "dtype": "bf16", "data": "synthetic",
           "peaks": pk_kind, "prefill_tokens": prefill_tokens, "batch": batch, "context": context, "steps": steps, "sizes": {}}
    for name in sizes:
        gemma = dict(load_config(name), num_hidden_layers=layers)
        gemma.pop("layer_types", None)
        if design == "vivazen":      # beside the design whose attention runs through the same kernel
            rec["sizes"][name] = {
                "sigalorn": _measure_design(sigalorn_like(gemma, layers), "sigalorn", pk, prefill_tokens, batch, context, steps, warmup),
                "vivazen": _measure_design(vivazen_like(gemma, layers), "vivazen", pk, prefill_tokens, batch, context, steps, warmup)}
            continue
        if design == "dekutar":      # beside the design with the like kernels: attention through the same kernel, a matrix of state per head
            rec["sizes"][name] = {
                "sigalorn": _measure_design(sigalorn_like(gemma, layers), "sigalorn", pk, prefill_tokens, batch, context, steps, warmup),
                "dekutar": _measure_design(dekutar_like(gemma, layers), "dekutar", pk, prefill_tokens, batch, context, steps, warmup)}
            continue
        if design == "nosolix":      # beside the closest design the library has: recurrent layers between attention over a limited span
            rec["sizes"][name] = {
                "sigalorn": _measure_design(sigalorn_like(gemma, layers), "sigalorn", pk, prefill_tokens, batch, context, steps, warmup),
                "nosolix": _measure_design(nosolix_like(gemma, layers), "nosolix", pk, prefill_tokens, batch, context, steps, warmup)}
            continue
        rec["sizes"][name] = {
            "gemma2": _measure_design(gemma, "gemma2", pk, prefill_tokens, batch, context, steps, warmup),
            "sigalorn": _measure_design(sigalorn_like(gemma, layers), "sigalorn", pk, prefill_tokens, batch, context, steps, warmup)}
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="janis bench")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256,
                    help="timed decode steps (0.6 s at the default sizes: several clock samples, and the first and last step of the end-to-end run weigh little)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="janis_b200")
    ap.add_argument("--batch", default="8", help="sequences decoded together; a list (8,1,64) also times the others")
    ap.add_argument("--context", "--ctx", dest="context", type=int, default=8192)
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prompt step")
    ap.add_argument("--json", action="store_true", help="accepted for familiarity: the record is always one JSON line")
    ap.add_argument("--config", default="gemma2-2b", help="2b, 9b, 27b, gemma2-2b ... or a config.json")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-workloads", action="store_true",
                    help="leave out the unequal-length decode points, the 9B and 27B measurements and the 32-bit check")
    ap.add_argument("--runs", type=int, default=3, help="timed runs of the headline; the median is reported")
    ap.add_argument("--prompt-lengths", default="", help="LO,HI: decode from prompts of seeded lengths uniform in [LO, HI] "
                    "instead of sequences that all reach --context")
    ap.add_argument("--profile", choices=["decode", "prefill"], default="",
                    help="open the CUDA profiler range around two timed decode steps, or the last prompt step")
    ap.add_argument("--compare", choices=["sigalorn", "nosolix", "vivazen", "dekutar"], default="",
                    help="instead of the benchmark: Sigalorn beside Gemma2, or Nosolix, Vivazen or Dekutar beside Sigalorn, at equal layer "
                    "sizes (prompt and decode throughput, and each design's own kernels against their rooflines); "
                    "--config picks one size")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Go module (no Go toolchain here, "
                          "nothing pip can install) and its Gemma2 loads MLX 4-bit checkpoints on Apple hardware only"}))
        return 0
    if a.gpus != 1:
        print(f"janis_b200 is a one-GPU library: --gpus {a.gpus} is not supported")
        return 2
    if a.compare:
        sizes = ("gemma2-2b", "gemma2-9b", "gemma2-27b") if a.config == "gemma2-2b" and "--config" not in (argv or sys.argv) \
            else ((a.config if a.config.startswith("gemma2-") else "gemma2-" + a.config),)
        print(json.dumps(compare(sizes, a.layers or 4, a.prefill, int(str(a.batch).split(",")[0]), min(a.context, 4096),
                                 min(a.steps, 64), max(3, min(a.warmup, 8)), a.compare)))
        return 0
    try:
        batches = [int(b) for b in str(a.batch).split(",") if b.strip()]
    except ValueError:
        batches = []
    if not batches or min(batches) < 1:
        print(f"--batch wants positive integers, found {a.batch!r}")
        return 2
    points = tuple(batches[1:]) if len(batches) > 1 else (1, 64)
    config = a.config if (os.path.exists(a.config) or a.config.startswith("gemma2-")) else "gemma2-" + a.config
    rec = run(a.steps, max(3, a.warmup), batches[0], a.context, config, a.layers or None,
              points=() if (a.no_points or a.profile) else points, prefill_tokens=a.prefill, profile=a.profile,
              runs=max(1, a.runs), workloads=not (a.no_workloads or a.no_points) and config == "gemma2-2b" and not a.layers,
              prompt_lengths=tuple(int(v) for v in a.prompt_lengths.split(",")) if a.prompt_lengths else None)
    print(json.dumps(rec))
    return 0
