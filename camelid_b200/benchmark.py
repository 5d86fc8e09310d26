"""Measurement: decode tokens a second at a batch size, prefill tokens a second, the same
end to end through the Python entry point, and the fractions of the roofline.

Shapes are those of the benchmark configurations (Llama 3.2 1B, 3.2 3B, 3.1 8B) with random
weights drawn on the device; prompts are seeded uniform token ids. The reference's own
bench loads a model once and times generate runs (src/main.rs:4152-4274); its decode rate
leaves out the first token (src/main.rs:4229-4235), as the decode numbers here do.

Timing: CUDA events on the launching stream around exactly K decode steps after W warm-up
steps; every step reads all weights (gigabytes, far more than the 126 MB of L2), so the
inputs themselves are larger than L2. Clocks are sampled with nvidia-smi meanwhile.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
import time

import numpy as np
import torch

_ROPE_32 = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192}
SHAPES = {
    2: dict(name="llama-3.2-1b", num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
            head_dim=64, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0, rope_scaling=_ROPE_32,
            rms_norm_eps=1e-5, tie_word_embeddings=True, seed=2, context=4096),
    3: dict(name="llama-3.2-3b", num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
            head_dim=128, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0, rope_scaling=_ROPE_32,
            rms_norm_eps=1e-5, tie_word_embeddings=True, seed=3, context=4096),
    4: dict(name="llama-3.1-8b", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
            head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0,
            rope_scaling={**_ROPE_32, "factor": 8.0}, rms_norm_eps=1e-5, tie_word_embeddings=False, seed=4, context=8192),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def config_for(index: int, layers: int | None = None) -> dict:
    s = dict(SHAPES[index])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "max_position_embeddings": 131072,
           **{k: v for k, v in s.items() if k not in ("name", "seed", "context")}}
    if layers:
        cfg["num_hidden_layers"] = layers
    return cfg


def peaks(repo_root: str | None = None) -> dict:
    root = repo_root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.samples: list = []
        self.proc = None
        self.thread = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _prompts(rng, n: int, length, vocab: int) -> list:
    """``n`` prompts of seeded uniform ids; ``length`` is one number or (lowest, highest) for
    lengths drawn uniformly between the two."""
    if isinstance(length, (tuple, list)):
        lengths = rng.integers(int(length[0]), int(length[1]) + 1, size=n).tolist()
    else:
        lengths = [int(length)] * n
    return [rng.integers(0, vocab, size=t).tolist() for t in lengths]


def linear_params(cfg: dict) -> int:
    h, i, l = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    return l * (h * (q + 2 * kv) + q * h + 3 * h * i)


def prefill_flops(cfg: dict, tokens: int, wanted: int = 1) -> float:
    attn = 2.0 * tokens * tokens * cfg["num_attention_heads"] * cfg["head_dim"] * cfg["num_hidden_layers"]   # causal: half of 4 T^2
    return 2.0 * tokens * linear_params(cfg) + attn + 2.0 * wanted * cfg["hidden_size"] * cfg["vocab_size"]


def decode_bytes(cfg: dict, batch: int, context: float, elem: int) -> float:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    weights = (linear_params(cfg) + cfg["hidden_size"] * cfg["vocab_size"]
               + (2 * cfg["num_hidden_layers"] + 1) * cfg["hidden_size"]) * elem
    kv = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * elem * context * batch
    return weights + kv


def measure_prefill(lm, cfg, tokens: int, rng, reps: int = 5, warmup: int = 3) -> dict:
    from .engine.model import StepEntry
    cache = lm.new_cache(((tokens + 63) // 64) * 64, max_slots=1)
    prompt = _prompts(rng, 1, tokens, cfg["vocab_size"])[0]
    times = []
    for r in range(warmup + reps):
        slot = cache.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lm.step(cache, [StepEntry(slot, prompt, [tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        cache.free_slot(slot)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    del cache
    return {"ms": ms, "tokens": tokens, "value": tokens / (ms / 1e3)}


def measure_prefill_batch(lm, cfg, prompts, reps: int = 3, warmup: int = 2) -> dict:
    """All prompts of a batch, of unequal lengths, in one step."""
    from .engine.model import StepEntry
    cache = lm.new_cache(sum(((len(p) + 63) // 64) * 64 for p in prompts), max_slots=len(prompts))
    times = []
    for r in range(warmup + reps):
        slots = [cache.alloc_slot() for _ in prompts]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lm.step(cache, [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        b.record()
        torch.cuda.synchronize()
        for s in slots:
            cache.free_slot(s)
        if r >= warmup:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    del cache
    tokens = sum(len(p) for p in prompts)
    return {"ms": ms, "tokens": tokens, "value": tokens / (ms / 1e3), "prompts": len(prompts),
            "shortest": min(len(p) for p in prompts), "longest": max(len(p) for p in prompts),
            "flops": sum(prefill_flops(cfg, len(p)) for p in prompts)}


def _prefill_batch(lm, cache, prompts, chunk: int = 8):
    """Prefill all prompts (a few per step, to bound the workspace); returns slots and the
    greedy first token of each."""
    from .engine.model import StepEntry
    slots, firsts = [], []
    for i in range(0, len(prompts), chunk):
        part = prompts[i:i + chunk]
        s = [cache.alloc_slot() for _ in part]
        logits = lm.step(cache, [StepEntry(sl, p, [len(p) - 1]) for sl, p in zip(s, part)])
        firsts += logits.argmax(dim=-1).to(torch.int32).tolist()
        slots += s
    return slots, firsts


def measure_decode_device(lm, cfg, batch: int, prompt_tokens, steps: int, warmup: int, rng, prompts=None,
                          sampling=None) -> dict:
    """K decode steps timed on the device, in the loop that ``generate`` runs
    (``DecoderModel.decode_fed``): the captured step graph picks each token and feeds it back on the
    device; per step the host sends the positions from pinned memory and reads the chosen tokens.
    CUDA events bracket exactly the K steps. ``prompt_tokens`` is one length or (lowest, highest);
    ``prompts`` given wins over it. ``sampling`` (``SamplingOptions``): None is greedy; with penalties
    the prompts and what is generated are the histories."""
    from .csrc import ops
    if prompts is None:
        prompts = _prompts(rng, batch, prompt_tokens, cfg["vocab_size"])
    cache = lm.new_cache(sum(((len(p) + steps + warmup + 1 + 63) // 64) * 64 for p in prompts), max_slots=batch)
    slots, firsts = _prefill_batch(lm, cache, prompts)
    model = lm.model
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    adjusts = sampling is not None and sampling.adjusts
    with ClockSampler() as clocks:
        hist = [list(p) + [int(f)] for p, f in zip(prompts, firsts)] if adjusts else None
        warm = model.decode_fed(cache, slots, firsts, warmup, sampling, histories=hist)
        if adjusts:
            hist = [h + [int(t) for t in warm[:, j]] for j, h in enumerate(hist)]
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        ev0.record()
        model.decode_fed(cache, slots, warm[-1].tolist(), steps, sampling, histories=hist)
        ev1.record()
        torch.cuda.synchronize()
    launches = ops.launch_count() - launches0
    model.check_device_errors()
    ms = ev0.elapsed_time(ev1)
    h2d = model.last_h2d_bytes
    model.drop_graphs(cache)
    for s in slots:
        cache.free_slot(s)
    return {"ms_total": ms, "ms_per_step": ms / steps, "value": batch * steps / (ms / 1e3), "launches": launches,
            "h2d_bytes_per_step": h2d, "clocks": clocks.summary(),
            "context": sum(len(p) for p in prompts) / float(batch) + warmup + steps / 2.0}


def measure_decode_e2e(lm, cfg, batch: int, prompt_tokens, steps: int, warmup: int, rng, prompts=None) -> dict:
    """The same through ``LanguageModel.generate``, the call a user makes: every step sends its
    tokens and positions from pinned host memory and reads the sampled tokens back. Two calls
    on the same prompts, one that stops after the warm-up steps and one that goes on for
    ``steps`` more; the difference of their wall-clock times is the time of exactly those steps."""
    if prompts is None:
        prompts = _prompts(rng, batch, prompt_tokens, cfg["vocab_size"])

    def timed(n_tokens):
        best = None
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = lm.generate(prompts, max_tokens=n_tokens, stop_token_ids=())
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            assert all(len(o) == n_tokens for o in out)
            best = dt if best is None else min(best, dt)
        return best

    lm.generate(prompts, max_tokens=warmup + steps + 1, stop_token_ids=())        # graphs captured, buffers made
    short, long = timed(warmup + 1), timed(warmup + steps + 1)
    dt = long - short
    return {"value": batch * steps / dt, "ms_per_step": dt / steps * 1e3, "h2d_bytes_per_step": lm.model.last_h2d_bytes,
            "d2h_bytes_per_step": batch * 4}


FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12        # plain FMA on every lane of 148 SMs at 1,965 MHz: nominal, 74.4


SAMPLED = "temperature 0.8, top-k 40, top-p 0.9, repeat 1.1, presence 0.1"


def _sampled_options(cfg):
    from .sampling import SamplingOptions
    return SamplingOptions(temperature=0.8, top_k=40, top_p=0.9, seed=1, repeat_penalty=1.1,
                           presence_penalty=0.1).validate(cfg["vocab_size"])


def _roofline(cfg, batch, dec, elem, pk) -> dict:
    bytes_step = decode_bytes(cfg, batch, dec["context"], elem)
    achieved = bytes_step / (dec["ms_per_step"] / 1e3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
            "bytes": bytes_step}


def run(batch: int = 8, prompt_tokens: int = 2048, decode_steps: int = 256, warmup: int = 8, dtype: str = "bfloat16",
        layers: int | None = None, config_index: int = 2, points: bool = True, e2e: bool = True,
        prefill_tokens: int = 2048, prefill: bool = True, decode: bool = True, prompt_range=None,
        fp32: bool = False, fp32_steps: int = 32, sampled: bool = False) -> dict:
    """``prompt_range`` (lowest, highest): prompts of unequal lengths drawn uniformly between the
    two instead of ``prompt_tokens`` each; the record then also times their one prefill step.
    ``fp32``: the same decode step and prefill again with a float32 model, as an ``fp32`` object.
    ``sampled``: the timed decode steps pick their tokens with the stochastic sampler and its
    adjustments (``SAMPLED``) instead of the argmax; the record says so in ``config``."""
    from . import api
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    pk = peaks()
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype)
    rng = np.random.default_rng(shape["seed"])
    elem = 2 if dtype == "bfloat16" else 4
    flop_peak = (pk["bf16_tflops"] if dtype == "bfloat16" else FP32_TFLOPS) * 1e12
    def timed_prefill():
        if not prefill:
            return {"value": None, "tokens": prefill_tokens, "ms": None, "frac": None}
        pre = measure_prefill(lm, cfg, prefill_tokens, rng)
        pre["frac"] = prefill_flops(cfg, prefill_tokens) / (pre["ms"] / 1e3) / flop_peak
        return pre
    if not decode:
        return {"prefill": timed_prefill(), "dtype": dtype,
                "config": {"model": shape["name"], "layers": cfg["num_hidden_layers"]}}
    # The decode steps are timed first: seconds of dense prefill products put the GPU under its power cap,
    # and the steps right behind them would be timed at the clocks that leaves.
    prompts = _prompts(rng, batch, prompt_range, cfg["vocab_size"]) if prompt_range else None
    dec = measure_decode_device(lm, cfg, batch, prompt_tokens, decode_steps, warmup, rng, prompts=prompts,
                                sampling=_sampled_options(cfg) if sampled else None)
    pre = timed_prefill()
    pre_batch = None
    if prompts is not None and prefill:
        pre_batch = measure_prefill_batch(lm, cfg, prompts)
        pre_batch["frac"] = pre_batch.pop("flops") / (pre_batch["ms"] / 1e3) / flop_peak
    roof = _roofline(cfg, batch, dec, elem, pk)
    e2e_steps = max(decode_steps, 128)
    rec = {
        "metric": "decode tokens/s, Llama 3.2 1B shape, batch 8 (2048-token prompts)" if (config_index, batch) == (2, 8)
                  else f"decode tokens/s, {shape['name']} shape, batch {batch}",
        "value": dec["value"], "unit": "tokens/s", "n_gpus": 1, "steps": decode_steps, "warmup": warmup,
        "ms_per_step": dec["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == "bfloat16" else "fp32", "data": "synthetic (seeded uniform token ids, random weights)",
        "config": {"model": shape["name"], "global_batch": batch, "seq_len": shape["context"],
                   "prompt_tokens": prompt_tokens if prompts is None else f"uniform in {list(prompt_range)}",
                   "decode_steps": decode_steps, "parallelism": "single-gpu",
                   "layers": cfg["num_hidden_layers"], "layers_of_model": shape["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": cfg["tie_word_embeddings"], "weights": f"random, seed {shape['seed']}",
                   "l2": "inputs larger than L2 (every step reads all weights)", "peaks": pk["source"],
                   "e2e_steps": e2e_steps, "fp32_steps": fp32_steps if fp32 else 0,
                   **({"sampling": SAMPLED} if sampled else {})},
        "prefill": {"value": pre["value"], "tokens": pre["tokens"], "ms": pre["ms"], "frac": pre["frac"]},
        "roofline": {k: roof[k] for k in ("bound", "achieved", "peak", "unit", "frac")},
        "clocks": dec["clocks"], "gpu_launches": dec["launches"],
    }
    if pre_batch is not None:
        rec["prefill_batch"] = pre_batch
    if e2e:
        e = measure_decode_e2e(lm, cfg, batch, prompt_tokens, e2e_steps, warmup, rng, prompts=prompts)
        rec["e2e"] = {"value": e["value"], "unit": "tokens/s", "h2d_bytes_per_step": e["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": e["d2h_bytes_per_step"], "ms_per_step": e["ms_per_step"], "steps": e2e_steps}
    if points:
        pts, detail = {}, {}
        for b in (1, 64):
            d = dec if b == batch else measure_decode_device(lm, cfg, b, prompt_tokens, min(decode_steps, 64),
                                                             min(warmup, 4), rng)
            r = _roofline(cfg, b, d, elem, pk)
            pts[f"decode_b{b}"] = d["value"]
            detail[f"decode_b{b}"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "bytes": r["bytes"],
                                      "frac": r["frac"]}
        # the same steps with the stochastic sampler and its adjustments in the graph (not a key of `points`:
        # those are the two the contract names)
        d = measure_decode_device(lm, cfg, batch, prompt_tokens, min(decode_steps, 64), min(warmup, 4), rng,
                                  sampling=_sampled_options(cfg))
        detail[f"decode_b{batch}_sampled"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "sampling": SAMPLED}
        rec["points"] = pts
        rec["points_detail"] = detail
    if fp32 and dtype == "bfloat16":
        del lm
        torch.cuda.empty_cache()
        lm32 = api.from_random(cfg, seed=shape["seed"], dtype="float32")
        d = measure_decode_device(lm32, cfg, batch, prompt_tokens, fp32_steps, 3, rng)
        r = _roofline(cfg, batch, d, 4, pk)
        p32 = measure_prefill(lm32, cfg, prefill_tokens, rng, reps=3, warmup=3)
        rec["fp32"] = {"value": d["value"], "ms_per_step": d["ms_per_step"], "bytes": r["bytes"], "frac": r["frac"],
                       "steps": fp32_steps,
                       "prefill": {"value": p32["value"], "tokens": p32["tokens"], "ms": p32["ms"],
                                   "frac": prefill_flops(cfg, prefill_tokens) / (p32["ms"] / 1e3) / (FP32_TFLOPS * 1e12),
                                   "peak_tflops": FP32_TFLOPS}}
    return rec


def ablate_decode(batch: int = 8, prompt_tokens: int = 2048, dtype: str = "bfloat16", layers: int | None = None,
                  config_index: int = 2, reps: int = 50) -> dict:
    """Where a decode step's time goes: the captured step graph is timed whole, and again with
    one kind of kernel switched off at a time (the results are then wrong, only the time is
    read). The difference is what that kernel costs in place, inside the chain of dependent
    launches, which no profiler that serialises kernels can show."""
    from . import api
    from .csrc import ops
    from .engine.graphs import DecodeGraph, bucket_width
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype)
    rng = np.random.default_rng(0)
    cache = lm.new_cache(batch * (((prompt_tokens + 256 + 63) // 64) * 64), max_slots=batch)
    slots, firsts = _prefill_batch(lm, cache, _prompts(rng, batch, prompt_tokens, cfg["vocab_size"]))
    book = cache.book
    book.check_extend([(s, 128) for s in slots])
    starts = np.array([book.extend(s, 128) for s in slots], dtype=np.int32)

    def time_graph():
        widths = [bucket_width(max(len(book.pages[g][s]) for s in slots)) for g in range(len(book.kv_specs))]
        g = DecodeGraph(lm.model, cache, batch, widths, feed=True)
        i = g.fill(slots, starts, firsts)
        g.send(i, True)
        g.capture()
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return {"us_per_step": a.elapsed_time(b) / reps * 1e3, "launches": g.launches}

    def noop(*_a, **_k):
        return None

    real_gemm = ops.gemm_tc

    def gemm_without(pred):
        def f(a, b, c, epi, bn, splits, err):
            return None if pred(a, epi) else real_gemm(a, b, c, epi, bn, splits, err)
        return f

    hidden, inter = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
    out = {"full": time_graph()}
    for name in ("attn_decode_fused", "attn_paged_mma", "attn_paged_simt", "rope_kv_from_partials", "rope_kv_write", "rmsnorm",
                 "argmax_rows", "gemm_tn_simt"):
        real = getattr(ops, name)
        setattr(ops, name, noop)
        out["without " + name] = time_graph()
        setattr(ops, name, real)
    for label, pred in (("qkv product", lambda a, e: a.shape[0] == qkv and e == ops.TC_T_PARTIAL),
                        ("output product", lambda a, e: tuple(a.shape) == (hidden, cfg["num_attention_heads"] * cfg["head_dim"])),
                        ("gate-up product", lambda a, e: e == ops.TC_T_SWIGLU),
                        ("down product", lambda a, e: tuple(a.shape) == (hidden, inter)),
                        ("output head", lambda a, e: a.shape[0] == cfg["vocab_size"]),
                        ("any product", lambda a, e: True)):
        ops.gemm_tc = gemm_without(pred)
        out["without " + label] = time_graph()
    ops.gemm_tc = real_gemm
    full = out["full"]["us_per_step"]
    for k, v in out.items():
        v["cost_us"] = round(full - v["us_per_step"], 1)
        v["us_per_step"] = round(v["us_per_step"], 1)
    return {"batch": batch, "prompt_tokens": prompt_tokens, "dtype": dtype, "model": shape["name"],
            "layers": cfg["num_hidden_layers"], "steps": out}


def ablate_prefill(tokens: int = 2048, dtype: str = "bfloat16", layers: int | None = None, config_index: int = 2) -> dict:
    """Where a prefill step's time goes: the step of one prompt is timed whole (as
    ``measure_prefill`` does) and again with one kind of kernel switched off at a time; the
    results are then wrong, only the time is read. The difference is that kernel's cost in
    place, with programmatic dependent launch overlapping its neighbours."""
    from . import api
    from .csrc import ops
    from .options import KernelOptions
    shape = SHAPES[config_index]
    cfg = config_for(config_index, layers)
    # every step launched eagerly: a captured step would replay the kernels it was captured with
    lm = api.from_random(cfg, seed=shape["seed"], dtype=dtype, options=KernelOptions(capture_repeated_steps=False))
    rng = np.random.default_rng(0)

    def timed():
        return {"us_per_step": measure_prefill(lm, cfg, tokens, rng)["ms"] * 1e3}

    def noop(*_a, **_k):
        return None

    out = {"full": timed()}
    for name in ("attn_prefill_tc", "attn_paged_mma", "attn_paged_simt", "gemm_tn_simt", "rope_kv_write", "rmsnorm",
                 "embed_gather"):
        real = getattr(ops, name)
        setattr(ops, name, noop)
        out["without " + name] = timed()
        setattr(ops, name, real)
    real_pair, real_add_norm, real_gemm = ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm, ops.gemm_tc
    hidden, inter = cfg["hidden_size"], cfg["intermediate_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]

    def pair_without(pred):
        def f(a, b, c, epi, err, row_scale=None):
            return None if pred(b, epi) else real_pair(a, b, c, epi, err, row_scale)
        return f

    def add_norm_without(pred):
        def f(a, b, h, err, norm_w, eps, x_out, sumsq):
            if pred(b):
                return ops.RowScale(sumsq, b.shape[0], eps)
            return real_add_norm(a, b, h, err, norm_w, eps, x_out, sumsq)
        return f

    ops.gemm_tc_pair = pair_without(lambda b, e: b.shape[0] == qkv and e == ops.TC_STORE)
    out["without qkv product"] = timed()
    ops.gemm_tc_pair = pair_without(lambda b, e: e == ops.TC_SWIGLU)
    out["without gate-up product"] = timed()
    ops.gemm_tc_pair = real_pair
    o_shape = (hidden, cfg["num_attention_heads"] * cfg["head_dim"])
    ops.gemm_tc_pair_add_norm = add_norm_without(lambda b: tuple(b.shape) == o_shape)
    out["without output product (+ norm)"] = timed()
    ops.gemm_tc_pair_add_norm = add_norm_without(lambda b: tuple(b.shape) == (hidden, inter))
    out["without down product (+ norm)"] = timed()
    ops.gemm_tc_pair_add_norm = real_add_norm
    ops.gemm_tc = lambda *a, **k: None
    out["without output head"] = timed()
    ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm = pair_without(lambda b, e: True), add_norm_without(lambda b: True)
    out["without any product"] = timed()
    ops.gemm_tc_pair, ops.gemm_tc_pair_add_norm, ops.gemm_tc = real_pair, real_add_norm, real_gemm
    full = out["full"]["us_per_step"]
    for v in out.values():
        v["cost_us"] = round(full - v["us_per_step"], 1)
        v["us_per_step"] = round(v["us_per_step"], 1)
    return {"tokens": tokens, "dtype": dtype, "model": shape["name"], "layers": cfg["num_hidden_layers"], "steps": out}
