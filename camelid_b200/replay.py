"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and has no forward pass, cache or loader of its own: it drives the
library's model, step function, cache and kernels, the ones that generation uses. Steps come
on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the places among them whose logits are
wanted; ``end`` names requests that are finished after the step (their slot and pages are
given back). For a step that wants something, ``<out>/<step>.f32`` holds the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32
[wanted, vocab]. After every step a line ``done <step>`` is printed and flushed. The
reference's precedents are its forced-token harness with per-step logit dumps
(src/main.rs:667-681, :7208-7350) and examples/parity_node.rs:184-211.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def add_arguments(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions that serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each request rounded up to a multiple of 64")


def run(args, stdin=None, stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    print("[trace_run] loading the library ...", file=sys.stderr, flush=True)
    import torch
    from .api import load
    from .engine.model import StepEntry

    os.makedirs(args.out, exist_ok=True)
    lm = load(args.model, dtype=args.dtype, device="cuda")
    cache = lm.new_cache(args.max_tokens)
    print(f"[trace_run] model loaded; cache of {cache.book.n_pages} pages ({cache.bytes} bytes)",
          file=sys.stderr, flush=True)
    slots: dict = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries, fresh = [], []
        try:
            for e in rec.get("entries", []):
                rid = e["id"]
                if rid not in slots:
                    slots[rid] = cache.alloc_slot()
                    fresh.append(rid)
                entries.append(StepEntry(slots[rid], e["tokens"], e.get("want", [])))
            if entries:
                logits = lm.step(cache, entries)
                if logits.shape[0]:
                    data = logits.to("cpu").contiguous().numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f"{step}.f32.tmp")
                    data.tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
                else:
                    torch.cuda.synchronize()
            for rid in rec.get("end", []):
                if rid in slots:
                    cache.free_slot(slots.pop(rid))
        except Exception:
            for rid in fresh:                       # a refused step leaves nothing behind
                if rid in slots:
                    cache.free_slot(slots.pop(rid))
            raise
        print(f"done {step}", file=stdout, flush=True)
    lm.model.check_device_errors()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay a token trace through the model and write logits")
    add_arguments(ap)
    return run(ap.parse_args(argv))
