"""The ``camelid`` command line.

    camelid generate MODEL [--prompt "5 17 3" | --prompt-file F] [--max-tokens 128]
                     [--temperature 0] [--top-k K] [--top-p P] [--min-p P] [--seed S] ...
    camelid bench-generate ...   the same, one JSON object per iteration on stdout
    camelid replay --model DIR --dtype T --out DIR --max-tokens N     (bin/trace_run)
    camelid bench [--batch 8] [--prompt-tokens 2048] [--decode-steps 256] ...
    camelid random-model CONFIG.json OUT --seed S
    camelid memory MODEL_OR_CONFIG --dtype T --max-tokens N [--max-slots S]     bytes of weights, cache, workspace

Option names and meanings are the reference's where it has them: ``bench-generate MODEL
--prompt-file --prompt --max-tokens (128) --temperature (0.0) --iterations (1) --warmup
--json --deterministic`` (src/main.rs:956-990), ``--top-p --top-k --seed``
(src/main.rs:401-417); the JSON record has its fields (src/main.rs:3216-3240), with
tokens_per_second = (generated - 1) / decode seconds (src/main.rs:4229-4235). Prompts are
token ids, since tokenizers are outside this library: ``--prompt`` takes ids separated by
blanks or commas, ``--prompt-file`` a JSON array of ids (or of several such arrays), or one
id per line (the format of the reference's ``--force-tokens``, src/main.rs:667-681).
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def read_prompts(args) -> list:
    if args.prompt_file:
        text = open(args.prompt_file).read().strip()
        try:
            data = json.loads(text)
        except json.JSONDecodeError:
            data = [int(x) for x in text.replace(",", " ").split()]
        if data and isinstance(data[0], list):
            return [[int(t) for t in p] for p in data]
        return [[int(t) for t in data]]
    if args.prompt:
        return [[int(x) for x in args.prompt.replace(",", " ").split()]]
    raise SystemExit("give --prompt or --prompt-file (token ids)")


def _generate_args(ap):
    ap.add_argument("model", help="model folder (config.json, model.safetensors)")
    ap.add_argument("--prompt-file", help="token ids: a JSON array (or array of arrays), or one id per line; wins over --prompt")
    ap.add_argument("--prompt", help="token ids separated by blanks or commas")
    ap.add_argument("--max-tokens", type=int, default=128, help="maximum tokens to generate per iteration")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature (0 = greedy/argmax, deterministic)")
    ap.add_argument("--top-p", type=float, default=None, help="nucleus sampling top-p (omit to leave unset)")
    ap.add_argument("--top-k", type=int, default=None, help="top-k sampling (omit to leave unset)")
    ap.add_argument("--min-p", type=float, default=None, help="keep tokens with p >= min_p * p_max")
    ap.add_argument("--seed", type=int, default=None, help="sampling seed (omit for the engine default, 0)")
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--stop-ids", default=None, help="stop token ids, comma separated (default: the model's eos ids)")
    ap.add_argument("--iterations", type=int, default=1, help="number of measured iterations (one JSON object each)")
    ap.add_argument("--warmup", action="store_true", help="run one unmeasured generation before the measured ones")
    ap.add_argument("--json", action="store_true", help="print the JSON record instead of the bare token ids")
    ap.add_argument("--deterministic", action="store_true",
                    help="run the true 32-bit path (the same as --dtype float32)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--random", action="store_true",
                    help="MODEL is a config.json: draw random weights for it on the device (see --weights-seed)")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights with --random")


def cmd_generate(args, always_json=False) -> int:
    import torch
    from . import api
    t0 = time.perf_counter()
    dtype = "float32" if args.deterministic else args.dtype
    if args.random:
        with open(args.model) as f:
            lm = api.from_random(json.load(f), args.weights_seed, dtype=dtype)
    else:
        lm = api.load(args.model, dtype=dtype)
    torch.cuda.synchronize()
    load_ms = (time.perf_counter() - t0) * 1e3
    prompts = read_prompts(args)
    stops = None if args.stop_ids is None else tuple(int(x) for x in args.stop_ids.split(",") if x.strip())
    opts = dict(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, seed=args.seed,
                repeat_penalty=args.repeat_penalty, presence_penalty=args.presence_penalty,
                frequency_penalty=args.frequency_penalty, stop_token_ids=stops)
    if args.warmup:
        lm.generate(prompts, max_tokens=args.max_tokens, **opts)
    for _ in range(args.iterations):
        torch.cuda.reset_peak_memory_stats()
        torch.cuda.synchronize()
        stamps = []
        t1 = time.perf_counter()
        out = lm.generate(prompts, max_tokens=args.max_tokens, on_step=lambda _live: stamps.append(time.perf_counter()),
                          **opts)
        torch.cuda.synchronize()
        # the first stamp is taken when the prompts have run and the first tokens are on the host
        ttft_ms = (stamps[0] - t1) * 1e3 if stamps else 0.0
        decode_ms = (stamps[-1] - stamps[0]) * 1e3 if len(stamps) > 1 else 0.0
        generated = sum(len(o) for o in out)
        rec = {
            "prompt_tokens": sum(len(p) for p in prompts), "generated_tokens": generated,
            "load_ms": load_ms, "prefill_ms": ttft_ms, "ttft_ms": ttft_ms, "decode_ms": decode_ms,
            "tokens_per_second": (generated - len(out)) / (decode_ms / 1e3) if decode_ms > 0 else 0.0,
            "peak_memory_bytes": torch.cuda.max_memory_allocated(),
            "output_token_ids": out[0] if len(out) == 1 else out, "dtype": dtype,
        }
        if args.json or always_json:
            print(json.dumps(rec), flush=True)
        else:
            for o in out:
                print(" ".join(str(t) for t in o), flush=True)
    return 0


def cmd_random_model(args) -> int:
    import torch
    from .weights.random_init import write_random_model
    with open(args.config) as f:
        cfg = json.load(f)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, cfg, args.seed, dt)
    print(args.out)
    return 0


def cmd_memory(args) -> int:
    from .memory import memory_plan
    config = args.model
    if config.endswith(".json"):
        with open(config) as f:
            config = json.load(f)
    plan = memory_plan(config, args.dtype, args.max_tokens, args.max_slots)
    print(json.dumps({**plan.as_dict(), "max_tokens": plan.max_tokens, "max_slots": plan.max_slots,
                      "step_tokens": plan.step_tokens, "dtype": args.dtype}), flush=True)
    return 0


def cmd_bench(args) -> int:
    from . import benchmark
    if args.ablate and args.no_decode:
        rec = benchmark.ablate_prefill(tokens=args.prefill_tokens, dtype=args.dtype, layers=args.layers,
                                       config_index=args.config)
        print(json.dumps(rec, indent=1), flush=True)
        return 0
    if args.ablate:
        rec = benchmark.ablate_decode(batch=args.batch, prompt_tokens=args.prompt_tokens, dtype=args.dtype,
                                      layers=args.layers, config_index=args.config)
        print(json.dumps(rec, indent=1), flush=True)
        return 0
    rec = benchmark.run(batch=args.batch, prompt_tokens=args.prompt_tokens, decode_steps=args.decode_steps,
                        warmup=args.warmup, dtype=args.dtype, layers=args.layers, config_index=args.config,
                        points=args.points, e2e=args.e2e, prefill=not args.no_prefill, decode=not args.no_decode,
                        prefill_tokens=args.prefill_tokens, prompt_range=args.prompt_range, sampled=args.sampled)
    print(json.dumps(rec), flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="camelid", description="generation for the dense Llama decoder on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    _generate_args(sub.add_parser("generate", help="generate token ids for a prompt of token ids"))
    _generate_args(sub.add_parser("bench-generate", help="generate and print one JSON record per iteration"))
    from . import replay
    replay.add_arguments(sub.add_parser("replay", help="feed given tokens step by step and write logits"))
    rm = sub.add_parser("random-model", help="write a model folder with random weights")
    rm.add_argument("config", help="a config.json")
    rm.add_argument("out", help="folder to write")
    rm.add_argument("--seed", type=int, default=0)
    rm.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    me = sub.add_parser("memory", help="bytes of weights, cache and workspace, without touching a device")
    me.add_argument("model", help="model folder or config.json")
    me.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    me.add_argument("--max-tokens", type=int, default=4096)
    me.add_argument("--max-slots", type=int, default=None)
    be = sub.add_parser("bench", help="decode and prefill throughput with random weights")
    be.add_argument("--batch", type=int, default=8)
    be.add_argument("--prompt-tokens", type=int, default=2048)
    be.add_argument("--prompt-range", type=int, nargs=2, metavar=("LOWEST", "HIGHEST"), default=None,
                    help="prompts of unequal lengths, uniform between the two, instead of --prompt-tokens each; "
                         "their one prefill step is timed too")
    be.add_argument("--decode-steps", type=int, default=64)
    be.add_argument("--warmup", type=int, default=3)
    be.add_argument("--layers", type=int, default=None)
    be.add_argument("--config", type=int, default=2, help="index into the benchmark shapes (2: Llama 3.2 1B)")
    be.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    be.add_argument("--prefill-tokens", type=int, default=2048)
    be.add_argument("--points", action="store_true", help="also decode at batch 1 and 64")
    be.add_argument("--e2e", action="store_true", help="also time the loop through the Python entry point")
    be.add_argument("--sampled", action="store_true",
                    help="the timed decode steps sample (temperature, top-k, top-p, penalties) instead of taking the argmax")
    be.add_argument("--no-prefill", action="store_true")
    be.add_argument("--no-decode", action="store_true")
    be.add_argument("--ablate", action="store_true",
                    help="time the decode step (with --no-decode: the prefill step) with one kind of kernel "
                         "switched off at a time")
    args = ap.parse_args(argv)
    if args.command == "generate":
        return cmd_generate(args)
    if args.command == "bench-generate":
        return cmd_generate(args, always_json=True)
    if args.command == "replay":
        return replay.run(args)
    if args.command == "random-model":
        return cmd_random_model(args)
    if args.command == "memory":
        return cmd_memory(args)
    if args.command == "bench":
        return cmd_bench(args)
    return 2


if __name__ == "__main__":
    sys.exit(main())
