"""python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line: decode tokens a second of the Llama 3.2 1B shape (random weights, batch 8,
2,048-token prompts, context 4,096) timed on the device over exactly K decode steps, the
same end to end through the Python entry point, the prefill of 2,048 tokens, the roofline
fraction of the decode step, decode at batch 1 and 64 (``points``, with time, bytes and
fraction in ``points_detail``), and the float32 model's decode step and prefill (``fp32``).
This library runs on one GPU: for --gpus above 1 it says so and exits with 2."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = ("karan68/Camelid is a Rust crate (Cargo.toml, no Python package): it cannot be installed with "
                         "pip and there is no Rust toolchain in this image")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-tokens", type=int, default=2048)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    ap.add_argument("--config", type=int, default=2, help="benchmark shape: 2 Llama 3.2 1B, 3 Llama 3.2 3B, 4 Llama 3.1 8B")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-fp32", action="store_true", help="leave out the float32 model's figures")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"camelid_b200 is a single-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    from camelid_b200 import benchmark
    rec = benchmark.run(batch=args.batch, prompt_tokens=args.prompt_tokens, decode_steps=args.steps,
                        warmup=max(args.warmup, 3), dtype=args.dtype, layers=args.layers, config_index=args.config,
                        points=not args.no_points, e2e=not args.no_e2e,
                        fp32=not args.no_fp32 and args.dtype == "bfloat16")
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
