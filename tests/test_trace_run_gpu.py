"""bin/trace_run as a user drives it: the same requests whole, with the last 32 tokens one
by one, and in batches of unequal lengths with slots used again, in both precisions."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import CONFIGS
from helpers import assert_close, oracle, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out_dir, max_tokens):
    """Feeds the steps one at a time, each only after ``done <step>`` of the one before."""
    proc = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                             str(out_dir), "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE,
                            stdout=subprocess.PIPE, text=True)
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return lambda step, vocab: np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_b_odd", "tiny_d"])
def test_replay_three_ways(cuda, model_folders, tmp_path, name, dtype):
    vocab = CONFIGS[name]["vocab_size"]
    lens = [100, 37, 64, 5]
    seqs = {f"r{i}": tokens(900 + i, n, vocab) for i, n in enumerate(lens)}
    refs = {rid: oracle(model_folders[name], s).numpy() for rid, s in seqs.items()}
    steps, expect = [], {}
    n = 0
    # 1. each request alone and whole
    for rid, s in seqs.items():
        steps.append({"step": n, "entries": [{"id": rid + "w", "tokens": s, "want": list(range(len(s)))}], "end": [rid + "w"]})
        expect[n] = refs[rid]
        n += 1
    # 2. the prefix, then the last 32 tokens one by one
    for rid, s in seqs.items():
        head = max(1, len(s) - 32)
        steps.append({"step": n, "entries": [{"id": rid + "d", "tokens": s[:head], "want": [head - 1]}], "end": []})
        expect[n] = refs[rid][head - 1:head]
        n += 1
        for t in range(head, len(s)):
            steps.append({"step": n, "entries": [{"id": rid + "d", "tokens": [s[t]], "want": [0]}],
                          "end": [rid + "d"] if t == len(s) - 1 else []})
            expect[n] = refs[rid][t:t + 1]
            n += 1
    # 3. batches of unequal lengths; shorter requests end earlier; a second batch reuses the slots
    for rep in range(2):
        ids = list(seqs)
        prompt = {rid: max(1, len(seqs[rid]) // 2) for rid in ids}
        steps.append({"step": n, "entries": [{"id": f"{rid}b{rep}", "tokens": seqs[rid][:prompt[rid]],
                                              "want": [0, prompt[rid] - 1]} for rid in ids], "end": []})
        expect[n] = np.concatenate([refs[rid][[0, prompt[rid] - 1]] for rid in ids])
        n += 1
        pos = dict(prompt)
        live = list(ids)
        while live:
            entries = [{"id": f"{rid}b{rep}", "tokens": [seqs[rid][pos[rid]]], "want": [0]} for rid in live]
            exp = np.concatenate([refs[rid][pos[rid]:pos[rid] + 1] for rid in live])
            for rid in live:
                pos[rid] += 1
            ending = [rid for rid in live if pos[rid] >= len(seqs[rid]) or pos[rid] >= prompt[rid] + 20]
            steps.append({"step": n, "entries": entries, "end": [f"{rid}b{rep}" for rid in ending]})
            expect[n] = exp
            n += 1
            live = [rid for rid in live if rid not in ending]
    # the cache fits one batch of the four requests: every page is used again
    max_tokens = sum(((len(s) + 63) // 64) * 64 for s in seqs.values())
    read = replay(model_folders[name], dtype, steps, tmp_path, max_tokens)
    for step, ref in expect.items():
        assert_close(read(step, vocab), ref, dtype, f"{name} step {step}")


def test_replay_writes_nothing_for_empty_want(cuda, model_folders, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]}]
    read = replay(model_folders["tiny_a"], "float32", steps, tmp_path, 64)
    assert not os.path.exists(tmp_path / "0.f32")
    assert_close(read(1, 256), oracle(model_folders["tiny_a"], [1, 2, 3, 4]).numpy()[3:4], "float32")
