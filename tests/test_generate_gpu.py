"""Generation through the Python entry point and the command line against the plain loop."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as pl
from conftest import CONFIGS
from helpers import tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_greedy_generation_float32(cuda, model_folders):
    """tiny_b, prompts of 17, 2, 40 and 9 tokens, 12 greedy steps: token for token."""
    import camelid_b200
    name = "tiny_b"
    lm = camelid_b200.load(model_folders[name], dtype="float32")
    prompts = [tokens(50 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([17, 2, 40, 9])]
    cfg, w = pl.read_model(model_folders[name])
    want = pl.generate(cfg, w, prompts, 12, dtype=torch.float64)
    got = lm.generate(prompts, max_tokens=12, stop_token_ids=())
    assert got == want
    assert len({tuple(g) for g in got}) > 1 and any(len(set(g)) > 2 for g in got)      # not a trivial repeat
    one = lm.generate(prompts[2], max_tokens=12, stop_token_ids=())                   # a single prompt, alone
    assert one == want[2]
    two = lm.generate(prompts, max_tokens=12, stop_token_ids=(), max_batch=2)         # two batches, slots reused
    assert two == want


def test_stop_tokens_and_details(cuda, model_folders):
    import camelid_b200
    name = "tiny_b"
    lm = camelid_b200.load(model_folders[name], dtype="float32")
    assert lm.stop_token_ids == (3, 11)
    prompts = [tokens(60 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([5, 11, 1])]
    free = lm.generate(prompts, max_tokens=8, stop_token_ids=())
    stop = free[1][3]
    res = lm.generate(prompts, max_tokens=8, stop_token_ids=(stop,), details=True)
    cfg, w = pl.read_model(model_folders[name])
    want = pl.generate(cfg, w, prompts, 8, stop_ids=(stop,), dtype=torch.float64)
    assert [r.tokens for r in res] == want
    assert res[1].finish_reason == "stop" and res[1].tokens[-1] == stop and len(res[1].tokens) <= 4
    assert all(r.finish_reason in ("stop", "length") for r in res)


def test_temperature_generation_matches_plain(cuda, model_folders):
    """tiny_a in float32 with temperature 0.8 and a fixed seed. A sampled token can differ
    from the plain loop only where the draw falls within rounding of a boundary of the
    cumulative distribution, so nearly all of the 4 x 12 tokens agree; the first ones must."""
    import camelid_b200
    name = "tiny_a"
    lm = camelid_b200.load(model_folders[name], dtype="float32")
    prompts = [tokens(70 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([17, 2, 40, 9])]
    cfg, w = pl.read_model(model_folders[name])
    want = pl.generate(cfg, w, prompts, 12, temperature=0.8, seed=1234, dtype=torch.float64)
    got = lm.generate(prompts, max_tokens=12, temperature=0.8, seed=1234, stop_token_ids=())
    assert [g[0] for g in got] == [x[0] for x in want]
    assert got == want
    again = lm.generate(prompts[::-1], max_tokens=12, temperature=0.8, seed=1234, stop_token_ids=())
    assert again == got[::-1]                           # a request's tokens do not depend on its batch


def test_bfloat16_generation_is_close(cuda, model_folders):
    import camelid_b200
    name = "tiny_b"
    lm = camelid_b200.load(model_folders[name], dtype="bfloat16")
    prompts = [tokens(50 + i, n, CONFIGS[name]["vocab_size"]) for i, n in enumerate([17, 2, 40, 9])]
    cfg, w = pl.read_model(model_folders[name])
    got = lm.generate(prompts, max_tokens=4, stop_token_ids=())
    # teacher-forced check: every generated token is the argmax of the plain logits, or within
    # the bfloat16 tolerance of it
    for p, g in zip(prompts, got):
        seq = list(p)
        for t in g:
            ref = pl.forward(cfg, w, seq, dtype=torch.float64)[-1]
            assert float(ref.max() - ref[t]) <= 2 * 3e-2 * float(ref.abs().max())
            seq.append(t)


def test_command_line(cuda, model_folders, tmp_path):
    prompt_file = tmp_path / "prompt.json"
    prompt_file.write_text(json.dumps([5, 17, 3, 200, 9]))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "camelid"), "generate", model_folders["tiny_b"],
                          "--prompt-file", str(prompt_file), "--max-tokens", "6", "--dtype", "float32", "--json"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    cfg, w = pl.read_model(model_folders["tiny_b"])
    want = pl.generate(cfg, w, [[5, 17, 3, 200, 9]], 6, stop_ids=(3, 11), dtype=torch.float64)[0]
    assert rec["output_token_ids"] == want and rec["prompt_tokens"] == 5 and rec["generated_tokens"] == len(want)
    for key in ("load_ms", "prefill_ms", "ttft_ms", "decode_ms", "tokens_per_second"):
        assert key in rec


def test_penalties_and_bias_on_the_device_match_plain(cuda, model_folders):
    """Penalties and bias ride along in the steps that feed themselves (token counts of each history kept on
    the device, the chosen tokens counted by the step); with the feeding switched off the same requests run the
    Python loop with the counts made on the host. Both must agree with the plain loop: greedy, sampled, with
    stop tokens (short runs, the counts set again at every run) and with requests that end at different times."""
    import camelid_b200
    from camelid_b200.options import KernelOptions
    name = "tiny_b"
    vocab = CONFIGS[name]["vocab_size"]
    prompts = [tokens(80 + i, n, vocab) for i, n in enumerate([6, 13, 40])]
    cfg, w = pl.read_model(model_folders[name])
    opts = dict(repeat_penalty=1.3, presence_penalty=0.2, frequency_penalty=0.1, logit_bias=[(5, 2.0), (7, -1.0), (5, 0.5)])
    want = pl.generate(cfg, w, prompts, 40, dtype=torch.float64, **opts)
    sampled = dict(opts, temperature=0.9, top_k=30, seed=11)
    want_sampled = pl.generate(cfg, w, prompts, 24, dtype=torch.float64, **sampled)
    for options in (None, KernelOptions(feed_on_device=False)):
        lm = camelid_b200.load(model_folders[name], dtype="float32", options=options)
        seen = []
        real = lm.model.decode_fed if options is None else None
        if real is not None:
            def spy(*a, **k):
                seen.append(k.get("histories") is not None)
                return real(*a, **k)
            lm.model.decode_fed = spy
        assert lm.generate(prompts, max_tokens=40, stop_token_ids=(), **opts) == want
        assert lm.generate(prompts, max_tokens=[24, 9, 17], stop_token_ids=(), **sampled) == [
            want_sampled[0][:24], want_sampled[1][:9], want_sampled[2][:17]]
        stop = want[0][20]                                  # a stop token in the middle of the first request
        cut = [t[:t.index(stop) + 1] if stop in t else t for t in want]
        assert lm.generate(prompts, max_tokens=40, stop_token_ids=(stop,), **opts) == cut
        if real is not None:
            assert seen and all(seen), "penalties must ride in the steps that feed themselves"
        plain_loop = lm.generate(prompts, max_tokens=10, stop_token_ids=())
        assert plain_loop == pl.generate(cfg, w, prompts, 10, dtype=torch.float64)


def test_long_generation_crosses_pages_in_the_native_loop(cuda, model_folders):
    """70 + 140 tokens: the C++ loop runs over two page boundaries, for two requests of unequal
    length that stop at different times."""
    import camelid_b200
    name = "tiny_c"
    lm = camelid_b200.load(model_folders[name], dtype="float32")
    prompts = [tokens(90, 70, CONFIGS[name]["vocab_size"]), tokens(91, 3, CONFIGS[name]["vocab_size"])]
    cfg, w = pl.read_model(model_folders[name])
    want = pl.generate(cfg, w, prompts, 140, dtype=torch.float64)
    got = lm.generate(prompts, max_tokens=[140, 90])
    assert got[0] == want[0] and got[1] == want[1][:90]
