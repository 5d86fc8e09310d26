"""What the measurement program decides without a device: the shapes it names, the bytes and
operations it counts for the roofline, where the peaks come from, the prompts it draws, and
what `bench.py` answers for the reference arm and for more than one GPU."""
import json
import os
import subprocess
import sys

import numpy as np

from camelid_b200 import benchmark

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shapes_are_whole_configurations():
    from camelid_b200.config.registry import load_config
    for index, shape in benchmark.SHAPES.items():
        cfg = benchmark.config_for(index)
        _arch, typed, _plan = load_config(cfg)
        assert typed.num_hidden_layers == shape["num_hidden_layers"] and typed.head_dim == shape["head_dim"]
        assert benchmark.config_for(index, layers=2)["num_hidden_layers"] == 2
    one_b = benchmark.config_for(2)
    assert (one_b["hidden_size"], one_b["num_attention_heads"], one_b["num_key_value_heads"], one_b["vocab_size"]) == \
        (2048, 32, 8, 128256)


def test_counts_for_the_roofline():
    cfg = benchmark.config_for(2)
    # 16 layers of q/k/v (3072 x 2048), output (2048 x 2048) and three feed-forward matrices (8192 x 2048)
    assert benchmark.linear_params(cfg) == 16 * (2048 * 3072 + 2048 * 2048 + 3 * 2048 * 8192)
    weights = (benchmark.linear_params(cfg) + 2048 * 128256 + 33 * 2048) * 2
    one = benchmark.decode_bytes(cfg, 1, 0, 2)
    assert one == weights
    # every cached position of every live request: keys and values of 8 heads of 64 in 16 layers
    assert benchmark.decode_bytes(cfg, 8, 2048, 2) - one == 8 * 2048 * 16 * 2 * 8 * 64 * 2
    assert benchmark.decode_bytes(cfg, 1, 0, 4) == 2 * weights
    t = 2048
    flops = benchmark.prefill_flops(cfg, t)
    assert flops == 2.0 * t * benchmark.linear_params(cfg) + 2.0 * t * t * 32 * 64 * 16 + 2.0 * 2048 * 128256
    assert 4.2e12 < flops < 4.3e12


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path):
    assert benchmark.peaks(str(tmp_path)) == benchmark.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 7000.5, "bf16_tflops": 1500, "other": 1}))
    got = benchmark.peaks(str(tmp_path))
    assert got["source"] == "measured" and got["hbm_gbs"] == 7000.5 and got["bf16_tflops"] == 1500.0
    assert got["bf16_tflops_sustained"] == benchmark.FALLBACK_PEAKS["bf16_tflops_sustained"]     # a key it lacks keeps the fallback
    (tmp_path / "MEASURED_PEAKS.json").write_text("not json")
    assert benchmark.peaks(str(tmp_path)) == benchmark.FALLBACK_PEAKS


def test_prompts_of_one_length_or_of_a_range():
    rng = np.random.default_rng(0)
    same = benchmark._prompts(rng, 3, 17, 100)
    assert [len(p) for p in same] == [17, 17, 17] and all(0 <= t < 100 for p in same for t in p)
    ragged = benchmark._prompts(rng, 64, (5, 9), 100)
    lengths = {len(p) for p in ragged}
    assert lengths <= {5, 6, 7, 8, 9} and len(lengths) > 1 and {5, 9} <= lengths


def _bench(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, env=e)


def test_reference_arm_says_why_it_is_unavailable():
    r = _bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "Rust" in rec["unavailable"] and "\n" not in rec["unavailable"]


def test_more_than_one_gpu_is_refused_with_one_line():
    r = _bench("--gpus", "2")
    assert r.returncode == 2 and len(r.stdout.strip().splitlines()) == 1 and "single-GPU" in r.stdout
    r = _bench("--gpus", "2", env={"WORLD_SIZE": "2", "RANK": "1"})
    assert r.returncode == 2 and r.stdout.strip() == ""        # only rank 0 speaks
