"""Sampling options: the reference's ranges (src/inference.rs:5834-5888) and the draw stream."""
import pytest

import plain_llama as pl
from camelid_b200 import SamplingError
from camelid_b200.sampling import SamplingOptions, splitmix64, unit_draw


def test_options_are_validated():
    for bad in (dict(temperature=-1.0), dict(top_k=0), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=-0.1),
                dict(repeat_penalty=0.0), dict(presence_penalty=3.0), dict(frequency_penalty=-2.5),
                dict(logit_bias=[(1, 200.0)]), dict(logit_bias=[(999, 1.0)]), dict(temperature=float("nan"))):
        with pytest.raises(SamplingError):
            SamplingOptions(**bad).validate(500)
    o = SamplingOptions(temperature=0.5, top_k=3, top_p=1.0, min_p=0.0, seed=2 ** 64 - 1).validate(500)
    assert not o.greedy and not o.adjusts
    assert SamplingOptions().greedy and SamplingOptions(repeat_penalty=1.1).adjusts


def test_draw_stream_equals_the_plain_one():
    for seed in (0, 1, 42, 2 ** 64 - 1):
        for pos in (0, 1, 5, 1000, 2 ** 40):
            assert unit_draw(seed, pos) == float(pl.unit_draw(seed, pos))
    assert splitmix64(1) == pl.splitmix64(1)
