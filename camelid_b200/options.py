"""The switches of the kernel paths, as one typed value that a model is built with.

Nothing in the library reads the environment to pick a kernel: a caller (a test, the
benchmark's ablations) passes ``KernelOptions`` to ``load`` / ``from_random`` /
``DecoderModel``. The defaults are the product path. The reference, in contrast, steers its
engine with several hundred ``CAMELID_*`` variables read where they are used
(e.g. src/cuda_resident.rs:5558-5571, src/inference.rs:2298-2309).
"""
from __future__ import annotations

from dataclasses import dataclass

from .errors import ConfigError


@dataclass(frozen=True)
class KernelOptions:
    # Steps of up to this many rows run their products transposed (weights as the 128-row
    # operand, K split over blocks); wider steps run on two-block tiles of 256 x 256.
    decode_rows: int = 128
    # A deep product on two-block tiles whose tiles leave most clusters idle is split over K.
    pair_splits: bool = True
    # The norm after a product of many rows runs inside that product's epilogue.
    fuse_norm: bool = True
    # Decode attention: "fused" (one launch from the q/k/v product's split sums to the attention
    # output) or "split" (rotary kernel, then attention split over blocks and merged by tickets).
    decode_attention: str = "fused"
    # Kernels are launched with programmatic dependent launch.
    dependent_launch: bool = True
    # Greedy requests decode with the token fed back on the device.
    feed_on_device: bool = True
    # A step of several tokens per sequence whose layout (tokens per sequence, wanted places,
    # block-table widths) has come back replays a captured graph; this many rows of such
    # layouts are kept at most (each keeps a workspace of its own), and a kept one gives way
    # only to a layout that has come by more often.
    capture_repeated_steps: bool = True
    captured_step_rows: int = 16384

    def __post_init__(self):
        if not 1 <= int(self.decode_rows) <= 128:
            raise ConfigError("KernelOptions.decode_rows", f"must be 1..128, got {self.decode_rows}")
        if self.decode_attention not in ("fused", "split"):
            raise ConfigError("KernelOptions.decode_attention", f"expected 'fused' or 'split', got {self.decode_attention!r}")
