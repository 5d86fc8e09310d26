"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w in float32 (src/tensor/mod.rs:2086-2096;
device twins rms_norm_f32 and rms_norm_batched at src/cuda_resident.rs:89, :1925). The
input is the float32 residual stream; the output has the compute type."""
from __future__ import annotations

import torch

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.hidden_size,), "norm")}

    def load(self, tensors, device, dtype):
        w = tensors[self.prefix + "weight"]
        # a weight stored in 32-bit stays so; a 16-bit one becomes float32 only on the float32 path
        keep = None if w.dtype == torch.float32 else dtype
        self.weight = to_device(w, device, keep)

    def forward(self, ctx, h, rows_index=None, n_rows=None, name="normed", allow_row_scale=False):
        """The normalised rows of ``h``. With ``allow_row_scale`` the caller promises that whoever
        reads the result takes ``ctx.take_row_scale()`` and applies it: then a product into ``h``
        that is still deferred runs here together with the residual add and the weight half of
        this norm, and only the rows' scale is left to the reader."""
        rows = h.shape[0] if n_rows is None else n_rows
        out = ctx.buffer(name, (rows, self.hidden_size))
        if ctx.deferred is not None:
            if allow_row_scale and rows_index is None and linear.product_add_norm(ctx, h, self.weight, self.eps, out):
                return out
            linear.run_deferred(ctx)
        pending, ctx.pending = ctx.pending, None            # split sums still to be added to h: added here
        ops.rmsnorm(h, self.weight, self.eps, out, rows_index, pending)
        return out
