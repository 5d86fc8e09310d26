"""SwiGLU feed-forward: g = x Wg^T, u = x Wu^T, act = (g / (1 + exp(-g))) * u,
d = act Wd^T, added into the residual stream (src/inference.rs:9657-9664, :6654-6706;
device twin silu_mul at src/cuda_resident.rs:1769). Gate and up are one packed matrix so
that one product makes both and the activation happens in its epilogue."""
from __future__ import annotations

from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("ffn", "swiglu")
class SwiGLU(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True
    accepts_row_scale = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.group = linear.swiglu_group(self.intermediate_size)
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p = self.prefix
        return {
            p + "gate_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "up_proj.weight": TensorSpec((self.intermediate_size, self.hidden_size)),
            p + "down_proj.weight": TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, tensors, device, dtype):
        p = self.prefix
        gate = to_device(tensors[p + "gate_proj.weight"], device, dtype)
        up = to_device(tensors[p + "up_proj.weight"], device, dtype)
        self.w_gate_up = linear.pack_gate_up(gate, up, self.group)
        self.w_down = to_device(tensors[p + "down_proj.weight"], device, dtype)

    def forward(self, ctx, x, residual):
        act = ctx.buffer("ffn_act", (ctx.n_rows, self.intermediate_size))
        linear.linear(ctx, x, self.w_gate_up, act, linear.SWIGLU, self.group, row_scale=ctx.take_row_scale())
        linear.add_into_residual(ctx, act, self.w_down, residual, "down_partial")
