"""Token embedding (a row gather into the float32 residual stream, no scaling:
src/tensor/mod.rs:2253-2283) and the output projection, which is the embedding matrix
itself when the model ties them (src/model.rs:772-775, src/inference.rs:314-316)."""
from __future__ import annotations

import torch

from ..csrc import ops
from . import linear
from .base import Part, TensorSpec, register_part, to_device


@register_part("embedding", "embedding")
class TokenEmbedding(Part):
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight = None

    def tensor_specs(self):
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size), "embedding")}

    def load(self, tensors, device, dtype):
        self.weight = to_device(tensors[self.prefix + "weight"], device, dtype)

    def forward(self, ctx, tokens, out, err):
        ops.embed_gather(self.weight, tokens, out, err)


@register_part("head", "lm_head")
class OutputProjection(Part):
    """logits = x W^T in float32, without bias, soft-cap or scale (src/inference.rs:4284-4290)."""
    graph_safe = True
    graph_safe_any_step = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.weight = None

    def tensor_specs(self):
        if self.tied_to:
            return {}
        return {self.prefix + "weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, device, dtype, tied_weight: torch.Tensor | None = None):
        if self.tied_to:
            self.weight = tied_weight
        else:
            self.weight = to_device(tensors[self.prefix + "weight"], device, dtype)

    def forward(self, ctx, x, out):
        linear.linear(ctx, x, self.weight, out, linear.STORE_F32)
