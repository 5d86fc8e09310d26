"""Arrangements of a layer's parts. ``prenorm`` is the reference's decoder layer
(src/inference.rs:6228-6804): r = x + mixer(norm1(x)); out = r + ffn(norm2(r)). The
residual stream stays float32; mixer and feed-forward add into it in place."""
from __future__ import annotations

from .base import Part, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    def __init__(self, layer_spec):
        super().__init__({}, "")
        self.norm1 = build_part("norm", layer_spec.norm1)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.norm2 = build_part("norm", layer_spec.norm2)
        self.ffn = build_part("ffn", layer_spec.ffn)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def tensor_specs(self):
        out = {}
        for p in self.parts():
            out.update(p.tensor_specs())
        return out

    def load(self, tensors, device, dtype):
        for p in self.parts():
            p.load(tensors, device, dtype)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def query_tile_sizes(self):
        return self.mixer.query_tile_sizes()

    def forward(self, ctx, h):
        # A built-in mixer or feed-forward may leave split sums pending on the context; the
        # norm that reads the stream next adds them. Parts from outside the library get a
        # settled stream.
        # A part that declares ``accepts_row_scale`` takes ``ctx.take_row_scale()`` and applies
        # it, which lets the norm before it run inside the product before that.
        x = self.norm1.forward(ctx, h, allow_row_scale=self.mixer.accepts_row_scale and self.mixer.graph_safe)
        if not self.mixer.graph_safe:
            ctx.settle(h)
        self.mixer.forward(ctx, x, h)
        x = self.norm2.forward(ctx, h, allow_row_scale=self.ffn.accepts_row_scale and self.ffn.graph_safe)
        if not self.ffn.graph_safe:
            ctx.settle(h)
        self.ffn.forward(ctx, x, h)
