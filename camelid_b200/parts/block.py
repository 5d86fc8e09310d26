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

    @property
    def graph_safe_any_step(self):
        return all(p.graph_safe_any_step for p in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def query_tile_sizes(self):
        return self.mixer.query_tile_sizes()

    def forward(self, ctx, h):
        # A built-in mixer or feed-forward may leave split sums pending on the context (or a
        # product deferred); the norm that reads the stream next adds them. Before any part that
        # does not declare ``handles_pending`` the block settles the stream itself, so a part
        # from outside the library, graph safe or not, reads and writes complete rows.
        # A part that declares ``accepts_row_scale`` takes ``ctx.take_row_scale()`` and applies
        # it, which lets the norm before it run inside the product before that.
        for norm, part in ((self.norm1, self.mixer), (self.norm2, self.ffn)):
            if not norm.handles_pending:
                ctx.settle(h)
            x = norm.forward(ctx, h, allow_row_scale=part.accepts_row_scale)
            if not part.handles_pending:
                ctx.settle(h)
            part.forward(ctx, x, h)
