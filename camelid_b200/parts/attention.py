"""Grouped-query attention over the paged cache, as a mixer.

q, k, v = x Wq^T, x Wk^T, x Wv^T without bias (src/inference.rs:6301-6336), here one
product with the three matrices stacked; rotary encoding of q and k before the keys are
kept (src/inference.rs:23244-23281); attention of every new row over the keys of its own
sequence, causal, head h reading kv head h / (heads / kv_heads), scale 1/sqrt(head_dim)
(src/inference.rs:23945-24025, src/inference/diagnostic_config.rs:300-317); output
projection added into the residual stream (src/inference.rs:6487-6522).

An entry of the schedule that reads another entry's cache projects only q and writes
nothing. ``window`` (None for Llama) limits every query to the last ``window`` keys.
"""
from __future__ import annotations

import math

import torch

from ..cache.book import PAGE, KVSpec
from ..config.plan import PartSpec
from ..csrc import ops
from ..errors import ConfigError
from . import linear
from .base import Part, TensorSpec, build_part, register_part, to_device


@register_part("mixer", "attention")
class GroupedQueryAttention(Part):
    graph_safe = True
    graph_safe_any_step = True
    handles_pending = True
    accepts_row_scale = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ConfigError("num_kv_heads", f"{self.num_kv_heads} kv heads do not divide {self.num_heads} heads")
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ConfigError("head_dim", f"the attention kernels take head sizes 16..256 in steps of 16, got {self.head_dim}")
        if self.window is not None and int(self.window) <= 0:
            raise ConfigError("window", f"must be greater than zero, got {self.window}")
        pos = params.get("position") or PartSpec("none")
        self.position = build_part("position", pos)
        if self.position.rotary_dim > self.head_dim:
            raise ConfigError("rotary_dim", f"{self.position.rotary_dim} exceeds head_dim {self.head_dim}")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.w_qkv = None
        self.w_o = None

    def tensor_specs(self):
        p = self.prefix
        return {
            p + "q_proj.weight": TensorSpec((self.q_width, self.hidden_size)),
            p + "k_proj.weight": TensorSpec((self.kv_width, self.hidden_size)),
            p + "v_proj.weight": TensorSpec((self.kv_width, self.hidden_size)),
            p + "o_proj.weight": TensorSpec((self.hidden_size, self.q_width)),
        }

    def load(self, tensors, device, dtype):
        p = self.prefix
        parts = [to_device(tensors[p + n], device, dtype) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = to_device(tensors[p + "o_proj.weight"], device, dtype)
        self.position.load(tensors, device, dtype)

    def cache_spec(self):
        return KVSpec(self.num_kv_heads, self.head_dim, self.window)

    def query_tile_sizes(self):
        return [ops.attn_tiling(self.num_heads, self.num_kv_heads, False)[0],
                ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)[0]]

    # ------------------------------------------------------------------------------
    def forward(self, ctx, x, residual):
        n = ctx.n_rows
        borrow = ctx.cache_source is not None
        group, k_pages, v_pages = ctx.kv()
        table = ctx.block_table(group)
        width = self.q_width if borrow else self.q_width + 2 * self.kv_width
        w_in = self.w_qkv[:width] if borrow else self.w_qkv      # a borrowed cache needs no keys or values of its own
        pos = self.position
        row_scale = ctx.take_row_scale()          # the rows of x may still lack their norm's scale
        part = linear.partial_sums(ctx, x, w_in, "qkv_partial", row_scale)
        if part is not None:
            row_scale = None
        out = ctx.buffer("attn_out", (n, self.q_width))
        splits = self._decode_splits(ctx, n, 1, True) if ctx.decode else 1
        if (part is not None and ctx.decode and ctx.options.decode_attention == "fused" and (splits <= 8 or ctx.max_len <= 8192)
                and ops.attn_decode_fused_usable(part, out, self.head_dim, self.num_heads, self.num_kv_heads)):
            # decode: one launch sums the product's splits, rotates, writes the cache and attends
            ops.attn_decode_fused(part, out, ctx.row_pos, ctx.row_seq, table, k_pages, v_pages, pos.inv_freq,
                                  pos.rotary_dim, self.num_heads, self.num_kv_heads, self.head_dim, not borrow,
                                  self.window or 0, self.scale,
                                  ops.attn_decode_fused_splits(splits, self.num_heads, self.num_kv_heads, self.head_dim))
            linear.add_into_residual(ctx, out, self.w_o, residual, "o_partial")
            return
        if part is not None:          # decode: the rotary kernel sums the splits of the product
            q = ctx.buffer("q_rot", (n, self.q_width))
            ops.rope_kv_from_partials(part, q, ctx.row_pos, ctx.row_seq, table, k_pages, v_pages, pos.inv_freq,
                                      pos.rotary_dim, self.num_heads, self.num_kv_heads, self.head_dim,
                                      write_kv=not borrow)
        else:
            qkv = ctx.buffer("qkv", (n, width))
            linear.linear(ctx, x, w_in, qkv, linear.STORE, row_scale=row_scale)
            ops.rope_kv_write(qkv, ctx.row_pos, ctx.row_seq, table, k_pages, v_pages, pos.inv_freq, pos.rotary_dim,
                              self.num_heads, self.num_kv_heads, self.head_dim, write_kv=not borrow)
            q = qkv[:, :self.q_width]
        # prefill: bfloat16 with a head size of 64 or 128 on the tcgen05 kernel, everything else in
        # float on the CUDA cores; decode (where the fused kernel did not take it): mma.sync tiles
        # for those head sizes, split over blocks
        if not ctx.decode and ops.attn_tc_usable(q, out, self.head_dim):
            rows, hpc, chunks = ops.attn_tc_tiling(self.num_heads, self.num_kv_heads)
            tile_seq, tile_q0, n_tiles = ctx.query_tiles(rows)
            ops.attn_prefill_tc(q, out, k_pages, v_pages, table, tile_seq, tile_q0, n_tiles, ctx.seq_row0,
                                ctx.seq_start, ctx.seq_new, self.num_heads, self.num_kv_heads, self.head_dim, rows,
                                hpc, chunks, self.window or 0, self.scale, linear._err_word(q.device))
        elif ctx.decode and ops.attn_mma_usable(q, self.head_dim):
            self._attend(ctx, q, out, k_pages, v_pages, table, tensor_cores=True)
        else:
            self._attend(ctx, q, out, k_pages, v_pages, table, tensor_cores=False)
        linear.add_into_residual(ctx, out, self.w_o, residual, "o_partial")

    def _decode_splits(self, ctx, n_tiles: int, chunks: int, tensor_cores: bool) -> int:
        """Blocks that share the keys of one (row, kv head) in a decode step: enough for all SMs
        to stream the cache, but no block with less than a few tiles of keys."""
        keys = ctx.max_len if not self.window else min(ctx.max_len, self.window + PAGE)
        ctas = n_tiles * self.num_kv_heads * chunks
        unit = 8 * 32 if tensor_cores else PAGE               # keys a block should at least have
        if tensor_cores:
            per_sm = 2 if self.head_dim <= 64 else 1          # blocks that run at the same time on an SM
        else:                                                 # the float kernel keeps two pages of keys and values
            rows, hpc, _ = ops.attn_tiling(self.num_heads, self.num_kv_heads, True)
            smem = ops.attn_simt_smem_bytes(self.head_dim, rows, hpc, True) + 1024
            per_sm = max(1, min(8, (227 * 1024) // smem))
        resident = per_sm * ops.sm_count(ctx.device)
        return max(1, min((keys + unit - 1) // unit, resident // ctas, 64))

    def _attend(self, ctx, q, out, k_pages, v_pages, table, tensor_cores: bool):
        """Attention of the step's rows over the cache. bfloat16 with a head size of 64 or 128
        runs on the tensor cores, everything else in float on the CUDA cores. A decode step
        splits each sequence's keys over several blocks so that all SMs stream the cache."""
        tiling = ops.attn_mma_tiling if tensor_cores else ops.attn_tiling
        rows, hpc, chunks = tiling(self.num_heads, self.num_kv_heads, ctx.decode)
        tile_seq, tile_q0, n_tiles = ctx.query_tiles(rows)
        n_splits, partial = 1, None
        if ctx.decode:
            n_splits = self._decode_splits(ctx, n_tiles, chunks, tensor_cores)
            if n_splits > 1:
                partial = ctx.buffer("attn_partial", (ops.attn_partial_floats(ctx.n_rows, self.num_heads, self.head_dim,
                                                                             n_splits),), torch.float32)
        fn = ops.attn_paged_mma if tensor_cores else ops.attn_paged_simt
        fn(q, out, k_pages, v_pages, table, tile_seq, tile_q0, n_tiles, ctx.seq_row0, ctx.seq_start, ctx.seq_new,
           ctx.n_rows, self.num_heads, self.num_kv_heads, self.head_dim, rows, hpc, chunks, n_splits,
           self.window or 0, self.scale, partial)
