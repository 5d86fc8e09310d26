"""y = x W^T for the parts: picks the kernel for the operands at hand.

bfloat16 operands whose sizes the tensor-core kernel takes go there; everything else
(float32, which must stay true 32-bit arithmetic, and the sizes that kernel refuses) goes
to the CUDA-core kernel. Both accumulate in float32 and share the epilogues: store in the
compute type, store float32, add into the float32 residual stream, or SwiGLU on packed
gate/up rows.

Steps of at most 128 rows (decode, short prompts) run the tensor-core kernel transposed, with
the weights as the 128-row operand and K split over several blocks so that every SM streams
weights. Steps of more rows run on tiles of 256 x 256 of two blocks; where a product has too
few of those for the SMs (a few hundred rows, a narrow output), K is split there too. The
split sums stay in float32 and are added, in split order, by the kernel that reads the
result next: the rotary kernel for q/k/v (``partial_sums``), the next norm for products that
go into the residual stream (``add_into_residual`` leaves them *pending* on the context).
"""
from __future__ import annotations

import os

import torch

from ..csrc import ops

STORE, STORE_F32, ADD_F32, SWIGLU = ops.EPI_STORE, ops.EPI_STORE_F32, ops.EPI_ADD_F32, ops.EPI_SWIGLU

SM_COUNT = 148
# Up to here a step runs the transposed kernel. Measured on the 1B shape (prefill step, ms): 96 rows
# 1.24 transposed against 1.38 on the tiles below, 128 rows 1.31 against 1.42; 144 rows 1.54 against
# 1.42, 256 rows 1.87 against 1.50: the float split sums that the transposed form writes and its
# readers sum again grow with the rows, the weights it streams do not.
DECODE_ROWS = int(os.environ.get("CAMELID_DECODE_ROWS", "128"))
CLUSTERS = SM_COUNT // 2      # pairs of blocks that run tiles of 256 x 256
_err: dict = {}


def _err_word(device) -> torch.Tensor:
    e = _err.get(device)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _err[device] = e
    return e


def check_errors() -> None:
    """Synchronising read of the tensor-core kernel's error word (a wait that ran out)."""
    from ..errors import KernelError
    for e in _err.values():
        if int(e.item()):
            e.zero_()
            raise KernelError("the tensor-core matrix product gave up waiting on a barrier")


def _bn_decode(rows: int) -> int:
    return next((bn for bn in (16, 32, 64) if rows <= bn), 128)


PAIR_SPLITS = os.environ.get("CAMELID_PAIR_SPLITS", "1") != "0"
FUSE_NORM = os.environ.get("CAMELID_FUSE_NORM", "1") != "0"   # the norm after a product of many rows runs inside it
PAIR_ROWS = max(128, DECODE_ROWS)     # above this many rows the product runs on 256 x 256 tiles of two blocks


def _bn_prefill(rows: int, out_features: int) -> int:
    """Tile width over the weight rows for a persistent launch: the one that needs fewer
    rounds of SM_COUNT blocks times its width (wider tiles reuse operands better on a tie)."""
    def cost(bn):
        tiles = ((rows + 127) // 128) * ((out_features + bn - 1) // bn)
        return ((tiles + SM_COUNT - 1) // SM_COUNT) * bn
    return 256 if cost(256) <= cost(128) else 128


def _splits(out_features: int, k: int) -> int:
    tiles = (out_features + 127) // 128
    return max(1, min((k + 63) // 64, round(SM_COUNT / tiles))) if tiles < SM_COUNT else 1


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, group: int = 0,
           row_scale=None) -> None:
    """out (op)= x @ w.T, complete on return. For SWIGLU ``w`` is the packed [2N, K] matrix
    and ``out`` is [M, N]. ``row_scale`` (``ops.RowScale``): what the rows of ``x`` still lack;
    the two-block kernel applies it to its output rows, any other path to ``x`` first."""
    tc = ops.gemm_tc_usable(x, w)
    rows = x.shape[0]
    pair = tc and rows > PAIR_ROWS          # tiles of 256 x 256 on two blocks: less operand traffic per flop
    swiglu_tc = group == 16 and w.shape[0] % 32 == 0
    if row_scale is not None and not (pair and (epilogue == STORE or (epilogue == SWIGLU and swiglu_tc))):
        ops.scale_rows(x, row_scale)
        row_scale = None
    if tc:
        err = _err_word(x.device)
        if rows <= DECODE_ROWS:
            bn = _bn_decode(rows)
            if epilogue == SWIGLU and swiglu_tc:
                ops.gemm_tc(w, x, out, ops.TC_T_SWIGLU, bn, 1, err)
                return
            if epilogue == STORE_F32:
                ops.gemm_tc(w, x, out.unsqueeze(0), ops.TC_T_PARTIAL, bn, 1, err)
                return
        # everything else on tiles of this step's rows by the weights' rows (for few rows only
        # what a part outside the library asks for: the library's own few-row products are above)
        bn = _bn_prefill(rows, w.shape[0])
        if epilogue == SWIGLU:
            if swiglu_tc:
                if pair:
                    ops.gemm_tc_pair(x, w, out, ops.TC_SWIGLU, err, row_scale)
                else:
                    ops.gemm_tc(x, w, out, ops.TC_SWIGLU, bn, 1, err)
                return
        else:
            epi = {STORE: ops.TC_STORE, STORE_F32: ops.TC_STORE_F32, ADD_F32: ops.TC_ADD_F32}[epilogue]
            if pair:
                ops.gemm_tc_pair(x, w, out, epi, err, row_scale)
            else:
                ops.gemm_tc(x, w, out, epi, bn, 1, err)
            return
    ops.gemm_tn_simt(x, w, out, epilogue, group)


def _pair_splits(rows: int, n: int, k: int) -> int:
    """Splits of K for a product on two-block tiles: more than 1 only for a deep product (K of
    4,096 or more) whose tiles leave half of the clusters or more without work; then as many as
    fill them, of at least 16 k-blocks of 64. (Measured at 512 rows of the 1B shape: the down
    product 53 -> 33 us with 4 splits, but a product of K = 2,048 gains less than the slower
    kernels that then read its split sums cost.)"""
    tiles = ((rows + 255) // 256) * ((n + 255) // 256)
    if 2 * tiles > CLUSTERS or k < 4096:
        return 1
    return ops.pair_partial_splits(k, max(1, min(CLUSTERS // tiles, (k + 63) // 64 // 16)))


def partial_sums(ctx, x: torch.Tensor, w: torch.Tensor, name: str, row_scale=None):
    """float32 [splits, rows, out] whose sum over splits is x @ w.T, where the tensor-core path
    splits K for this step's size; None (and nothing done) where it does not. ``row_scale``
    (``ops.RowScale``): what the rows of ``x`` still lack; applied if a result is returned."""
    rows = x.shape[0]
    if not ops.gemm_tc_usable(x, w):
        return None
    n, k = w.shape
    if rows <= DECODE_ROWS:
        if row_scale is not None:
            ops.scale_rows(x, row_scale)
        splits = min(_splits(n, k), (k + 63) // 64)
        part = ctx.buffer(name, (splits, rows, n), torch.float32)
        ops.gemm_tc(w, x, part, ops.TC_T_PARTIAL, _bn_decode(rows), splits, _err_word(x.device))
        return part
    splits = _pair_splits(rows, n, k) if PAIR_SPLITS else 1
    if splits == 1:
        return None
    part = ctx.buffer(name, (splits, rows, n), torch.float32)
    ops.gemm_tc_pair_partial(x, w, part, _err_word(x.device), row_scale)
    return part


def add_into_residual(ctx, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, name: str) -> None:
    """residual += x @ w.T. On the decode path the split sums are left pending on the context
    and the next norm adds them. A product of many rows on the tensor cores is *deferred*: the
    norm that reads the stream next launches it with the weight half of that norm in its
    epilogue (``product_add_norm``), or plainly where that does not fit. Otherwise the product's
    own epilogue adds now."""
    ctx.settle(residual)
    part = partial_sums(ctx, x, w, name)
    if part is not None:
        ctx.pending = part
    elif FUSE_NORM and x.shape[0] > PAIR_ROWS and ops.gemm_tc_usable(x, w) and residual.dtype == torch.float32:
        ctx.deferred = (x, w, residual)
    else:
        linear(ctx, x, w, residual, ADD_F32)


def run_deferred(ctx) -> None:
    """Launch a deferred product with its plain epilogue: the residual stream is complete after."""
    if ctx.deferred is not None:
        (x, w, residual), ctx.deferred = ctx.deferred, None
        linear(ctx, x, w, residual, ADD_F32)


def product_add_norm(ctx, residual: torch.Tensor, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> bool:
    """If a product into ``residual`` is deferred and the sizes allow: one launch that runs it,
    adds it into ``residual`` and writes ``out`` = bfloat16(residual * norm_w), and the rows'
    scale rsqrt(mean(residual^2) + eps) goes to ``ctx.row_scale`` for the reader of ``out`` to
    apply. False (and nothing done) otherwise."""
    if ctx.deferred is None:
        return False
    x, w, res = ctx.deferred
    rows, n = x.shape[0], w.shape[0]
    if (res is not residual or out.dtype != torch.bfloat16 or out.shape != (rows, n) or residual.shape != (rows, n)
            or norm_w.dtype not in (torch.float32, torch.bfloat16) or norm_w.numel() != n):
        return False
    ctx.deferred = None
    sumsq = ctx.buffer("norm_sumsq", ((n + 255) // 256, rows), torch.float32)
    ctx.row_scale = ops.gemm_tc_pair_add_norm(x, w, residual, _err_word(x.device), norm_w, eps, out, sumsq)
    return True


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int) -> torch.Tensor:
    """[2I, K] with rows interleaved in groups: ``group`` gate rows, then the ``group`` up
    rows of the same outputs, and so on."""
    inter, k = gate.shape
    assert up.shape == gate.shape and inter % group == 0
    g = gate.view(inter // group, 1, group, k)
    u = up.view(inter // group, 1, group, k)
    return torch.cat([g, u], dim=1).reshape(2 * inter, k).contiguous()


def swiglu_group(inter: int) -> int:
    """Rows per interleave group of the packed gate/up matrix: 16 when that divides the width
    (the granularity at which the tensor-core epilogue pairs gate and up), else all of it."""
    return 16 if inter % 16 == 0 else inter
