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

import torch

from ..csrc import ops
from ..options import KernelOptions

STORE, STORE_F32, ADD_F32, SWIGLU = ops.EPI_STORE, ops.EPI_STORE_F32, ops.EPI_ADD_F32, ops.EPI_SWIGLU

# Which form a product takes is decided by the step's rows and ``ctx.options`` (KernelOptions):
# up to ``decode_rows`` rows the transposed kernel (the float split sums that form writes, and
# that its readers sum again, grow with the rows; the weights it streams do not), above that
# tiles of 256 x 256 on pairs of blocks. The number of SMs is the device's own.
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


_DEFAULTS = KernelOptions()


def _opt(ctx) -> KernelOptions:
    """The options of the step (the defaults where a part is driven without a context)."""
    return ctx.options if ctx is not None else _DEFAULTS


def _pair_rows(ctx) -> int:
    """Above this many rows a product runs on 256 x 256 tiles of two blocks."""
    return max(128, _opt(ctx).decode_rows)


def _bn_prefill(rows: int, out_features: int, sms: int) -> int:
    """Tile width over the weight rows for a persistent launch: the one that needs fewer
    rounds of one block per SM times its width (wider tiles reuse operands better on a tie)."""
    def cost(bn):
        tiles = ((rows + 127) // 128) * ((out_features + bn - 1) // bn)
        return ((tiles + sms - 1) // sms) * bn
    return 256 if cost(256) <= cost(128) else 128


def _splits(out_features: int, k: int, sms: int) -> int:
    tiles = (out_features + 127) // 128
    return max(1, min((k + 63) // 64, round(sms / tiles))) if tiles < sms else 1


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, group: int = 0,
           row_scale=None) -> None:
    """out (op)= x @ w.T, complete on return. For SWIGLU ``w`` is the packed [2N, K] matrix
    and ``out`` is [M, N]. ``row_scale`` (``ops.RowScale``): what the rows of ``x`` still lack;
    the two-block kernel applies it to its output rows, any other path to ``x`` first."""
    tc = ops.gemm_tc_usable(x, w)
    rows = x.shape[0]
    pair = tc and rows > _pair_rows(ctx)    # tiles of 256 x 256 on two blocks: less operand traffic per flop
    swiglu_tc = group == 16 and w.shape[0] % 32 == 0
    if row_scale is not None and not (pair and (epilogue == STORE or (epilogue == SWIGLU and swiglu_tc))):
        ops.scale_rows(x, row_scale)
        row_scale = None
    if tc:
        err = _err_word(x.device)
        if rows <= _opt(ctx).decode_rows:
            bn = _bn_decode(rows)
            if epilogue == SWIGLU and swiglu_tc:
                ops.gemm_tc(w, x, out, ops.TC_T_SWIGLU, bn, 1, err)
                return
            if epilogue == STORE_F32:
                ops.gemm_tc(w, x, out.unsqueeze(0), ops.TC_T_PARTIAL, bn, 1, err)
                return
        # everything else on tiles of this step's rows by the weights' rows (for few rows only
        # what a part outside the library asks for: the library's own few-row products are above)
        bn = _bn_prefill(rows, w.shape[0], ops.sm_count(x.device))
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
    ops.gemm_tn_simt(x, w, out, epilogue, group, _err_word(x.device))


def _pair_splits(rows: int, n: int, k: int, clusters: int) -> int:
    """Splits of K for a product on two-block tiles: more than 1 only for a deep product (K of
    4,096 or more) whose tiles leave half of the clusters or more without work; then as many as
    fill them, of at least 16 k-blocks of 64. A product of K = 2,048 gains less from a split
    than the slower kernels that then read its split sums cost."""
    tiles = ((rows + 255) // 256) * ((n + 255) // 256)
    if 2 * tiles > clusters or k < 4096:
        return 1
    return ops.pair_partial_splits(k, max(1, min(clusters // tiles, (k + 63) // 64 // 16)))


def partial_sums(ctx, x: torch.Tensor, w: torch.Tensor, name: str, row_scale=None):
    """float32 [splits, rows, out] whose sum over splits is x @ w.T, where the tensor-core path
    splits K for this step's size; None (and nothing done) where it does not. ``row_scale``
    (``ops.RowScale``): what the rows of ``x`` still lack; applied if a result is returned."""
    rows = x.shape[0]
    if not ops.gemm_tc_usable(x, w):
        # float: a step of at most 64 rows leaves the K ranges of its streaming blocks as they are
        splits = ops.gemv_f32_partial_splits(x, w) if rows <= 64 else 0
        if splits < 2:
            return None
        if row_scale is not None:
            ops.scale_rows(x, row_scale)
        part = ctx.buffer(name, (splits, rows, w.shape[0]), torch.float32)
        ops.gemv_f32_partial(x, w, part, _err_word(x.device))
        return part
    n, k = w.shape
    sms = ops.sm_count(x.device)
    if rows <= _opt(ctx).decode_rows:
        if row_scale is not None:
            ops.scale_rows(x, row_scale)
        splits = min(_splits(n, k, sms), (k + 63) // 64)
        part = ctx.buffer(name, (splits, rows, n), torch.float32)
        ops.gemm_tc(w, x, part, ops.TC_T_PARTIAL, _bn_decode(rows), splits, _err_word(x.device))
        return part
    splits = _pair_splits(rows, n, k, sms // 2) if _opt(ctx).pair_splits else 1
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
    elif (_opt(ctx).fuse_norm and x.shape[0] > _pair_rows(ctx) and ops.gemm_tc_usable(x, w)
          and residual.dtype == torch.float32):
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
