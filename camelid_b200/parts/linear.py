"""y = x W^T for the parts: picks the kernel for the operands at hand.

bfloat16 operands whose sizes the tensor-core kernel takes go there; everything else
(float32, which must stay true 32-bit arithmetic, and the sizes that kernel refuses) goes
to the CUDA-core kernel. Both accumulate in float32 and share the epilogues: store in the
compute type, store float32, add into the float32 residual stream, or SwiGLU on packed
gate/up rows.
"""
from __future__ import annotations

import torch

from ..csrc import ops

STORE, STORE_F32, ADD_F32, SWIGLU = ops.EPI_STORE, ops.EPI_STORE_F32, ops.EPI_ADD_F32, ops.EPI_SWIGLU

_tensor_core = None           # set by camelid_b200.parts.linear_tc when its kernel is available


def set_tensor_core_path(fn) -> None:
    global _tensor_core
    _tensor_core = fn


def linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, group: int = 0) -> None:
    """out (op)= x @ w.T. For SWIGLU ``w`` is the packed [2N, K] matrix and ``out`` [M, N]."""
    if _tensor_core is not None and x.dtype == torch.bfloat16 and _tensor_core(ctx, x, w, out, epilogue, group):
        return
    ops.gemm_tn_simt(x, w, out, epilogue, group)


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
