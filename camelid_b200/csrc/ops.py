"""Python faces of the CUDA launchers: argument checks, then one ctypes call on torch's
current stream. Tensors must live on a CUDA device; a CPU tensor or a missing extension is
an error, never a detour through library code."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from ..errors import KernelError
from . import build

PAGE = 64                      # tokens of a cache page; CML_PAGE in common.cuh
F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU = 0, 1, 2, 3

_ERRORS = {-2: "unsupported element type", -3: "a size is outside what the kernel takes",
           -4: "a pointer or stride is not aligned as the kernel needs"}

_SIGNATURES = {
    ("rowwise", "cml_embed_gather"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    ("rowwise", "cml_rmsnorm"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
                                 c_int, c_long, c_void_p],
    ("rowwise", "cml_add_partials"): [c_void_p, c_void_p, c_int, c_long, c_void_p],
    ("rowwise", "cml_swiglu_packed"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("rope_kv", "cml_rope_kv_write"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("rope_kv", "cml_rope_kv_from_partials"): [c_void_p, c_int, c_long, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_void_p],
    ("gemm_tc", "cml_gemm_tc"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_int, c_int,
                                 c_int, c_void_p, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_int,
                                      c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair_partial"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long,
                                              c_long, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    ("gemm_tc", "cml_gemm_tc_pair_add_norm"): [c_void_p, c_long, c_int, c_void_p, c_long, c_int, c_int, c_void_p, c_long,
                                               c_void_p, c_void_p, c_int, c_void_p, c_long, c_void_p, c_void_p],
    ("rowwise", "cml_scale_rows"): [c_void_p, c_int, c_long, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    ("attention_simt", "cml_attn_paged_simt"): [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                c_void_p, c_void_p],
    ("attention_simt", "cml_attn_simt_smem_bytes"): [c_int, c_int, c_int, c_int],
    ("attention_mma", "cml_attn_paged_mma"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                              c_void_p, c_void_p],
    ("attention_mma", "cml_attn_decode_fused"): [c_void_p, c_int, c_long, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_float, c_int, c_void_p, c_int, c_void_p],
    ("attention_tc", "cml_attn_prefill_tc"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_long, c_void_p,
                                              c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    ("gemm_simt", "cml_gemm_tn_simt"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("gemm_simt", "cml_gemv_f32_scratch_bytes"): [c_int, c_int, c_int, c_int],
    ("gemm_simt", "cml_gemv_f32_partial_splits"): [c_int, c_int, c_int, c_int, c_int],
    ("gemm_simt", "cml_gemv_f32_partial"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_long, c_int, c_int,
                                            c_int, c_int, c_void_p, c_void_p],
    ("sampling", "cml_argmax_rows"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_adjust_dense"): [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_count_tokens"): [c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("sampling", "cml_adjust_logits"): [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_float,
                                        c_void_p],
    ("sampling", "cml_decode_loop_size"): [],
    ("sampling", "cml_decode_loop_init"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "cml_decode_loop_run"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                         c_int, c_float, c_int, c_float, c_float, ctypes.c_ulonglong, c_void_p, c_void_p],
    ("sampling", "cml_decode_fed_run"): [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    ("sampling", "cml_draws_at"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    ("sampling", "cml_sample_rows"): [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p],
    ("random_fill", "cml_random_fill"): [c_void_p, c_int, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_ulonglong,
                                         ctypes.c_double, ctypes.c_double, c_void_p],
}
_fns: dict = {}
_libs: dict = {}
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (graph replays included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _fn(module: str, name: str):
    f = _fns.get(name)
    if f is None:
        lib = build.load(module)
        if module not in _libs:
            _libs[module] = lib
            _apply_dependent_launch(lib)
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[(module, name)]
        f.restype = c_int
        _fns[name] = f
    return f


def _check(code: int, what: str, launches: int = 1):
    global _launches
    _launches += launches
    if code != 0:
        if code in _ERRORS:
            raise KernelError(f"{what}: {_ERRORS[code]}")
        raise KernelError(f"{what}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("camelid_b200 kernels run on CUDA tensors only; there is no CPU path")


def _p(t):
    return None if t is None else t.data_ptr()


_sm_counts: dict = {}


def sm_count(device) -> int:
    """Multiprocessors of ``device`` (the number the launchers read from the runtime too)."""
    device = torch.device(device)
    n = _sm_counts.get(device)
    if n is None:
        n = int(torch.cuda.get_device_properties(device).multi_processor_count)
        _sm_counts[device] = n
    return n


_dependent_launch = True


def set_dependent_launch(on: bool) -> None:
    """Whether kernels are launched with programmatic dependent launch (the default). Applies
    to every kernel module, those loaded later included."""
    global _dependent_launch
    if bool(on) == _dependent_launch:
        return
    _dependent_launch = bool(on)
    for lib in _libs.values():
        _apply_dependent_launch(lib)


def _apply_dependent_launch(lib) -> None:
    try:
        setter = lib.cml_set_dependent_launch
    except AttributeError:          # a module without kernels that depend on their predecessors
        return
    setter.argtypes, setter.restype = [c_int], None
    setter(1 if _dependent_launch else 0)


try:        # the raw handle of the current stream without building a Stream object (a third of a launch's host time)
    _raw_stream, _device_now = torch._C._cuda_getCurrentRawStream, torch._C._cuda_getDevice
except AttributeError:      # a torch without these: the public way
    _raw_stream = None


def _stream():
    if _raw_stream is not None:
        return _raw_stream(_device_now())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"element type {dt} is not supported (float32 and bfloat16 are)") from None


# ---------------------------------------------------------------------------------------

def random_fill(out: torch.Tensor, key: int, first: int, mean: float, std: float):
    """out.view(-1)[i] = element ``first + i`` of the counter-based generator under ``key``
    (weights/counter_random.py is the host's definition of the same numbers)."""
    _dev(out)
    assert out.is_contiguous()
    _check(_fn("random_fill", "cml_random_fill")(_p(out), dtype_code(out.dtype), out.numel(), int(key), int(first),
                                                 float(mean), float(std), _stream()), "random_fill")


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err: torch.Tensor):
    """out[r] = table[tokens[r]] as float32. ``err`` (int32[1]) gets bit 1 on a bad id."""
    _dev(table, tokens, out, err)
    rows, hidden = out.shape
    assert table.shape[1] == hidden and tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous() and tokens.numel() >= rows
    _check(_fn("rowwise", "cml_embed_gather")(_p(table), dtype_code(table.dtype), _p(tokens), _p(out), rows, hidden,
                                             table.shape[0], _p(err), _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, rows_index: torch.Tensor | None = None,
            partial: torch.Tensor | None = None):
    """out[r] = rmsnorm(x[rows_index[r] or r]) * weight; x float32, out float32 or bfloat16.
    ``partial`` (float32 [splits, x rows, hidden]) is first added to x, split by split; without
    ``rows_index`` the sum is written back to x."""
    _dev(x, weight, out, rows_index, partial)
    rows, hidden = out.shape
    assert x.dtype == torch.float32 and x.shape[1] == hidden and weight.shape[0] == hidden
    assert x.is_contiguous() and out.is_contiguous()
    if rows_index is not None:
        assert rows_index.dtype == torch.int32 and rows_index.numel() >= rows
    n_splits, stride = 0, 0
    if partial is not None:
        assert partial.dtype == torch.float32 and partial.is_contiguous() and partial.shape[1:] == x.shape
        n_splits, stride = partial.shape[0], partial.stride(0)
    _check(_fn("rowwise", "cml_rmsnorm")(_p(x), _p(weight), dtype_code(weight.dtype), _p(out), dtype_code(out.dtype),
                                        _p(rows_index), rows, hidden, float(eps), _p(partial), n_splits, stride,
                                        _stream()), "rmsnorm")


def add_partials(x: torch.Tensor, partial: torch.Tensor):
    """x += sum over splits of partial[split] (float32), splits in index order."""
    _dev(x, partial)
    assert x.dtype == torch.float32 and partial.dtype == torch.float32 and partial.shape[1:] == x.shape
    assert x.is_contiguous() and partial.is_contiguous()
    _check(_fn("rowwise", "cml_add_partials")(_p(x), _p(partial), partial.shape[0], x.numel(), _stream()), "add_partials")


def swiglu_packed(gu: torch.Tensor, act: torch.Tensor, group: int):
    _dev(gu, act)
    rows, inter = act.shape
    assert gu.shape == (rows, 2 * inter) and gu.dtype == act.dtype and gu.is_contiguous() and act.is_contiguous()
    _check(_fn("rowwise", "cml_swiglu_packed")(_p(gu), _p(act), dtype_code(act.dtype), rows, inter, group, _stream()),
           "swiglu_packed")


def rope_kv_write(qkv: torch.Tensor, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq, rotary_dim: int,
                  n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool):
    """Rotate q (and k) of packed rows in place; write k and v into their cache pages."""
    _dev(qkv, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    rows = qkv.shape[0]
    assert qkv.stride(1) == 1 and inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rotary_dim
    need = (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    assert qkv.shape[1] >= need, (qkv.shape, need)
    if write_kv:
        assert k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype
        assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
        max_blocks = block_table.shape[1]
    else:
        max_blocks = 0
    _check(_fn("rope_kv", "cml_rope_kv_write")(
        _p(qkv), dtype_code(qkv.dtype), rows, qkv.stride(0), _p(row_pos), _p(row_seq), _p(block_table), max_blocks,
        _p(k_pages), _p(v_pages), _p(inv_freq), rotary_dim, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0,
        _stream()), "rope_kv_write")


def rope_kv_from_partials(partial: torch.Tensor, q_out: torch.Tensor, row_pos, row_seq, block_table, k_pages, v_pages,
                          inv_freq, rotary_dim: int, n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool):
    """The same as rope_kv_write on the split sums ``partial`` (float32 [splits, rows, width]) of
    the q/k/v product; the rotated q goes to ``q_out`` in the compute type."""
    _dev(partial, q_out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    n_splits, rows, width = partial.shape
    assert partial.dtype == torch.float32 and partial.is_contiguous() and q_out.stride(1) == 1
    assert q_out.shape == (rows, n_heads * head_dim) and inv_freq.numel() * 2 == rotary_dim
    if write_kv:
        assert k_pages.dtype == q_out.dtype and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim)
        assert k_pages.is_contiguous() and v_pages.is_contiguous()
    _check(_fn("rope_kv", "cml_rope_kv_from_partials")(
        _p(partial), n_splits, partial.stride(0), width, _p(q_out), q_out.stride(0), dtype_code(q_out.dtype), rows,
        _p(row_pos), _p(row_seq), _p(block_table), block_table.shape[1] if write_kv else 0, _p(k_pages), _p(v_pages),
        _p(inv_freq), rotary_dim, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0, _stream()),
        "rope_kv_from_partials")


TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU, TC_T_PARTIAL, TC_T_SWIGLU = 0, 1, 2, 3, 4, 5


def _tc_operand(t: torch.Tensor) -> bool:
    """Whether TMA can fetch tiles of ``t`` ([rows, K] bfloat16, K-major): 16-byte aligned base and
    row stride, so K and the stride are multiples of 8. Remembered on the tensor: weights and
    the workspace's views are the same objects step after step."""
    try:
        return t._cml_tc_operand
    except AttributeError:
        ok = (t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0 and t.stride(1) == 1
              and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)
        t._cml_tc_operand = ok
        return ok


def gemm_tc_usable(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands ([rows, K] bfloat16, K-major): TMA
    needs 16-byte aligned bases and row strides, so K and the strides must be multiples of 8."""
    return _tc_operand(a) and _tc_operand(b) and a.shape[1] == b.shape[1]


def gemm_tc(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epilogue: int, bn: int, splits: int, err: torch.Tensor):
    """D = a @ b.T on the tensor cores (see gemm_tc.cu). Epilogues 0..3 write c[row of a][row of b];
    4 and 5 are transposed: c[split][row of b][row of a] partial sums, or SwiGLU of packed a rows."""
    _dev(a, b, c, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc: operands must be bfloat16 [rows, K] with K and the row strides multiples of 8 "
                          "and 16-byte aligned bases")
    assert c.stride(-1) == 1
    ldc = c.stride(-2)
    _check(_fn("gemm_tc", "cml_gemm_tc")(_p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1],
                                        _p(c), ldc, epilogue, bn, splits, _p(err), _stream()), "gemm_tc")


class RowScale:
    """What a norm left undone when the product before it wrote the norm's output: the rows of
    that output lack the factor rsqrt(sum over parts of sumsq[part][row] / hidden + eps).
    The product that reads those rows applies it to its own output rows (a product is linear
    in its input rows), or ``scale_rows`` applies it in place."""

    def __init__(self, sumsq: torch.Tensor, hidden: int, eps: float):
        assert sumsq.dim() == 2 and sumsq.dtype == torch.float32 and sumsq.is_contiguous()
        self.sumsq, self.hidden, self.eps = sumsq, int(hidden), float(eps)


def gemm_tc_pair(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, epilogue: int, err: torch.Tensor,
                 row_scale: "RowScale | None" = None):
    """c[row of a][row of b] (op)= a @ b.T with epilogues 0..3 of ``gemm_tc``, on tiles of
    256 x 256 that the two blocks of a cluster share (tcgen05 cta_group::2): the kernel for
    products with many rows of ``a``. ``row_scale``: the scale the rows of ``a`` still lack."""
    _dev(a, b, c, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair: operands must be bfloat16 [rows, K] with K and the row strides multiples "
                          "of 8 and 16-byte aligned bases")
    assert c.stride(-1) == 1 and epilogue in (TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU)
    sumsq, parts, hidden, eps = None, 0, 0, 0.0
    if row_scale is not None:
        sumsq, hidden, eps = row_scale.sumsq, row_scale.hidden, row_scale.eps
        _dev(sumsq)
        parts = sumsq.shape[0]
        assert sumsq.shape[1] == a.shape[0]
    _check(_fn("gemm_tc", "cml_gemm_tc_pair")(_p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1],
                                             _p(c), c.stride(-2), epilogue, _p(err), _p(sumsq), parts, hidden, eps,
                                             _stream()), "gemm_tc_pair")


def pair_partial_splits(k: int, wanted: int) -> int:
    """How many splits of K ``gemm_tc_pair_partial`` makes when asked for ``wanted``: k-blocks of
    64 are dealt out evenly and no split stays empty."""
    blocks = (k + 63) // 64
    per = (blocks + max(1, min(wanted, blocks)) - 1) // max(1, min(wanted, blocks))
    return (blocks + per - 1) // per


def gemm_tc_pair_partial(a: torch.Tensor, b: torch.Tensor, part: torch.Tensor, err: torch.Tensor,
                         row_scale: "RowScale | None" = None):
    """part[s] (float32 [splits, rows of a, rows of b]) = the share of a @ b.T of the s-th split of
    K, on the two-block tiles of ``gemm_tc_pair``; the splits are work items of their own, which
    gives a product of a few hundred rows enough of them for every SM. ``part.shape[0]`` must be
    a count that ``pair_partial_splits`` returns."""
    _dev(a, b, part, err)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair_partial: operands must be bfloat16 [rows, K] with K and the row strides "
                          "multiples of 8 and 16-byte aligned bases")
    assert part.dtype == torch.float32 and part.dim() == 3 and part.stride(2) == 1
    assert part.shape[1:] == (a.shape[0], b.shape[0])
    sumsq, parts, hidden, eps = None, 0, 0, 0.0
    if row_scale is not None:
        sumsq, hidden, eps = row_scale.sumsq, row_scale.hidden, row_scale.eps
        _dev(sumsq)
        parts = sumsq.shape[0]
        assert sumsq.shape[1] == a.shape[0]
    _check(_fn("gemm_tc", "cml_gemm_tc_pair_partial")(
        _p(a), a.stride(0), a.shape[0], _p(b), b.stride(0), b.shape[0], a.shape[1], _p(part), part.stride(1),
        part.stride(0), part.shape[0], _p(err), _p(sumsq), parts, hidden, eps, _stream()), "gemm_tc_pair_partial")


def gemm_tc_pair_add_norm(a: torch.Tensor, b: torch.Tensor, h: torch.Tensor, err: torch.Tensor, norm_w: torch.Tensor,
                          eps: float, x_out: torch.Tensor, sumsq: torch.Tensor) -> RowScale:
    """h (float32 [rows, out]) += a @ b.T, and the first half of the RMS norm that reads h next:
    x_out = bfloat16(h * norm_w) and the sums of squares of every row, one per tile of 256
    columns, in ``sumsq`` (float32 [ceil(out / 256), rows]). Returns the scale the rows of
    x_out still lack."""
    _dev(a, b, h, err, norm_w, x_out, sumsq)
    if not gemm_tc_usable(a, b):
        raise KernelError("gemm_tc_pair_add_norm: operands must be bfloat16 [rows, K] with K and the row strides "
                          "multiples of 8 and 16-byte aligned bases")
    rows, n = a.shape[0], b.shape[0]
    assert h.dtype == torch.float32 and h.shape == (rows, n) and h.stride(1) == 1
    assert x_out.dtype == torch.bfloat16 and x_out.shape == (rows, n) and x_out.stride(1) == 1
    assert norm_w.numel() == n and norm_w.is_contiguous()
    assert sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.shape == ((n + 255) // 256, rows)
    _check(_fn("gemm_tc", "cml_gemm_tc_pair_add_norm")(
        _p(a), a.stride(0), rows, _p(b), b.stride(0), n, a.shape[1], _p(h), h.stride(0), _p(err), _p(norm_w),
        dtype_code(norm_w.dtype), _p(x_out), x_out.stride(0), _p(sumsq), _stream()), "gemm_tc_pair_add_norm")
    return RowScale(sumsq, n, eps)


def scale_rows(x: torch.Tensor, row_scale: RowScale):
    """x[r] *= the scale its rows still lack, in place."""
    _dev(x, row_scale.sumsq)
    assert x.dim() == 2 and x.stride(1) == 1 and row_scale.sumsq.shape[1] == x.shape[0]
    _check(_fn("rowwise", "cml_scale_rows")(_p(x), dtype_code(x.dtype), x.stride(0), x.shape[0], x.shape[1],
                                           _p(row_scale.sumsq), row_scale.sumsq.shape[0], row_scale.hidden,
                                           row_scale.eps, _stream()), "scale_rows")


def attn_heads_per_warp(heads_per_cta: int, decode: bool) -> int:
    """Heads of one token that a warp of the float attention kernel owns: in prefill as many of
    4, 2, 1 as divide the block's heads (a key read from shared memory serves them all). 0 names
    the decode kernel, whose four warps share every page by keys and all work on the block's 2 or
    4 heads; a decode step on single heads gives each its own warp."""
    if decode:
        return 0 if heads_per_cta in (2, 4) else 1
    return 4 if heads_per_cta % 4 == 0 else 2 if heads_per_cta % 2 == 0 else 1


def attn_tiling(n_heads: int, n_kv_heads: int, decode: bool) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the float attention kernel. Prefill: at most
    16 warps, each with one token and ``attn_heads_per_warp`` of its heads; the heads of a kv group
    are cut in chunks if above 16. Decode: one token and 2 or 4 heads of a kv group per block."""
    group = n_heads // n_kv_heads
    if decode:
        hpc = 1 if group == 1 else 2 if group == 2 else 4
        return 1, hpc, (group + hpc - 1) // hpc
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    rows = max(1, 16 * attn_heads_per_warp(hpc, False) // hpc)
    return rows, hpc, chunks


def attn_simt_smem_bytes(head_dim: int, rows_per_tile: int, heads_per_cta: int, decode: bool) -> int:
    """Shared memory of a block of the float attention kernel with this tiling."""
    f = _fn("attention_simt", "cml_attn_simt_smem_bytes")
    f.restype = c_long
    return int(f(head_dim, rows_per_tile, heads_per_cta, attn_heads_per_warp(heads_per_cta, decode)))


def attn_partial_floats(n_rows: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return n_rows * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def attn_paged_simt(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                    n_rows, n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits,
                    window, scale, partial, heads_per_warp=None):
    """Attention of packed query rows over the paged cache (float arithmetic). ``q`` may be a
    column slice of a wider matrix (its row stride is used). ``heads_per_warp``: by default what
    ``attn_tiling`` assumed (one where a tile is a single row)."""
    if heads_per_warp is None:
        heads_per_warp = attn_heads_per_warp(heads_per_cta, rows_per_tile == 1)
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, partial)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == v_pages.dtype
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    if n_splits > 1:
        assert partial is not None and partial.dtype == torch.float32
        assert partial.numel() >= attn_partial_floats(n_rows, n_heads, head_dim, n_splits)
    _check(_fn("attention_simt", "cml_attn_paged_simt")(
        _p(q), q.stride(0), _p(out), out.stride(0), dtype_code(q.dtype), _p(k_pages), _p(v_pages), _p(block_table),
        block_table.shape[1], _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_rows,
        n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, heads_per_warp, head_chunks, n_splits,
        int(window or 0), float(scale), _p(partial), _stream()), "attn_paged_simt", 2 if n_splits > 1 else 1)


def attn_mma_tiling(n_heads: int, n_kv_heads: int, decode: bool) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the mma.sync attention kernel: the 16
    rows of an MMA hold the grouped heads of one kv head times a few consecutive tokens."""
    group = n_heads // n_kv_heads
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    rows = 1 if decode else max(1, 16 // hpc)
    return rows, hpc, chunks


def attn_mma_usable(q: torch.Tensor, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and head_dim in (64, 128) and q.stride(0) % 2 == 0


def attn_paged_mma(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                   n_rows, n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits,
                   window, scale, partial):
    """bfloat16 attention of packed query rows over the paged cache on the tensor cores."""
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, partial)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == torch.bfloat16
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    tickets = None
    if n_splits > 1:
        assert partial is not None and partial.dtype == torch.float32
        assert partial.numel() >= attn_partial_floats(n_rows, n_heads, head_dim, n_splits)
        tickets = zeroed_scratch(q.device, "attention_tickets", 4 * n_tiles * n_kv_heads * head_chunks)
    _check(_fn("attention_mma", "cml_attn_paged_mma")(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), _p(block_table), block_table.shape[1],
        _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_rows, n_heads, n_kv_heads,
        head_dim, rows_per_tile, heads_per_cta, head_chunks, n_splits, int(window or 0), float(scale), _p(partial),
        _p(tickets), _stream()), "attn_paged_mma")


def attn_decode_fused_usable(partial, out, head_dim: int, n_heads: int, n_kv_heads: int) -> bool:
    return (partial is not None and partial.dtype == torch.float32 and out.dtype == torch.bfloat16
            and head_dim in (64, 128) and n_heads // n_kv_heads <= 16 and out.stride(0) % 2 == 0)


def attn_decode_fused_splits(n_splits: int, n_heads: int, n_kv_heads: int, head_dim: int) -> int:
    """The number of blocks per cluster the fused decode kernel can take, at most ``n_splits``:
    block 0 keeps the ranges of all blocks in shared memory beside its own cache tiles."""
    group = n_heads // n_kv_heads
    stages = 4 * 3 * 2 * 32 * head_dim * 2
    n_splits = max(1, min(8, n_splits))
    while n_splits > 1 and stages + n_splits * group * (head_dim + 2) * 4 + 8 * 1024 > 227 * 1024:
        n_splits -= 1
    return n_splits


def attn_decode_fused(partial, out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq, rotary_dim: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool, window: int, scale: float,
                      n_splits: int):
    """Decode attention in one launch from the partial sums [splits, rows, width] of the q/k/v
    product: sums them, rotates q and the new key, writes the new key and value to the cache
    (``write_kv``) and attends every row (one new token of a sequence each) over its cache,
    the keys split over the ``n_splits`` (at most 8) blocks of a cluster."""
    _dev(partial, out, row_pos, row_seq, block_table, k_pages, v_pages, inv_freq)
    assert partial.dim() == 3 and partial.is_contiguous() and out.stride(1) == 1
    assert k_pages.dtype == torch.bfloat16 and k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and 1 <= n_splits <= 8
    rows = partial.shape[1]
    _check(_fn("attention_mma", "cml_attn_decode_fused")(
        _p(partial), partial.shape[0], partial.stride(0), partial.shape[2], rows, _p(row_pos), _p(row_seq),
        _p(block_table), block_table.shape[1], _p(k_pages), _p(v_pages), _p(inv_freq), rotary_dim, n_heads, n_kv_heads,
        head_dim, 1 if write_kv else 0, int(window or 0), float(scale), n_splits, _p(out), out.stride(0), _stream()),
        "attn_decode_fused")


def attn_tc_tiling(n_heads: int, n_kv_heads: int) -> tuple[int, int, int]:
    """(rows_per_tile, heads_per_cta, head_chunks) of the tcgen05 prefill attention kernel: the
    128 lanes of tensor memory hold the grouped heads of one kv head times consecutive tokens."""
    group = n_heads // n_kv_heads
    chunks = (group + 15) // 16
    hpc = (group + chunks - 1) // chunks
    return max(1, 128 // hpc), hpc, chunks


def attn_tc_usable(q: torch.Tensor, out: torch.Tensor, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128) and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attn_prefill_tc(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, n_tiles, seq_row0, seq_start, seq_new,
                    n_heads, n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, window, scale, err):
    """bfloat16 prefill attention of packed query rows over the paged cache with tcgen05.mma."""
    _dev(q, out, k_pages, v_pages, block_table, tile_seq, tile_q0, seq_row0, seq_start, seq_new, err)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype == torch.bfloat16
    assert k_pages.shape[1:] == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous() and v_pages.is_contiguous()
    _check(_fn("attention_tc", "cml_attn_prefill_tc")(
        _p(q), q.stride(0), _p(out), out.stride(0), _p(k_pages), _p(v_pages), k_pages.shape[0], _p(block_table),
        block_table.shape[1], _p(tile_seq), _p(tile_q0), n_tiles, _p(seq_row0), _p(seq_start), _p(seq_new), n_heads,
        n_kv_heads, head_dim, rows_per_tile, heads_per_cta, head_chunks, int(window or 0), float(scale), _p(err),
        _stream()), "attn_prefill_tc")


def gemm_tn_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, group: int = 0, err=None):
    """c[M, N] (op)= a[M, K] @ w[N, K]^T with float accumulation on the CUDA cores.
    EPI_SWIGLU reads w as packed [2N, K] gate/up rows interleaved in groups of ``group``.
    ``err`` (int32[1]): set to 8 by the form that streams float weights through shared memory if one
    of its bounded waits runs out; by default this module's own word (``simt_error_word``)."""
    _dev(a, w, c)
    M, K = a.shape
    N = c.shape[1]
    assert c.shape[0] == M and w.shape[1] == K and a.dtype == w.dtype
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] == 2 * N and c.dtype == a.dtype
    else:
        assert w.shape[0] == N
        assert c.dtype == (a.dtype if epilogue == EPI_STORE else torch.float32)
    scratch = None
    if err is None:
        err = simt_error_word(a.device)
    if a.dtype == torch.float32 and M <= 64:      # the streaming form for few float rows: tickets and split sums
        f = _fn("gemm_simt", "cml_gemv_f32_scratch_bytes")
        f.restype = c_long
        scratch = zeroed_scratch(a.device, "gemv_f32", int(f(M, N, K, epilogue)))
    _check(_fn("gemm_simt", "cml_gemm_tn_simt")(_p(a), a.stride(0), _p(w), w.stride(0), _p(c), c.stride(0), M, N, K,
                                                dtype_code(a.dtype), epilogue, group, _p(scratch), _p(err), _stream()),
           "gemm_tn_simt")


def gemv_f32_partial_splits(a: torch.Tensor, w: torch.Tensor) -> int:
    """Ranges of K that ``gemv_f32_partial`` cuts a[M, K] @ w[N, K]^T into; 0 where it does not take
    the product (more than 64 rows, not float, sizes that do not allow 16-byte copies)."""
    if a.dtype != torch.float32 or w.dtype != torch.float32 or a.stride(1) != 1 or w.stride(1) != 1:
        return 0
    if (a.data_ptr() | w.data_ptr()) & 15:
        return 0
    return int(_fn("gemm_simt", "cml_gemv_f32_partial_splits")(a.shape[0], w.shape[0], a.shape[1], a.stride(0),
                                                               w.stride(0)))


def gemv_f32_partial(a: torch.Tensor, w: torch.Tensor, part: torch.Tensor, err: torch.Tensor):
    """part[r] = a @ w^T over range r of K (float, at most 64 rows): the product's sums left as
    partial sums for the kernel that reads them next, with no pass over them in between."""
    _dev(a, w, part, err)
    splits, M, N = part.shape
    assert part.dtype == torch.float32 and part.stride(2) == 1 and a.shape[0] == M and w.shape[0] == N
    _check(_fn("gemm_simt", "cml_gemv_f32_partial")(_p(a), a.stride(0), _p(w), w.stride(0), _p(part), part.stride(1),
                                                    part.stride(0), splits, M, N, a.shape[1], _p(err), _stream()),
           "gemv_f32_partial")


_scratch: dict = {}
_retired: list = []
_simt_err: dict = {}


def simt_error_word(device) -> torch.Tensor:
    """The error word ``gemm_tn_simt`` hands its kernels when the caller gives none."""
    key = torch.device(device)
    e = _simt_err.get(key)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _simt_err[key] = e
    return e


def zeroed_scratch(device, name: str, n_bytes: int) -> torch.Tensor:
    """Device memory that kernels of this library leave zeroed between calls (tickets of
    the blocks of a kernel and the like); it only ever grows. Not to be made while a CUDA
    graph is being captured: the first call of a kernel that needs it should come before."""
    key = (torch.device(device), name)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n_bytes:
        if buf is not None:
            _retired.append(buf)               # captured graphs may still point at it
        buf = torch.zeros(max(n_bytes, 4096), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def argmax_rows(logits: torch.Tensor, out: torch.Tensor, err: torch.Tensor):
    """out[r] = index of the largest logit of row r, the lowest index among equals."""
    _dev(logits, out, err)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= rows
    scratch = zeroed_scratch(logits.device, "argmax", 16 * max(rows, 64))
    _check(_fn("sampling", "cml_argmax_rows")(_p(logits), logits.stride(0), rows, vocab, _p(out), _p(err), _p(scratch),
                                             _stream()), "argmax_rows")


def adjust_logits(logits: torch.Tensor, entries: torch.Tensor, biases: torch.Tensor, repeat_penalty: float,
                  presence_penalty: float, frequency_penalty: float):
    """entries: int32 [n, 3] of (row, token, count in history); biases: float32 [n]."""
    _dev(logits, entries, biases)
    n = entries.shape[0]
    assert entries.dtype == torch.int32 and entries.is_contiguous() and biases.dtype == torch.float32 and biases.numel() == n
    _check(_fn("sampling", "cml_adjust_logits")(_p(logits), logits.stride(0), logits.shape[1], _p(entries), _p(biases),
                                               n, float(repeat_penalty), float(presence_penalty),
                                               float(frequency_penalty), _stream()), "adjust_logits")


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float,
                draws: torch.Tensor, out: torch.Tensor, err: torch.Tensor, params=None):
    """One token per row of ``logits`` by the reference's stochastic sampler. ``params`` (float32 [4] on the
    device: temperature, top_k or 0, top_p or 1, min_p or 0), if given, is read by the kernel instead of
    the four arguments, so that a captured launch serves any values."""
    _dev(logits, draws, out, err, params)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and draws.dtype == torch.float32
    assert draws.numel() >= rows and out.dtype == torch.int32 and out.numel() >= rows
    _check(_fn("sampling", "cml_sample_rows")(_p(logits), logits.stride(0), rows, vocab, float(temperature),
                                             int(top_k or 0), float(top_p if top_p is not None else 1.0),
                                             float(min_p or 0.0), _p(params), _p(draws), _p(out), _p(err), _stream()),
           "sample_rows")


def adjust_dense(logits: torch.Tensor, counts: torch.Tensor, bias: torch.Tensor, penalties: torch.Tensor):
    """Bias and penalties from device-side state: ``counts`` int32 [rows, vocab] (how often a token
    stands in the row's history), ``bias`` float32 [vocab], ``penalties`` float32 [3] = repeat,
    presence, frequency. In place on ``logits`` (float32 [rows, vocab])."""
    _dev(logits, counts, bias, penalties)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and counts.dtype == torch.int32
    assert counts.shape == (rows, vocab) and counts.is_contiguous() and bias.numel() == vocab and penalties.numel() == 3
    assert bias.dtype == torch.float32 and penalties.dtype == torch.float32
    _check(_fn("sampling", "cml_adjust_dense")(_p(logits), logits.stride(0), rows, vocab, _p(counts), _p(bias),
                                              _p(penalties), _stream()), "adjust_dense")


def count_tokens(tokens: torch.Tensor, counts: torch.Tensor):
    """counts[r][tokens[r]] += 1 for the rows of ``counts`` (int32 [rows, vocab])."""
    _dev(tokens, counts)
    rows, vocab = counts.shape
    assert tokens.dtype == torch.int32 and tokens.numel() >= rows and counts.dtype == torch.int32 and counts.is_contiguous()
    _check(_fn("sampling", "cml_count_tokens")(_p(tokens), _p(counts), rows, vocab, _stream()), "count_tokens")


def draws_at(positions: torch.Tensor, seed: torch.Tensor, draws: torch.Tensor):
    """draws[r] = the draw of the stream of ``seed`` (int64 [1] on the device) for a history of
    positions[r] + 1 tokens: what ``sampling.options.unit_draw`` gives on the host."""
    _dev(positions, seed, draws)
    rows = draws.numel()
    assert positions.dtype == torch.int32 and positions.numel() >= rows and seed.dtype == torch.int64
    assert draws.dtype == torch.float32
    _check(_fn("sampling", "cml_draws_at")(_p(positions), _p(seed), _p(draws), rows, _stream()), "draws_at")


class NativeDecodeLoop:
    """The C++ decode loop (decode_loop.cu) bound to one captured step graph: ``run`` performs up
    to ``max_steps`` one-token steps (copy in, graph, sampling kernel, copy out) per call."""

    def __init__(self, n: int, layout, meta_dev: torch.Tensor, head_template, logits: torch.Tensor, err: torch.Tensor):
        import numpy as np
        dev = meta_dev.device
        size = _fn("sampling", "cml_decode_loop_size")()
        self._state = ctypes.create_string_buffer(size)
        self.n = n
        self.head_ints = layout.offsets["seq_start"][0] + n
        self.meta_host = torch.zeros(self.head_ints, dtype=torch.int32).pin_memory()
        self.meta_host.numpy()[:] = head_template[:self.head_ints]
        self.tokens_dev = torch.zeros(n, dtype=torch.int32, device=dev)
        self.tokens_host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.draws_dev = torch.zeros(n, dtype=torch.float32, device=dev)
        self.draws_host = torch.zeros(n, dtype=torch.float32).pin_memory()
        self.scratch = zeroed_scratch(dev, "argmax", 16 * max(n, 64))
        self.logits, self.err, self.meta_dev = logits, err, meta_dev
        self._np = np
        _check(_fn("sampling", "cml_decode_loop_init")(
            ctypes.addressof(self._state), n, layout.offsets["tokens"][0], layout.offsets["row_pos"][0],
            layout.offsets["seq_slot"][0], layout.offsets["seq_start"][0], self.head_ints, _p(meta_dev), _p(self.meta_host), _p(logits),
            logits.stride(0), logits.shape[1], _p(self.tokens_dev), _p(self.tokens_host), _p(err), _p(self.scratch),
            _p(self.draws_dev), _p(self.draws_host)), "decode_loop_init", 0)
        self.h2d_bytes_per_step = self.head_ints * 4
        self.d2h_bytes_per_step = n * 4

    def run(self, graph_exec: int, tokens, positions, slots, history_lens, max_steps: int, stop_ids, temperature: float,
            top_k: int, top_p: float, min_p: float, seed: int, launches_per_step: int):
        np = self._np
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        slo = np.ascontiguousarray(slots, dtype=np.int32)
        assert tok.size == pos.size == slo.size == self.n
        hist = np.ascontiguousarray(history_lens, dtype=np.int32)
        stops = np.ascontiguousarray(list(stop_ids), dtype=np.int32)
        out = np.empty((max_steps, self.n), dtype=np.int32)
        done = ctypes.c_int(0)
        rc = _fn("sampling", "cml_decode_loop_run")(
            ctypes.addressof(self._state), graph_exec, _stream(), tok.ctypes.data, pos.ctypes.data, slo.ctypes.data,
            hist.ctypes.data,
            max_steps, stops.ctypes.data if stops.size else None, int(stops.size), float(temperature), int(top_k or 0),
            float(top_p if top_p is not None else 1.0), float(min_p or 0.0), int(seed or 0), out.ctypes.data,
            ctypes.addressof(done))
        _check(rc, "decode_loop_run", (launches_per_step + 1) * done.value)
        return out[:done.value], done.value


class FedDecodeLoop:
    """The C++ loop for a captured step graph that picks the greedy token itself and feeds it to
    the next step on the device: ``run`` queues all its steps at once and waits once."""
    RING = 256                  # steps one call can queue

    def __init__(self, n: int, layout, meta_dev: torch.Tensor, head_template):
        import numpy as np
        self._np = np
        self.n = n
        self.offsets = [layout.offsets[k][0] for k in ("tokens", "row_pos", "seq_slot", "seq_start")]
        self.head_ints = layout.offsets["seq_start"][0] + n
        self.meta_dev = meta_dev
        self.ring = torch.zeros((self.RING, self.head_ints), dtype=torch.int32).pin_memory()
        self.ring.numpy()[:] = head_template[:self.head_ints]
        self.out = torch.zeros((self.RING, n), dtype=torch.int32).pin_memory()
        self.h2d_bytes_per_step = (self.head_ints - n) * 4
        self.d2h_bytes_per_step = n * 4

    def run(self, graph_exec: int, tokens, positions, slots, steps: int, launches_per_step: int):
        np = self._np
        assert 1 <= steps <= self.RING
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        slo = np.ascontiguousarray(slots, dtype=np.int32)
        assert tok.size == pos.size == slo.size == self.n
        rc = _fn("sampling", "cml_decode_fed_run")(
            self.n, *self.offsets, self.head_ints, _p(self.meta_dev), self.ring.data_ptr(), graph_exec, _stream(),
            tok.ctypes.data, pos.ctypes.data, slo.ctypes.data, int(steps), self.out.data_ptr())
        _check(rc, "decode_fed_run", launches_per_step * steps)
        return self.out.numpy()[:steps].copy()
