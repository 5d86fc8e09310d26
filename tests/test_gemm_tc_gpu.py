"""The tensor-core matrix product (TMA + tcgen05) alone against float64 products, in both
orientations, with ragged edges in every dimension and split K."""
import math

import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _ops():
    from camelid_b200.csrc import ops
    return ops


def _operands(m, n, k, cuda, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(BF).to(cuda)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(BF).to(cuda)
    return a, w, a.cpu().double() @ w.cpu().double().T


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (200, 300, 136), (1000, 520, 192), (65, 517, 72), (2048, 1024, 2048)])
def test_normal_orientation(cuda, m, n, k, bn):
    ops = _ops()
    a, w, ref = _operands(m, n, k, cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    c = torch.full((m, n), float("nan"), dtype=BF, device=cuda)
    ops.gemm_tc(a, w, c, ops.TC_STORE, bn, 1, err)
    assert rel_err(c.cpu(), ref) <= 2 ** -8
    c32 = torch.full((m, n), float("nan"), device=cuda)
    ops.gemm_tc(a, w, c32, ops.TC_STORE_F32, bn, 1, err)
    assert rel_err(c32.cpu(), ref) <= 1e-5
    res = torch.randn(m, n, device=cuda)
    want = res.cpu().double() + ref
    ops.gemm_tc(a, w, res, ops.TC_ADD_F32, bn, 1, err)
    assert rel_err(res.cpu(), want) <= 1e-5
    assert int(err) == 0


def test_strided_operands_and_output(cuda):
    ops = _ops()
    a, w, _ = _operands(300, 200, 128, cuda)
    wide = torch.randn(300, 136).to(BF).to(cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    c = torch.full((300, 208), float("nan"), device=cuda)
    ops.gemm_tc(wide[:, 8:], w, c[:, :200], ops.TC_STORE_F32, 128, 1, err)
    assert rel_err(c[:, :200].cpu(), wide[:, 8:].cpu().double() @ w.cpu().double().T) <= 1e-5
    assert torch.isnan(c[:, 200:]).all()
    assert not ops.gemm_tc_usable(wide[:, 4:], w[:, :132])          # K and strides must be multiples of 8


@pytest.mark.parametrize("m,inter,k", [(300, 160, 64), (130, 528, 200), (1024, 2048, 512)])
def test_swiglu_normal(cuda, m, inter, k):
    ops = _ops()
    from camelid_b200.parts.linear import pack_gate_up
    x, wg, g = _operands(m, inter, k, cuda, 1)
    _, wu, _ = _operands(m, inter, k, cuda, 2)
    u = x.cpu().double() @ wu.cpu().double().T
    ref = (g / (1 + torch.exp(-g))) * u
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    for bn in (64, 128, 256):
        act = torch.full((m, inter), float("nan"), dtype=BF, device=cuda)
        ops.gemm_tc(x, pack_gate_up(wg, wu, 16), act, ops.TC_SWIGLU, bn, 1, err)
        assert rel_err(act.cpu(), ref) <= 2 ** -7, bn


def _bn_for(rows):
    return next((bn for bn in (16, 32, 64) if rows <= bn), 128)


@pytest.mark.parametrize("rows", [1, 8, 17, 64, 100, 129, 256, 300])
@pytest.mark.parametrize("n,k,splits", [(100, 64, 1), (384, 200, 3), (3072, 2048, 6), (2048, 8192, 9), (517, 136, 7)])
def test_transposed_partials(cuda, rows, n, k, splits):
    """Weights as the 128-row operand, the step's rows as the other (tiles of 16 to 128 of them,
    several tiles beyond that), K split."""
    ops = _ops()
    x, w, ref = _operands(rows, n, k, cuda, 3)
    bn = _bn_for(rows)
    splits = min(splits, (k + 63) // 64)
    part = torch.full((splits, rows, n), float("nan"), device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    ops.gemm_tc(w, x, part, ops.TC_T_PARTIAL, bn, splits, err)
    assert rel_err(part.sum(0).cpu(), ref) <= 1e-5
    assert int(err) == 0


@pytest.mark.parametrize("rows", [1, 8, 33, 90, 200, 260])
@pytest.mark.parametrize("inter,k", [(160, 64), (528, 200), (8192, 2048)])
def test_swiglu_transposed(cuda, rows, inter, k):
    ops = _ops()
    from camelid_b200.parts.linear import pack_gate_up
    x, wg, g = _operands(rows, inter, k, cuda, 4)
    _, wu, _ = _operands(rows, inter, k, cuda, 5)
    u = x.cpu().double() @ wu.cpu().double().T
    ref = (g / (1 + torch.exp(-g))) * u
    bn = _bn_for(rows)
    act = torch.full((rows, inter), float("nan"), dtype=BF, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    ops.gemm_tc(pack_gate_up(wg, wu, 16), x, act, ops.TC_T_SWIGLU, bn, 1, err)
    assert rel_err(act.cpu(), ref) <= 2 ** -7


@pytest.mark.parametrize("rows,hidden,splits", [(5, 96, 3), (8, 2048, 9), (3, 517, 4), (2, 8192, 20), (1, 3000, 1), (6, 6, 2)])
@pytest.mark.parametrize("out_dtype", [torch.float32, BF])
def test_consumers_of_split_sums(cuda, rows, hidden, splits, out_dtype):
    """The norm adds the split sums itself, row first and then split by split (rows that are
    whole 16-byte groups by cp.async through shared memory, others element by element)."""
    ops = _ops()
    import plain_llama as pl
    g = torch.Generator().manual_seed(0)
    h = torch.randn(rows, hidden, generator=g).to(cuda)
    part = torch.randn(splits, rows, hidden, generator=g).to(cuda)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(cuda)
    total = h.cpu().double()
    exact = h.cpu().clone()
    for sp in range(splits):
        total = total + part[sp].cpu().double()
        exact = exact + part[sp].cpu()                                  # the kernel's order, in float32
    tol = 1e-5 if out_dtype == torch.float32 else 2 ** -8
    out = torch.empty(rows, hidden, dtype=out_dtype, device=cuda)
    h2 = h.clone()
    ops.rmsnorm(h2, w, 1e-5, out, None, part)
    assert torch.equal(h2.cpu(), exact)
    assert rel_err(out.cpu(), pl.rms_norm(total, w.cpu().double(), 1e-5)) <= tol
    pick = [rows - 1, rows - 1, 0]
    idx = torch.tensor(pick, dtype=torch.int32, device=cuda)
    h3 = h.clone()
    out3 = torch.empty(3, hidden, dtype=out_dtype, device=cuda)
    ops.rmsnorm(h3, w, 1e-5, out3, idx, part)
    assert torch.equal(h3, h)                                           # gathered rows: nothing is written back
    assert rel_err(out3.cpu(), pl.rms_norm(total[pick], w.cpu().double(), 1e-5)) <= tol
    h4 = h.clone()
    ops.add_partials(h4, part)
    assert rel_err(h4.cpu(), total) <= 1e-6


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 300, 136), (1000, 520, 192), (129, 517, 72), (2048, 1024, 2048),
                                   (513, 2048, 1088), (4096, 768, 4104)])
def test_pair_tiles(cuda, m, n, k):
    """Tiles of 256 x 256 shared by two blocks of a cluster: ragged edges in every dimension,
    row counts that leave the second block of a pair without rows, many k-blocks, several
    tiles per cluster."""
    ops = _ops()
    a, w, ref = _operands(m, n, k, cuda, seed=3)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    c = torch.full((m, n), float("nan"), dtype=BF, device=cuda)
    ops.gemm_tc_pair(a, w, c, ops.TC_STORE, err)
    assert rel_err(c.cpu(), ref) <= 2 ** -8
    c32 = torch.full((m, n), float("nan"), device=cuda)
    ops.gemm_tc_pair(a, w, c32, ops.TC_STORE_F32, err)
    assert rel_err(c32.cpu(), ref) <= 1e-5
    res = torch.randn(m, n, device=cuda)
    want = res.cpu().double() + ref
    ops.gemm_tc_pair(a, w, res, ops.TC_ADD_F32, err)
    assert rel_err(res.cpu(), want) <= 1e-5
    assert int(err) == 0


@pytest.mark.parametrize("m,n,k,splits", [(300, 300, 136, 3), (512, 2048, 8192, 4), (257, 517, 2048, 5), (1000, 3072, 2048, 3),
                                          (400, 256, 64, 2), (300, 2048, 1088, 17)])
def test_pair_tiles_split_over_k(cuda, m, n, k, splits):
    """The two-block tiles with K split into partial sums (the splits are work items of their
    own): ragged edges, more splits asked than there are k-blocks, rows that still lack a scale."""
    ops = _ops()
    a, w, ref = _operands(m, n, k, cuda, seed=6)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    n_splits = ops.pair_partial_splits(k, splits)
    assert 1 <= n_splits <= min(splits, (k + 63) // 64)
    part = torch.full((n_splits, m, n), float("nan"), device=cuda)
    ops.gemm_tc_pair_partial(a, w, part, err)
    assert rel_err(part.sum(0).cpu(), ref) <= 1e-5
    if n_splits > 1:                              # every split holds only its own share
        per = -(-((k + 63) // 64) // n_splits) * 64
        first = a.cpu().double()[:, :per] @ w.cpu().double()[:, :per].T
        assert rel_err(part[0].cpu(), first) <= 1e-5
    sumsq = torch.rand(2, m, device=cuda) * 50 + 1
    scale = torch.rsqrt(sumsq.sum(0).cpu().double() / 77 + 1e-5)
    part.fill_(float("nan"))
    ops.gemm_tc_pair_partial(a, w, part, err, ops.RowScale(sumsq, 77, 1e-5))
    assert rel_err(part.sum(0).cpu(), ref * scale[:, None]) <= 1e-5
    with pytest.raises(Exception):
        ops.gemm_tc_pair_partial(a, w, torch.empty(n_splits + 64, m, n, device=cuda), err)
    assert int(err) == 0


@pytest.mark.parametrize("m,inter,k", [(300, 160, 64), (130, 528, 200), (1024, 2048, 512), (2048, 8192, 256)])
def test_pair_tiles_swiglu(cuda, m, inter, k):
    ops = _ops()
    from camelid_b200.parts.linear import pack_gate_up
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=g).to(BF).to(cuda)
    wg = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(BF)
    wu = (torch.randn(inter, k, generator=g) / math.sqrt(k)).to(BF)
    packed = pack_gate_up(wg, wu, 16).to(cuda)
    gate = x.cpu().double() @ wg.double().T
    ref = torch.nn.functional.silu(gate) * (x.cpu().double() @ wu.double().T)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    out = torch.full((m, inter), float("nan"), dtype=BF, device=cuda)
    for bn in (128, 256):
        out.fill_(float("nan"))
        ops.gemm_tc_pair(x, packed, out, ops.TC_SWIGLU, err)
        assert rel_err(out.cpu(), ref) <= 2 ** -7, bn
    assert int(err) == 0


@pytest.mark.parametrize("w_dtype", [torch.float32, BF])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 136), (2048, 2048, 512), (513, 72, 200)])
def test_pair_product_with_the_norm_split_over_two_products(cuda, m, n, k, w_dtype):
    """The product before a norm adds into the residual stream and writes the rows times the
    norm's weight and their sums of squares; the product after it applies the rows' scale to its
    output. Together: the plain residual add, RMS norm and product."""
    import plain_llama as pl
    ops = _ops()
    a, w, prod = _operands(m, n, k, cuda, seed=6)
    g = torch.Generator().manual_seed(8)
    h0 = torch.randn(m, n, generator=g)
    norm_w = (1 + 0.1 * torch.randn(n, generator=g)).to(w_dtype)
    eps = 1e-5
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    h = h0.to(cuda)
    x_out = torch.full((m, n), float("nan"), dtype=BF, device=cuda)
    sumsq = torch.full(((n + 255) // 256, m), float("nan"), device=cuda)
    scale = ops.gemm_tc_pair_add_norm(a, w, h, err, norm_w.to(cuda), eps, x_out, sumsq)
    want_h = h0.double() + prod
    assert rel_err(h.cpu(), want_h) <= 1e-5
    assert rel_err(scale.sumsq.sum(dim=0).cpu(), (want_h * want_h).sum(dim=-1)) <= 1e-5
    normed = pl.rms_norm(want_h, norm_w.double(), eps)
    # scaled in place: the norm's output
    x_done = x_out.clone()
    ops.scale_rows(x_done, scale)
    assert rel_err(x_done.cpu(), normed) <= 2 ** -7
    # or left to the next product, which scales its own output rows
    n2 = 264 if n % 8 == 0 else 64
    w2 = (torch.randn(n2, n, generator=g) / math.sqrt(n)).to(BF).to(cuda)
    ref2 = normed.to(BF).double() @ w2.cpu().double().T
    out2 = torch.full((m, n2), float("nan"), dtype=BF, device=cuda)
    ops.gemm_tc_pair(x_out, w2, out2, ops.TC_STORE, err, scale)
    assert rel_err(out2.cpu(), ref2) <= 2 ** -6
    from camelid_b200.parts.linear import pack_gate_up
    inter = 48
    wg = (torch.randn(inter, n, generator=g) / math.sqrt(n)).to(BF)
    wu = (torch.randn(inter, n, generator=g) / math.sqrt(n)).to(BF)
    xn = normed.to(BF).double()
    ref3 = torch.nn.functional.silu(xn @ wg.double().T) * (xn @ wu.double().T)
    out3 = torch.full((m, inter), float("nan"), dtype=BF, device=cuda)
    ops.gemm_tc_pair(x_out, pack_gate_up(wg, wu, 16).to(cuda), out3, ops.TC_SWIGLU, err, scale)
    assert rel_err(out3.cpu(), ref3) <= 2 ** -6
    assert int(err) == 0
