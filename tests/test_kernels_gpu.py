"""Each kernel alone against its plain reference, at other sizes than the engine's tests,
with inputs made so that an addressing fault shows (a far key that dominates, a window's
edge, stale and non-finite contents in unused cache rows)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
from helpers import TOL, rel_err

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _i32(x, dev):
    return torch.tensor(x, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,hidden,vocab", [(7, 72, 101), (3, 2048, 50)])
def test_embed_gather(cuda, dtype, rows, hidden, vocab):
    from camelid_b200.csrc import ops
    table = torch.randn(vocab, hidden).to(DT[dtype]).to(cuda)
    toks = torch.randint(0, vocab, (rows,), dtype=torch.int32, device=cuda)
    out = torch.empty(rows, hidden, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    ops.embed_gather(table, toks, out, err)
    assert torch.equal(out, table.float()[toks.long()]) and int(err) == 0
    toks[1] = vocab
    ops.embed_gather(table, toks, out, err)
    assert int(err) == 1 and float(out[1].abs().max()) == 0.0


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("w_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,hidden,eps", [(5, 72, 1e-5), (2, 3000, 1e-6), (1, 16, 1e-2)])
def test_rmsnorm(cuda, out_dtype, w_dtype, rows, hidden, eps):
    from camelid_b200.csrc import ops
    x = (torch.randn(rows + 3, hidden) * 3).to(cuda)
    w = (1 + 0.1 * torch.randn(hidden)).to(DT[w_dtype]).to(cuda)
    idx = _i32([(r * 2) % (rows + 3) for r in range(rows)], cuda)
    out = torch.empty(rows, hidden, dtype=DT[out_dtype], device=cuda)
    ops.rmsnorm(x, w, eps, out, idx)
    ref = pl.rms_norm(x.cpu().double()[idx.cpu().long()], w.cpu().double(), eps)
    tol = 1e-5 if out_dtype == "float32" else 2 ** -8
    assert rel_err(out.cpu(), ref) <= tol
    ops.rmsnorm(x, w, eps, out[:1], None)
    assert rel_err(out[:1].cpu(), pl.rms_norm(x[:1].cpu().double(), w.cpu().double(), eps)) <= tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 40, 24), (70, 130, 200), (129, 64, 1030), (5, 517, 96), (300, 520, 136),
                                   (2048, 384, 2048), (64, 129, 4), (257, 128, 20)])
def test_gemm_simt_epilogues(cuda, dtype, M, N, K):
    from camelid_b200.csrc import ops
    a = torch.randn(M, K).to(DT[dtype]).to(cuda)
    w = (torch.randn(N, K) / math.sqrt(K)).to(DT[dtype]).to(cuda)
    ref = a.cpu().double() @ w.cpu().double().T
    tol = 1e-5 if dtype == "float32" else 2 ** -8
    c = torch.empty(M, N, dtype=DT[dtype], device=cuda)
    ops.gemm_tn_simt(a, w, c, ops.EPI_STORE)
    assert rel_err(c.cpu(), ref) <= tol
    c32 = torch.empty(M, N, device=cuda)
    ops.gemm_tn_simt(a, w, c32, ops.EPI_STORE_F32)
    assert rel_err(c32.cpu(), ref) <= 1e-5
    res = torch.randn(M, N, device=cuda)
    want = res.cpu().double() + ref
    ops.gemm_tn_simt(a, w, res, ops.EPI_ADD_F32)
    assert rel_err(res.cpu(), want) <= 1e-5
    # rows of a wider matrix (strided views), as the attention mixer uses
    wide = torch.randn(M, K + 8).to(DT[dtype]).to(cuda)
    ops.gemm_tn_simt(wide[:, 8:], w, c32, ops.EPI_STORE_F32)
    assert rel_err(c32.cpu(), wide[:, 8:].cpu().double() @ w.cpu().double().T) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 2048, 2048), (8, 2048, 8192), (5, 517, 132), (32, 100, 640),
                                   (17, 33, 4100), (2, 128256, 256), (8, 40, 128), (64, 96, 640), (41, 2048, 2048)])
def test_gemv_float_streaming_form(cuda, M, N, K):
    """Float products of at most 64 rows whose sizes allow 16-byte loads: tiles of 32 weight rows,
    K split over blocks where there are few tiles, the splits summed in index order by the
    block that comes last. Every epilogue; tickets are left zero, so a second call is as good; a row's
    value does not depend on the other rows of the step."""
    from camelid_b200.csrc import ops
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    a = torch.randn(M, K, generator=g).to(cuda)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(cuda)
    ref = a.cpu().double() @ w.cpu().double().T
    for rep in range(2):
        c = torch.full((M, N), float("nan"), device=cuda)
        ops.gemm_tn_simt(a, w, c, ops.EPI_STORE_F32)
        assert rel_err(c.cpu(), ref) <= 2e-6, rep
    res = torch.randn(M, N, generator=g).to(cuda)
    want = res.cpu().double() + ref
    ops.gemm_tn_simt(a, w, res, ops.EPI_ADD_F32)
    assert rel_err(res.cpu(), want) <= 2e-6
    one = torch.empty(1, N, device=cuda)
    ops.gemm_tn_simt(a[M - 1:], w, one, ops.EPI_STORE_F32)
    assert torch.equal(one[0], c[M - 1]), "a row alone differs from the same row in a step of several"
    # products of other shapes share the scratch: their sums must not land on this one's tickets
    other = torch.randn(8, 4096, generator=g).to(cuda)
    ops.gemm_tn_simt(other, torch.randn(64, 4096, generator=g).to(cuda), torch.empty(8, 64, device=cuda), ops.EPI_STORE_F32)
    ops.gemm_tn_simt(a, w, c, ops.EPI_STORE_F32)
    assert rel_err(c.cpu(), ref) <= 2e-6
    if N % 32 == 0:
        inter = N // 2
        act = torch.full((M, inter), float("nan"), device=cuda)
        from camelid_b200.parts.linear import pack_gate_up
        packed = pack_gate_up(w[:inter].contiguous(), w[inter:].contiguous(), 16)
        ops.gemm_tn_simt(a, packed, act, ops.EPI_SWIGLU, 16)
        gate, up = ref[:, :inter], ref[:, inter:]
        assert rel_err(act.cpu(), (gate / (1 + torch.exp(-gate))) * up) <= 2e-6
    # rows of a wider matrix (a strided view whose rows still start on 16-byte boundaries)
    wide = torch.randn(M, K + 8, generator=g).to(cuda)
    ops.gemm_tn_simt(wide[:, 8:], w, c, ops.EPI_STORE_F32)
    assert rel_err(c.cpu(), wide[:, 8:].cpu().double() @ w.cpu().double().T) <= 2e-6
    assert int(ops.simt_error_word(cuda).item()) == 0


@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 2048, 2048), (8, 2048, 8192), (5, 517, 260), (3, 33, 4100),
                                   (8, 40, 256), (7, 100, 648), (64, 2048, 2048), (19, 96, 1024)])
def test_gemv_float_partial_sums(cuda, M, N, K):
    """The streaming float product with its K ranges left as partial sums: their sum in range order is the
    product; ranges do not overlap or leave a gap (a row of ones against weights that name their column)."""
    from camelid_b200.csrc import ops
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(cuda)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(cuda)
    splits = ops.gemv_f32_partial_splits(a, w)
    assert splits >= 1
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    part = torch.full((splits, M, N), float("nan"), device=cuda)
    ops.gemv_f32_partial(a, w, part, err)
    assert int(err.item()) == 0
    assert rel_err(part.sum(0).cpu(), a.cpu().double() @ w.cpu().double().T) <= 2e-6
    ones = torch.ones(M, K, device=cuda)
    cols = torch.arange(K, dtype=torch.float32, device=cuda).repeat(N, 1).contiguous()
    ops.gemv_f32_partial(ones, cols, part, err)
    per = part[:, 0, 0].cpu().double()
    assert (per > 0).all() or K < 256, per                   # no empty range
    assert float(per.sum()) == K * (K - 1) / 2               # exact in float up to 2^24 per range
    assert ops.gemv_f32_partial_splits(torch.randn(65, K, device=cuda), w) == 0      # more than 64 rows: not taken


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,inter,K,group", [(3, 48, 40, 16), (66, 136, 72, 136), (9, 160, 64, 16), (200, 160, 64, 16),
                                             (129, 8192, 256, 16), (64, 16, 12, 16)])
def test_gemm_swiglu_and_packing(cuda, dtype, M, inter, K, group):
    from camelid_b200.csrc import ops
    from camelid_b200.parts.linear import pack_gate_up
    x = torch.randn(M, K).to(DT[dtype]).to(cuda)
    wg = (torch.randn(inter, K) / math.sqrt(K)).to(DT[dtype]).to(cuda)
    wu = (torch.randn(inter, K) / math.sqrt(K)).to(DT[dtype]).to(cuda)
    packed = pack_gate_up(wg, wu, group)
    g = x.cpu().double() @ wg.cpu().double().T
    u = x.cpu().double() @ wu.cpu().double().T
    ref = (g / (1 + torch.exp(-g))) * u
    act = torch.empty(M, inter, dtype=DT[dtype], device=cuda)
    ops.gemm_tn_simt(x, packed, act, ops.EPI_SWIGLU, group)
    tol = 1e-5 if dtype == "float32" else 2 ** -7
    assert rel_err(act.cpu(), ref) <= tol
    gu = torch.empty(M, 2 * inter, dtype=DT[dtype], device=cuda)
    ops.gemm_tn_simt(x, packed, gu, ops.EPI_STORE)
    act2 = torch.empty_like(act)
    ops.swiglu_packed(gu, act2, group)
    assert rel_err(act2.cpu(), ref) <= (1e-5 if dtype == "float32" else 2 ** -6)


def _paged(seq_lens, n_kv, hd, dtype, dev, n_pages=64, seed=0):
    """Random keys and values for sequences of the given lengths, scattered over shuffled
    pages; unused rows hold NaN."""
    g = torch.Generator().manual_seed(seed)
    k_pages = torch.full((n_pages, n_kv, 64, hd), float("nan")).to(dtype)
    v_pages = torch.full((n_pages, n_kv, 64, hd), float("nan")).to(dtype)
    perm = torch.randperm(n_pages, generator=g).tolist()
    tables, ks, vs = [], [], []
    for n in seq_lens:
        k = torch.randn(n, n_kv, hd, generator=g).to(dtype)
        v = torch.randn(n, n_kv, hd, generator=g).to(dtype)
        blocks = [perm.pop() for _ in range((n + 63) // 64)]
        for p in range(n):
            k_pages[blocks[p // 64], :, p % 64] = k[p]
            v_pages[blocks[p // 64], :, p % 64] = v[p]
        tables.append(blocks)
        ks.append(k)
        vs.append(v)
    width = max(len(t) for t in tables)
    table = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    return k_pages.to(dev), v_pages.to(dev), table.to(dev), ks, vs


def _attn_case(cuda, dtype, n_heads, n_kv, hd, starts, news, window, decode, n_splits=1, spike=None):
    from camelid_b200.csrc import ops
    dt = DT[dtype]
    totals = [s + n for s, n in zip(starts, news)]
    k_pages, v_pages, table, ks, vs = _paged(totals, n_kv, hd, dt, cuda)
    g = torch.Generator().manual_seed(1)
    n_rows = sum(news)
    q = torch.randn(n_rows, n_heads, hd, generator=g).to(dt)
    row0 = [sum(news[:i]) for i in range(len(news))]
    if spike is not None:            # one far key gets a score that stands out for one query
        seq, key = spike
        r = row0[seq] + news[seq] - 1
        ks[seq][key] *= 0
        ks[seq][key, :, 0] = 8.0
        q[r, :, 0] = 8.0 * math.sqrt(hd) / 4
        k_pages[int(table[seq, key // 64]), :, key % 64] = ks[seq][key].to(cuda)
    rows, hpc, chunks = ops.attn_tiling(n_heads, n_kv, decode)
    tile_seq, tile_q0 = [], []
    for i, n in enumerate(news):
        for q0 in range(0, n, rows):
            tile_seq.append(i)
            tile_q0.append(q0)
    out = torch.empty(n_rows, n_heads * hd, dtype=dt, device=cuda)
    partial = torch.empty(max(1, ops.attn_partial_floats(n_rows, n_heads, hd, n_splits)), device=cuda)
    ops.attn_paged_simt(q.view(n_rows, -1).to(cuda), out, k_pages, v_pages, table, _i32(tile_seq, cuda),
                        _i32(tile_q0, cuda), len(tile_seq), _i32(row0, cuda), _i32(starts, cuda), _i32(news, cuda),
                        n_rows, n_heads, n_kv, hd, rows, hpc, chunks, n_splits, window or 0, 1 / math.sqrt(hd), partial)
    out = out.cpu().view(n_rows, n_heads, hd)
    for i, (s, n) in enumerate(zip(starts, news)):
        qfull = torch.zeros(s + n, n_heads, hd, dtype=torch.float64)
        qfull[s:] = q[row0[i]:row0[i] + n].double()
        ref = pl.attention(qfull, ks[i].double(), vs[i].double(), window)[s:]
        e = rel_err(out[row0[i]:row0[i] + n], ref)
        assert e <= (1e-5 if dtype == "float32" else 2 ** -7), f"sequence {i}: {e}"
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 2, 16), (6, 1, 32), (5, 5, 48), (8, 2, 128), (34, 1, 64), (2, 1, 256)])
def test_attention_prefill_shapes(cuda, dtype, n_heads, n_kv, hd):
    _attn_case(cuda, dtype, n_heads, n_kv, hd, starts=[0, 0, 0], news=[1, 70, 129], window=None, decode=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_continues_from_cache_and_far_key(cuda, dtype):
    """New rows on top of cached positions; one key hundreds of positions back dominates the
    last query of the second sequence: if a page were addressed wrongly it would show."""
    out = _attn_case(cuda, dtype, 4, 2, 32, starts=[64, 300, 5], news=[3, 20, 64], window=None, decode=False,
                     spike=(1, 7))
    assert out is not None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_splits", [1, 2, 5, 16])
def test_attention_decode_splits(cuda, dtype, n_splits):
    """One new row per sequence, keys split over several blocks (also more splits than pages)."""
    _attn_case(cuda, dtype, 8, 2, 64, starts=[0, 63, 64, 700], news=[1, 1, 1, 1], window=None, decode=True,
               n_splits=n_splits, spike=(3, 130))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv,hd", [(3, 1, 16), (6, 1, 48), (5, 5, 32), (12, 2, 128), (2, 1, 256), (34, 1, 64)])
def test_attention_decode_shapes(cuda, dtype, n_heads, n_kv, hd):
    """Decode tiling of the float kernel at other groupings and head sizes: groups that do not fill a block's 2 or
    4 heads (3, 6, 34 heads on one kv head), single heads (their own warp each), the largest head size (one
    page deep)."""
    _attn_case(cuda, dtype, n_heads, n_kv, hd, starts=[0, 5, 64, 130], news=[1, 1, 1, 1], window=None, decode=True,
               n_splits=2, spike=(3, 70))
    _attn_case(cuda, dtype, n_heads, n_kv, hd, starts=[17, 200], news=[1, 1], window=40, decode=True, n_splits=1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("edge", [0, 1], ids=["first key outside", "first key inside"])
@pytest.mark.parametrize("window", [1, 64, 70, 199])
def test_attention_window_edges(cuda, dtype, window, edge):
    """The query at position 199 sees keys 200 - window .. 199. A key just outside the window must
    not count and the first one inside must: the outstanding key sits on each in turn."""
    _attn_case(cuda, dtype, 4, 2, 32, starts=[0, 190], news=[150, 10], window=window, decode=False,
               spike=(1, 199 - window + edge))
    _attn_case(cuda, dtype, 4, 2, 32, starts=[199, 80], news=[1, 1], window=window, decode=True, n_splits=3,
               spike=(0, 199 - window + edge))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv,hd,rot", [(4, 2, 16, 16), (3, 1, 48, 32), (2, 2, 64, 0), (32, 8, 64, 64), (5, 1, 128, 64),
                                                 (3, 3, 48, 24), (2, 1, 32, 6)])
def test_rope_kv_write(cuda, dtype, n_heads, n_kv, hd, rot):
    from camelid_b200.csrc import ops
    from camelid_b200.parts.position import rotary_frequencies
    dt = DT[dtype]
    cfg = {"hidden_size": rot, "num_attention_heads": 1, "head_dim": rot, "rope_theta": 10000.0}
    freqs = rotary_frequencies(rot, 10000.0, None) if rot else np.zeros(0, dtype=np.float32)
    if rot:
        assert np.array_equal(freqs, pl.rope_frequencies(cfg))
    positions = [0, 1, 63, 64, 130, 5]
    seqs = [0, 0, 0, 0, 0, 1]
    table = _i32([[9, 2, 4], [7, -1, -1]], cuda)
    width = (n_heads + 2 * n_kv) * hd
    qkv = torch.randn(len(positions), width + 5).to(dt)
    k_pages = torch.zeros(12, n_kv, 64, hd, dtype=dt, device=cuda)
    v_pages = torch.zeros_like(k_pages)
    dev = qkv.to(cuda)[:, :width]
    ops.rope_kv_write(dev, _i32(positions, cuda), _i32(seqs, cuda), table, k_pages, v_pages,
                      torch.from_numpy(freqs).to(cuda), rot, n_heads, n_kv, hd, True)
    q = qkv[:, :n_heads * hd].double().view(-1, n_heads, hd)
    k = qkv[:, n_heads * hd:(n_heads + n_kv) * hd].double().view(-1, n_kv, hd)
    v = qkv[:, (n_heads + n_kv) * hd:width].view(-1, n_kv, hd)
    pos = torch.tensor(positions)
    q_ref = pl.rope(q, pos, freqs) if rot else q
    k_ref = pl.rope(k, pos, freqs) if rot else k
    tol = 1e-6 if dtype == "float32" else 2 ** -8
    assert rel_err(dev.cpu()[:, :n_heads * hd].view(-1, n_heads, hd), q_ref) <= tol
    tab = table.cpu()
    for r, (p, s) in enumerate(zip(positions, seqs)):
        page = int(tab[s, p // 64])
        assert rel_err(k_pages[page, :, p % 64].cpu(), k_ref[r]) <= tol
        assert torch.equal(v_pages[page, :, p % 64].cpu(), v[r])
    assert int((k_pages != 0).any(dim=-1).sum()) <= len(positions) * n_kv     # nothing else was written
    before = k_pages.clone()
    ops.rope_kv_write(dev, _i32(positions, cuda), _i32(seqs, cuda), table, k_pages, v_pages,
                      torch.from_numpy(freqs).to(cuda), rot, n_heads, n_kv, hd, False)
    assert torch.equal(before, k_pages)


def test_kernels_refuse_what_they_cannot_do(cuda):
    from camelid_b200 import KernelError
    from camelid_b200.csrc import ops
    with pytest.raises(KernelError):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.zeros(2, 8))          # CPU tensors
    with pytest.raises(KernelError):
        ops.dtype_code(torch.float16)
    a = torch.zeros(4, 8, device=cuda)
    with pytest.raises(KernelError):
        ops.gemm_tn_simt(a, torch.zeros(6, 8, device=cuda), torch.zeros(4, 3, device=cuda), ops.EPI_SWIGLU, 2)


# ---- the tensor-core attention kernel (bfloat16, head sizes 64 and 128) ----

def _attn_mma_case(cuda, n_heads, n_kv, hd, starts, news, window, decode, n_splits=1, spike=None):
    from camelid_b200.csrc import ops
    dt = torch.bfloat16
    totals = [s + n for s, n in zip(starts, news)]
    k_pages, v_pages, table, ks, vs = _paged(totals, n_kv, hd, dt, cuda)
    g = torch.Generator().manual_seed(1)
    n_rows = sum(news)
    q = torch.randn(n_rows, n_heads, hd, generator=g).to(dt)
    row0 = [sum(news[:i]) for i in range(len(news))]
    if spike is not None:
        seq, key = spike
        r = row0[seq] + news[seq] - 1
        ks[seq][key] *= 0
        ks[seq][key, :, 0] = 8.0
        q[r, :, 0] = 8.0 * math.sqrt(hd) / 4
        k_pages[int(table[seq, key // 64]), :, key % 64] = ks[seq][key].to(cuda)
    rows, hpc, chunks = ops.attn_mma_tiling(n_heads, n_kv, decode)
    tile_seq, tile_q0 = [], []
    for i, n in enumerate(news):
        for q0 in range(0, n, rows):
            tile_seq.append(i)
            tile_q0.append(q0)
    out = torch.full((n_rows, n_heads * hd), float("nan"), dtype=dt, device=cuda)
    partial = torch.empty(max(1, ops.attn_partial_floats(n_rows, n_heads, hd, n_splits)), device=cuda)
    ops.attn_paged_mma(q.view(n_rows, -1).to(cuda), out, k_pages, v_pages, table, _i32(tile_seq, cuda),
                       _i32(tile_q0, cuda), len(tile_seq), _i32(row0, cuda), _i32(starts, cuda), _i32(news, cuda),
                       n_rows, n_heads, n_kv, hd, rows, hpc, chunks, n_splits, window or 0, 1 / math.sqrt(hd), partial)
    out = out.cpu().view(n_rows, n_heads, hd)
    for i, (s, n) in enumerate(zip(starts, news)):
        qfull = torch.zeros(s + n, n_heads, hd, dtype=torch.float64)
        qfull[s:] = q[row0[i]:row0[i] + n].double()
        ref = pl.attention(qfull, ks[i].double(), vs[i].double(), window)[s:]
        e = rel_err(out[row0[i]:row0[i] + n], ref)
        assert e <= 2 ** -6, f"sequence {i}: {e}"


@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 1, 64), (32, 8, 64), (6, 2, 128), (5, 5, 64), (34, 1, 128), (12, 2, 64)])
def test_attention_mma_rows_of_several_tokens(cuda, n_heads, n_kv, hd):
    _attn_mma_case(cuda, n_heads, n_kv, hd, starts=[0, 0, 0, 64], news=[1, 70, 129, 33], window=None, decode=False,
                   spike=(2, 3))


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("n_splits", [1, 2, 5, 16])
def test_attention_mma_decode_splits(cuda, hd, n_splits):
    _attn_mma_case(cuda, 8, 2, hd, starts=[0, 31, 32, 63, 64, 700], news=[1] * 6, window=None, decode=True,
                   n_splits=n_splits, spike=(5, 130))


@pytest.mark.parametrize("edge", [0, 1], ids=["first key outside", "first key inside"])
@pytest.mark.parametrize("window", [1, 32, 70, 199])
def test_attention_mma_window_edges(cuda, window, edge):
    _attn_mma_case(cuda, 4, 2, 64, starts=[0, 190], news=[150, 10], window=window, decode=False,
                   spike=(1, 199 - window + edge))
    _attn_mma_case(cuda, 4, 2, 64, starts=[199, 80], news=[1, 1], window=window, decode=True, n_splits=3,
                   spike=(0, 199 - window + edge))


# ---- the tcgen05 prefill attention kernel ----

def _attn_tc_case(cuda, n_heads, n_kv, hd, starts, news, window, spike=None):
    from camelid_b200.csrc import ops
    dt = torch.bfloat16
    totals = [s + n for s, n in zip(starts, news)]
    k_pages, v_pages, table, ks, vs = _paged(totals, n_kv, hd, dt, cuda)
    g = torch.Generator().manual_seed(1)
    n_rows = sum(news)
    q = torch.randn(n_rows, n_heads, hd, generator=g).to(dt)
    row0 = [sum(news[:i]) for i in range(len(news))]
    if spike is not None:
        seq, key = spike
        r = row0[seq] + news[seq] - 1
        ks[seq][key] *= 0
        ks[seq][key, :, 0] = 8.0
        q[r, :, 0] = 8.0 * math.sqrt(hd) / 4
        k_pages[int(table[seq, key // 64]), :, key % 64] = ks[seq][key].to(cuda)
    rows, hpc, chunks = ops.attn_tc_tiling(n_heads, n_kv)
    tile_seq, tile_q0 = [], []
    for i, n in enumerate(news):
        for q0 in range(0, n, rows):
            tile_seq.append(i)
            tile_q0.append(q0)
    out = torch.full((n_rows, n_heads * hd), float("nan"), dtype=dt, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    ops.attn_prefill_tc(q.view(n_rows, -1).to(cuda), out, k_pages, v_pages, table, _i32(tile_seq, cuda),
                        _i32(tile_q0, cuda), len(tile_seq), _i32(row0, cuda), _i32(starts, cuda), _i32(news, cuda),
                        n_heads, n_kv, hd, rows, hpc, chunks, window or 0, 1 / math.sqrt(hd), err)
    assert int(err) == 0
    out = out.cpu().view(n_rows, n_heads, hd)
    for i, (s, n) in enumerate(zip(starts, news)):
        qfull = torch.zeros(s + n, n_heads, hd, dtype=torch.float64)
        qfull[s:] = q[row0[i]:row0[i] + n].double()
        ref = pl.attention(qfull, ks[i].double(), vs[i].double(), window)[s:]
        e = rel_err(out[row0[i]:row0[i] + n], ref)
        assert e <= 2 ** -6, f"sequence {i}: {e}"


@pytest.mark.parametrize("n_heads,n_kv,hd", [(4, 1, 64), (32, 8, 64), (6, 2, 128), (5, 5, 64), (34, 1, 128), (12, 2, 64)])
def test_attention_tc_prefill_shapes(cuda, n_heads, n_kv, hd):
    _attn_tc_case(cuda, n_heads, n_kv, hd, starts=[0, 0, 0, 64], news=[1, 70, 300, 33], spike=(2, 3), window=None)


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_tc_continues_from_cache(cuda, hd):
    _attn_tc_case(cuda, 8, 2, hd, starts=[64, 300, 5, 0], news=[3, 200, 64, 129], spike=(1, 7), window=None)


@pytest.mark.parametrize("edge", [0, 1], ids=["first key outside", "first key inside"])
@pytest.mark.parametrize("window", [1, 32, 70, 199])
def test_attention_tc_window_edges(cuda, window, edge):
    _attn_tc_case(cuda, 4, 2, 64, starts=[0, 190], news=[150, 10], window=window, spike=(1, 199 - window + edge))


def _attn_fused_case(cuda, n_heads, n_kv, hd, rot, starts, window, n_splits, gsplits, write_kv=True, spike=None,
                     n_pages=64):
    """Decode attention in one launch from the partial sums of the q/k/v product: against the
    plain rotary encoding and attention of the whole sequences, and the cache rows it writes."""
    from camelid_b200.csrc import ops
    from camelid_b200.parts.position import rotary_frequencies
    dt = torch.bfloat16
    n = len(starts)
    totals = [s + 1 for s in starts]
    k_pages, v_pages, table, ks, vs = _paged(totals, n_kv, hd, dt, cuda, n_pages=n_pages, seed=4)
    freqs = rotary_frequencies(rot, 10000.0, None) if rot else np.zeros(0, dtype=np.float32)
    g = torch.Generator().manual_seed(7)
    width = (n_heads + 2 * n_kv) * hd
    part = torch.randn(gsplits, n, width, generator=g) / math.sqrt(gsplits)
    pos = torch.tensor(starts)
    if spike is not None:
        # One cached key gets a score that stands out for every head of its sequence: the key is
        # 8 in its last dimension and nothing else, and the query is made so that, after the
        # kernel's rotation at its position, it is large in that dimension (the query before
        # the rotation is the wanted one turned back). A kernel that drops that key, or counts
        # it when the window excludes it, is off by far more than the tolerance.
        seq, key = spike
        ks[seq][key] *= 0
        ks[seq][key, :, hd - 1] = 8.0
        k_pages[int(table[seq, key // 64]), :, key % 64] = ks[seq][key].to(cuda)
        want_q = torch.randn(1, n_heads, hd, generator=g, dtype=torch.float64)
        want_q[..., hd - 1] = 8.0 * math.sqrt(hd) / 4
        before = pl.rope(want_q, -pos[seq:seq + 1], freqs) if rot else want_q
        rest = part[1:, seq, :n_heads * hd].sum(0) if gsplits > 1 else 0.0
        part[0, seq, :n_heads * hd] = before.reshape(-1).float() - rest
    total = torch.zeros(n, width)
    for s in range(gsplits):
        total = total + part[s]                       # the kernel's order of adding
    qkv = total.to(dt)
    q = qkv[:, :n_heads * hd].double().view(n, n_heads, hd)
    k = qkv[:, n_heads * hd:(n_heads + n_kv) * hd].double().view(n, n_kv, hd)
    v = qkv[:, (n_heads + n_kv) * hd:].view(n, n_kv, hd)
    q_rot = (pl.rope(q, pos, freqs) if rot else q).to(dt)
    k_rot = (pl.rope(k, pos, freqs) if rot else k).to(dt)
    tab = table.cpu()
    slots = [(int(tab[i, s // 64]), s % 64) for i, s in enumerate(starts)]
    if write_kv:                                      # the row's own place holds something else until the kernel writes it
        for page, off in slots:
            k_pages[page, :, off] = float("nan")
            v_pages[page, :, off] = float("nan")
    else:                                             # a borrowed cache already holds the row's key and value
        for i, (page, off) in enumerate(slots):
            k_pages[page, :, off] = k_rot[i].to(cuda)
            v_pages[page, :, off] = v[i].to(cuda)
    before_k = k_pages.clone()
    out = torch.full((n, n_heads * hd), float("nan"), dtype=dt, device=cuda)
    ops.attn_decode_fused(part.to(cuda), out, _i32(starts, cuda), _i32(list(range(n)), cuda), table, k_pages, v_pages,
                          torch.from_numpy(freqs).to(cuda), rot, n_heads, n_kv, hd, write_kv, window or 0,
                          1 / math.sqrt(hd), n_splits)
    out = out.cpu().view(n, n_heads, hd)
    for i, s in enumerate(starts):
        page, off = slots[i]
        if write_kv:
            assert rel_err(k_pages[page, :, off].cpu(), k_rot[i].double()) <= 2 ** -8
            assert torch.equal(v_pages[page, :, off].cpu(), v[i])
        kfull = torch.cat([ks[i][:s].double(), k_rot[i].double()[None]], dim=0)
        vfull = torch.cat([vs[i][:s].double(), v[i].double()[None]], dim=0)
        qfull = torch.zeros(s + 1, n_heads, hd, dtype=torch.float64)
        qfull[s] = q_rot[i].double()
        ref = pl.attention(qfull, kfull, vfull, window)[s:]
        e = rel_err(out[i:i + 1], ref)
        assert e <= 2 ** -6, f"sequence {i} at position {s}: {e}"
    changed = (before_k != k_pages) & ~(torch.isnan(before_k) & torch.isnan(k_pages))
    assert int(changed.any(dim=-1).sum()) <= (n * n_kv if write_kv else 0)     # nothing else was written


@pytest.mark.parametrize("n_splits", [1, 2, 5, 8])
@pytest.mark.parametrize("n_heads,n_kv,hd,rot", [(8, 2, 64, 64), (6, 2, 128, 64), (5, 5, 64, 32), (16, 1, 64, 0)])
def test_attention_decode_fused(cuda, n_heads, n_kv, hd, rot, n_splits):
    _attn_fused_case(cuda, n_heads, n_kv, hd, rot, starts=[0, 31, 32, 63, 64, 700], window=None, n_splits=n_splits,
                     gsplits=3, spike=(5, 130))


@pytest.mark.parametrize("edge", ["first key inside", "first key outside"])
@pytest.mark.parametrize("window", [1, 32, 70, 199])
def test_attention_decode_fused_window_and_borrowed_cache(cuda, window, edge):
    """The query at position 199 with a window of w sees keys 200 - w .. 199: the outstanding key
    sits once on the first key inside the window (it must count) and once on the first key
    outside (it must not)."""
    key = 200 - window if edge == "first key inside" else 199 - window
    if key == 199:              # a window of 1 sees only the new key, which the kernel makes itself
        key = None
    _attn_fused_case(cuda, 4, 2, 64, 64, starts=[199, 80, 0], window=window, n_splits=3, gsplits=9,
                     spike=None if key is None else (0, key))
    _attn_fused_case(cuda, 4, 2, 64, 64, starts=[199, 80, 0], window=window, n_splits=4, gsplits=1, write_kv=False,
                     spike=None if key is None else (0, key))
    _attn_fused_case(cuda, 8, 2, 128, 128, starts=[300, 5], window=None, n_splits=2, gsplits=2, write_kv=False)


@pytest.mark.parametrize("n_splits,key", [(1, 2100), (1, 8999), (3, 130), (3, 5003), (8, 2100), (8, 8999)])
def test_attention_decode_fused_long_context(cuda, n_splits, key):
    """Thousands of cached keys: a warp walks more tiles than the 32 page numbers it keeps in
    registers, and one outstanding key, near the start, past a warp's first 32 pages, in the
    middle or at the very end of the range, must be found."""
    _attn_fused_case(cuda, 8, 2, 64, 64, starts=[9000, 4100, 64], window=None, n_splits=n_splits, gsplits=2,
                     spike=(0, key), n_pages=256)
