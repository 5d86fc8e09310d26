"""Each part alone (built from its PartSpec through the registry, with weights of its own)
against the plain function of the same mathematics."""
import math

import pytest
import torch

import plain_llama as pl
from helpers import rel_err

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ctx(cache, dtype, slots, starts, token_lists, want=None, tile_sizes=(1,)):
    from camelid_b200.engine.context import StepContext, Workspace
    return StepContext.for_step(cache=cache, workspace=Workspace("cuda"), dtype=DT[dtype], device="cuda", slots=slots,
                                starts=starts, tokens=token_lists, want=want or [[] for _ in slots],
                                tile_sizes=tile_sizes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(cuda, dtype):
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": 88, "eps": 1e-3}, "n."))
    assert list(norm.tensor_specs()) == ["n.weight"] and norm.tensor_specs()["n.weight"].shape == (88,)
    w = 1 + 0.1 * torch.randn(88)
    norm.load({"n.weight": w}, "cuda", DT[dtype])
    assert norm.weight.dtype == torch.float32            # stored in 32-bit: stays so
    norm.load({"n.weight": w.to(torch.bfloat16)}, "cuda", DT[dtype])
    assert norm.weight.dtype == DT[dtype]
    h = torch.randn(5, 88, device="cuda") * 2
    ctx = _ctx(None, dtype, [0], [0], [[1, 2, 3, 4, 5]])
    out = norm.forward(ctx, h)
    ref = pl.rms_norm(h.cpu().double(), norm.weight.cpu().double(), 1e-3)
    assert out.dtype == DT[dtype] and rel_err(out.cpu(), ref) <= (1e-5 if dtype == "float32" else 2 ** -8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,inter", [(40, 48), (72, 136)])
def test_swiglu_part(cuda, dtype, hidden, inter):
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    from camelid_b200.weights import random_tensors
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": inter}, "f."))
    w = {n: t * 10 for n, t in random_tensors(ffn.tensor_specs(), 0, DT[dtype]).items()}
    ffn.load(w, "cuda", DT[dtype])
    x = torch.randn(7, hidden).to(DT[dtype]).cuda()
    res = torch.randn(7, hidden, device="cuda")
    want = res.cpu().double() + pl.swiglu(x.cpu().double(), w["f.gate_proj.weight"], w["f.up_proj.weight"], w["f.down_proj.weight"])
    ctx = _ctx(None, dtype, [0], [0], [[0] * 7])
    ffn.forward(ctx, x, res)
    ctx.settle(res)                  # a built-in part may leave split sums for the next norm to add
    assert rel_err(res.cpu(), want) <= (1e-5 if dtype == "float32" else 2 ** -7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(cuda, dtype):
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": 99, "hidden_size": 24}, "e."))
    head = build_part("head", PartSpec("lm_head", {"vocab_size": 99, "hidden_size": 24, "tied_to": "e."}, "h."))
    assert head.tensor_specs() == {}
    table = torch.randn(99, 24).to(DT[dtype])
    emb.load({"e.weight": table}, "cuda", DT[dtype])
    head.load({}, "cuda", DT[dtype], tied_weight=emb.weight)
    assert head.weight is emb.weight
    toks = torch.tensor([5, 98, 0], dtype=torch.int32, device="cuda")
    out = torch.empty(3, 24, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    emb.forward(None, toks, out, err)
    assert torch.equal(out.cpu(), table.float()[[5, 98, 0]])
    x = torch.randn(3, 24).to(DT[dtype]).cuda()
    logits = torch.empty(3, 99, device="cuda")
    head.forward(None, x, logits)
    assert rel_err(logits.cpu(), x.cpu().double() @ table.double().T) <= 1e-5
    untied = build_part("head", PartSpec("lm_head", {"vocab_size": 99, "hidden_size": 24, "tied_to": None}, "h."))
    assert untied.tensor_specs()["h.weight"].shape == (99, 24)


def test_rotary_part_frequencies(cuda):
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    sc = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    rope = build_part("position", PartSpec("rope", {"rotary_dim": 64, "theta": 500000.0, "scaling": sc}))
    rope.load({}, "cuda", torch.float32)
    ref = pl.rope_frequencies({"head_dim": 64, "hidden_size": 64, "num_attention_heads": 1, "rope_theta": 500000.0,
                               "rope_scaling": sc})
    assert torch.equal(rope.inv_freq.cpu(), torch.from_numpy(ref))
    none = build_part("position", PartSpec("none"))
    none.load({}, "cuda", torch.float32)
    assert none.rotary_dim == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,hd,rot", [(4, 2, 16, 16), (6, 3, 32, 16), (2, 2, 48, 0)])
def test_attention_part(cuda, dtype, heads, kv_heads, hd, rot):
    """The mixer alone with a cache of its own: a prompt in one step, then three single
    tokens, for two sequences of unequal length; partial rotary dimensions and none."""
    from camelid_b200.cache.sequence_cache import SequenceCache
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    from camelid_b200.weights import random_tensors
    hidden = 40
    pos = PartSpec("rope", {"rotary_dim": rot, "theta": 10000.0, "scaling": None}) if rot else PartSpec("none")
    mixer = build_part("mixer", PartSpec("attention", {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads,
                                                        "head_dim": hd, "position": pos, "window": None}, "a."))
    w = {n: t * 8 for n, t in random_tensors(mixer.tensor_specs(), 0, DT[dtype]).items()}
    mixer.load(w, "cuda", DT[dtype])
    cache = SequenceCache([mixer.cache_spec()], [None], max_tokens=512, max_position=512, dtype=DT[dtype], device="cuda")
    lens = [70, 9]
    xs = [torch.randn(n, hidden).to(DT[dtype]) for n in lens]

    def plain(x):
        T = x.shape[0]
        x = x.double()
        p = torch.arange(T)
        fr = pl.rope_frequencies({"head_dim": rot, "hidden_size": rot, "num_attention_heads": 1}) if rot else None
        q = (x @ w["a.q_proj.weight"].double().T).view(T, heads, hd)
        k = (x @ w["a.k_proj.weight"].double().T).view(T, kv_heads, hd)
        v = (x @ w["a.v_proj.weight"].double().T).view(T, kv_heads, hd)
        if rot:
            q, k = pl.rope(q, p, fr), pl.rope(k, p, fr)
        return pl.attention(q, k, v).reshape(T, -1) @ w["a.o_proj.weight"].double().T

    refs = [plain(x) for x in xs]
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    got = [[], []]
    done = [0, 0]
    for step, news in enumerate([[l - 3 for l in lens], [1, 1], [1, 1], [1, 1]]):
        for s, n in zip(slots, news):
            cache.book.extend(s, n)
        ctx = _ctx(cache, dtype, slots, list(done), [[0] * n for n in news], tile_sizes=mixer.query_tile_sizes())
        ctx.entry = 0
        x = torch.cat([xs[i][done[i]:done[i] + n] for i, n in enumerate(news)]).cuda()
        res = torch.zeros(sum(news), hidden, device="cuda")
        mixer.forward(ctx, x, res)
        ctx.settle(res)
        off = 0
        for i, n in enumerate(news):
            got[i].append(res[off:off + n].cpu())
            off += n
            cache.book.commit(slots[i], n)
            done[i] += n
    for i in range(2):
        e = rel_err(torch.cat(got[i]), refs[i])
        assert e <= (1e-5 if dtype == "float32" else 2 ** -6), f"sequence {i}: {e}"


@pytest.mark.skipif(False, reason="")
def test_unknown_part_is_a_clear_error():
    from camelid_b200 import ConfigError
    from camelid_b200.config import PartSpec
    from camelid_b200.parts import build_part
    with pytest.raises(ConfigError) as e:
        build_part("mixer", PartSpec("mamba"))
    assert "attention" in str(e.value)
    with pytest.raises(ConfigError):
        build_part("mixer", PartSpec("attention", {"hidden_size": 8, "num_heads": 2, "num_kv_heads": 1, "head_dim": 24}))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [3, 70, 128, 129, 300, 600])
def test_linear_every_epilogue_at_every_step_size(cuda, dtype, rows):
    """``parts.linear.linear`` as a part from outside the library may call it: store, float store
    and add into a float stream, whatever form the product takes for the step's rows; and the
    split sums of ``partial_sums`` where it gives some."""
    from camelid_b200.parts import linear
    g = torch.Generator().manual_seed(rows)
    k, n = 264, 200
    x = torch.randn(rows, k, generator=g).to(DT[dtype]).cuda()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(DT[dtype]).cuda()
    ref = x.cpu().double() @ w.cpu().double().T
    ctx = _ctx(None, dtype, [0], [0], [[0] * rows])
    tol = 1e-5 if dtype == "float32" else 2 ** -7
    out = torch.full((rows, n), float("nan"), dtype=DT[dtype], device="cuda")
    linear.linear(ctx, x, w, out, linear.STORE)
    assert rel_err(out.cpu(), ref) <= tol
    out32 = torch.full((rows, n), float("nan"), device="cuda")
    linear.linear(ctx, x, w, out32, linear.STORE_F32)
    assert rel_err(out32.cpu(), ref) <= 1e-5
    res = torch.randn(rows, n, generator=g).cuda()
    want = res.cpu().double() + ref
    linear.linear(ctx, x, w, res, linear.ADD_F32)
    assert rel_err(res.cpu(), want) <= 1e-5
    part = linear.partial_sums(ctx, x, w, "test_partial")
    if part is not None:
        assert part.dtype == torch.float32 and part.shape[1:] == (rows, n)
        assert rel_err(part.sum(0).cpu(), ref) <= 1e-5
    linear.check_errors()
