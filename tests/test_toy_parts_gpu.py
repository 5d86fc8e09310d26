"""Generality of the parts, shown with toy parts that exist only here: a mixer with state of
its own (no keys and values), registered, built and stepped without a change to the
library's files; a schedule that names layers twice and lets an entry read another entry's
cache; a layer with a window next to layers without one (two cache groups); a feed-forward
that routes every row to one of several experts; a position encoding with a frequency law of
its own, used by the library's attention."""
import dataclasses

import pytest
import torch

import plain_llama as pl
from conftest import TINY_A
from helpers import assert_close, tokens

pytestmark = pytest.mark.gpu


def _register_toys():
    from camelid_b200.cache import StateSpec
    from camelid_b200.config import LlamaConfig, ScheduleEntry, llama_plan, register_architecture
    from camelid_b200.config.plan import LayerSpec, PartSpec
    from camelid_b200.parts import Part, TensorSpec, build_part, register_part

    @register_part("mixer", "toy_running_sum")
    class RunningSum(Part):
        """y_t = (sum of x_0..x_t) * w: the sum so far is the state, one vector per sequence."""

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.hidden = params["hidden_size"]

        def tensor_specs(self):
            return {self.prefix + "w": TensorSpec((self.hidden,), "norm")}

        def load(self, tensors, device, dtype):
            self.w = tensors[self.prefix + "w"].to(device=device, dtype=torch.float32)

        def cache_spec(self):
            return StateSpec((self.hidden,), "float32")

        def forward(self, ctx, x, residual):
            state = ctx.state()                                   # [slots, hidden]
            for slot, r0, n in zip(ctx.h_slots, ctx.h_row0, ctx.h_new):
                sums = torch.cumsum(x[r0:r0 + n].float(), 0) + state[slot]
                residual[r0:r0 + n] += sums * self.w
                state[slot] = sums[-1]

    @register_part("mixer", "toy_device_sum")
    class DeviceRunningSum(Part):
        """The running sum again, but written for a captured graph: a one-token step finds its
        sequences' state through ``ctx.seq_slot`` on the device and reads nothing on the host.
        It also reads the residual stream (its output is sum * w + 0.1 * residual) and knows
        nothing of what the library's own parts may have left pending on the context."""
        graph_safe = True

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.hidden = params["hidden_size"]

        def tensor_specs(self):
            return {self.prefix + "w": TensorSpec((self.hidden,), "norm")}

        def load(self, tensors, device, dtype):
            self.w = tensors[self.prefix + "w"].to(device=device, dtype=torch.float32)

        def cache_spec(self):
            return StateSpec((self.hidden,), "float32")

        def forward(self, ctx, x, residual):
            state = ctx.state()
            if ctx.decode:                                        # device arrays only
                slots = ctx.seq_slot.long()
                sums = state.index_select(0, slots) + x.float()
                state.index_copy_(0, slots, sums)
                residual.add_(sums * self.w + 0.1 * residual)
                return
            for slot, r0, n in zip(ctx.h_slots, ctx.h_row0, ctx.h_new):
                sums = torch.cumsum(x[r0:r0 + n].float(), 0) + state[slot]
                residual[r0:r0 + n] += sums * self.w + 0.1 * residual[r0:r0 + n]
                state[slot] = sums[-1]

    def device_sum_plan(cfg):
        base = llama_plan(cfg)
        layers = list(base.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("toy_device_sum", {"hidden_size": cfg.hidden_size},
                                                                  "model.layers.1.toy."))
        return dataclasses.replace(base, layers=tuple(layers))

    def toy_plan(cfg):
        base = llama_plan(cfg)
        layers = list(base.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("toy_running_sum", {"hidden_size": cfg.hidden_size},
                                                                  "model.layers.1.toy."))
        return dataclasses.replace(base, layers=tuple(layers))

    def twice_plan(cfg):
        base = llama_plan(cfg)
        return dataclasses.replace(base, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                                                   ScheduleEntry(1, cache_source=1)))

    def window_plan(cfg):
        base = llama_plan(cfg)
        layers = list(base.layers)
        mixer = layers[1].mixer
        layers[1] = dataclasses.replace(layers[1], mixer=PartSpec(mixer.kind, {**mixer.params, "window": 70}, mixer.prefix))
        return dataclasses.replace(base, layers=tuple(layers))

    @register_part("ffn", "toy_top1_experts")
    class Top1Experts(Part):
        """Router logits in float32; every row goes to its best expert e and gets
        softmax(logits)[e] * (x W_e^T). Plain torch on the device: not graph safe."""

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.hidden, self.experts = params["hidden_size"], params["experts"]

        def tensor_specs(self):
            return {self.prefix + "router": TensorSpec((self.experts, self.hidden)),
                    self.prefix + "experts": TensorSpec((self.experts * self.hidden, self.hidden))}

        def load(self, tensors, device, dtype):
            self.router = tensors[self.prefix + "router"].to(device=device, dtype=torch.float32)
            self.w = tensors[self.prefix + "experts"].to(device=device, dtype=torch.float32).view(self.experts, self.hidden, self.hidden)

        def forward(self, ctx, x, residual):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.T, dim=-1)
            best = prob.argmax(dim=-1)
            for e in range(self.experts):
                rows = (best == e).nonzero().flatten()
                if rows.numel():
                    residual[rows] += prob[rows, e, None] * (xf[rows] @ self.w[e].T)

    @register_part("position", "toy_harmonic")
    class HarmonicRotary(Part):
        """A rotary encoding whose frequency i is 1 / (i + 2): the attention kernels rotate by
        whatever frequencies the position part hands them."""
        graph_safe = True

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.rotary_dim = int(params["rotary_dim"])
            self.inv_freq = None

        def load(self, tensors, device, dtype):
            self.inv_freq = (1.0 / (torch.arange(self.rotary_dim // 2, dtype=torch.float32) + 2.0)).to(device)

    @register_part("norm", "toy_layernorm")
    class ToyLayerNorm(Part):
        """(x - mean) / sqrt(var + eps) * w: a norm from outside that knows nothing of pending sums
        or of rows' scales (plain torch, so the model steps eagerly)."""

        def __init__(self, params, prefix=""):
            super().__init__(params, prefix)
            self.hidden, self.eps = params["hidden_size"], params["eps"]

        def tensor_specs(self):
            return {self.prefix + "weight": TensorSpec((self.hidden,), "norm")}

        def load(self, tensors, device, dtype):
            self.w = tensors[self.prefix + "weight"].to(device=device, dtype=torch.float32)

        def forward(self, ctx, h, rows_index=None, n_rows=None, name="normed", allow_row_scale=False):
            x = h if rows_index is None else h[rows_index.long()[:n_rows]]
            y = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + self.eps) * self.w
            return y.to(ctx.dtype)

    @register_part("block", "toy_parallel")
    class ParallelBlock(Part):
        """out = x + mixer(norm(x)) + ffn(norm(x)): both branches read the same normed rows."""

        def __init__(self, layer_spec):
            super().__init__({}, "")
            self.norm = build_part("norm", layer_spec.norm1)
            self.mixer = build_part("mixer", layer_spec.mixer)
            self.ffn = build_part("ffn", layer_spec.ffn)

        def tensor_specs(self):
            return {**self.norm.tensor_specs(), **self.mixer.tensor_specs(), **self.ffn.tensor_specs()}

        def load(self, tensors, device, dtype):
            for part in (self.norm, self.mixer, self.ffn):
                part.load(tensors, device, dtype)

        @property
        def graph_safe(self):
            return self.norm.graph_safe and self.mixer.graph_safe and self.ffn.graph_safe

        def cache_spec(self):
            return self.mixer.cache_spec()

        def query_tile_sizes(self):
            return self.mixer.query_tile_sizes()

        def forward(self, ctx, h):
            ctx.settle(h)                       # what the layer before left pending
            x = self.norm.forward(ctx, h).clone()          # the norm's buffer is reused by the next norm
            self.mixer.forward(ctx, x, h)
            ctx.settle(h)
            self.ffn.forward(ctx, x, h)

    def layernorm_parallel_plan(cfg):
        base = llama_plan(cfg)
        layers = list(base.layers)
        ln = PartSpec("toy_layernorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.layers.1.input_layernorm.")
        layers[1] = dataclasses.replace(layers[1], arrangement="toy_parallel", norm1=ln)
        final = PartSpec("toy_layernorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm.")
        return dataclasses.replace(base, layers=tuple(layers), final_norm=final)

    def routed_plan(cfg):
        base = llama_plan(cfg)
        layers = list(base.layers)
        layers[0] = dataclasses.replace(layers[0], ffn=PartSpec("toy_top1_experts", {"hidden_size": cfg.hidden_size, "experts": 3},
                                                                "model.layers.0.moe."))
        return dataclasses.replace(base, layers=tuple(layers))

    def harmonic_plan(cfg):
        base = llama_plan(cfg)
        layers = []
        for layer in base.layers:
            m = layer.mixer
            pos = PartSpec("toy_harmonic", {"rotary_dim": cfg.head_dim // 2})          # half of every head rotates
            layers.append(dataclasses.replace(layer, mixer=PartSpec(m.kind, {**m.params, "position": pos}, m.prefix)))
        return dataclasses.replace(base, layers=tuple(layers))

    register_architecture("ToyRoutedForCausalLM", LlamaConfig.from_dict, routed_plan)
    register_architecture("ToyParallelForCausalLM", LlamaConfig.from_dict, layernorm_parallel_plan)
    register_architecture("ToyHarmonicForCausalLM", LlamaConfig.from_dict, harmonic_plan)
    register_architecture("ToyStateForCausalLM", LlamaConfig.from_dict, toy_plan)
    register_architecture("ToyDeviceSumForCausalLM", LlamaConfig.from_dict, device_sum_plan)
    register_architecture("ToyTwiceForCausalLM", LlamaConfig.from_dict, twice_plan)
    register_architecture("ToyWindowForCausalLM", LlamaConfig.from_dict, window_plan)


def _model(arch, dtype, seed=3, **over):
    from camelid_b200.engine.model import DecoderModel
    from camelid_b200.weights import random_tensors
    cfg = {**TINY_A, "architectures": [arch], "max_position_embeddings": 512, **over}
    model = DecoderModel.from_config(cfg, dtype=dtype, device="cuda")
    tensors = random_tensors(model.tensor_specs(), seed)
    model.load_tensors(tensors)
    return cfg, model, tensors


def _drive(model, seqs, cut):
    """Two requests in one batch: prompts of ``cut`` tokens, then token by token until the
    shorter one ends; then a third request in the freed slot."""
    from camelid_b200 import StepEntry
    cache = model.new_cache(1024, max_slots=2)
    outs = [[], [], []]
    a, b = cache.alloc_slot(), cache.alloc_slot()
    lg = model.step(cache, [StepEntry(a, seqs[0][:cut[0]], list(range(cut[0]))),
                            StepEntry(b, seqs[1][:cut[1]], list(range(cut[1])))]).cpu()
    outs[0].append(lg[:cut[0]])
    outs[1].append(lg[cut[0]:])
    pos = list(cut)
    while pos[0] < len(seqs[0]) or pos[1] < len(seqs[1]):
        entries, who = [], []
        for i, slot in ((0, a), (1, b)):
            if pos[i] < len(seqs[i]):
                entries.append(StepEntry(slot, [seqs[i][pos[i]]], [0]))
                who.append(i)
            elif slot is not None and cache.book.slots.is_held(slot):
                cache.free_slot(slot)
        lg = model.step(cache, entries).cpu()
        for r, i in enumerate(who):
            outs[i].append(lg[r:r + 1])
            pos[i] += 1
    for slot in (a, b):
        if cache.book.slots.is_held(slot):
            cache.free_slot(slot)
    c = cache.alloc_slot()
    assert c == 0
    outs[2].append(model.step(cache, [StepEntry(c, seqs[2], list(range(len(seqs[2]))))]).cpu())
    cache.free_slot(c)
    cache.book.audit()
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state(cuda, dtype):
    _register_toys()
    cfg, model, w = _model("ToyStateForCausalLM", dtype)
    assert "model.layers.1.toy.w" in w and "model.layers.1.self_attn.q_proj.weight" not in w
    from camelid_b200.cache import KVSpec, StateSpec
    specs = model.entry_cache_specs()
    assert isinstance(specs[0], KVSpec) and isinstance(specs[1], StateSpec)

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        fr = pl.rope_frequencies(cfg)
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        h, _ = pl.decoder_layer(h, w, 0, cfg, pos, fr)
        p = "model.layers.1."
        n = pl.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        if dtype == "bfloat16":
            n = n.to(torch.bfloat16).double()          # the toy reads the normed rows in the compute type
        r = h + torch.cumsum(n, 0) * w[p + "toy.w"].double()
        n2 = pl.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        r = r + pl.swiglu(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return pl.rms_norm(r, w["model.norm.weight"], cfg["rms_norm_eps"]) @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(1, 40, 256), tokens(2, 23, 256), tokens(3, 30, 256)]
    got = _drive(model, seqs, cut=[17, 20])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"toy state, request {i}")      # request 2: a used slot starts from zero


WIDE = {"hidden_size": 256, "head_dim": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 256}


@pytest.mark.parametrize("over", [{}, WIDE], ids=["head16", "head64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_layers_twice_and_shares_a_cache(cuda, dtype, over):
    """head64 in bfloat16 decodes with the kernel that goes from the q/k/v product to the
    attention output in one launch; the entry that borrows a cache must not write it."""
    _register_toys()
    cfg, model, w = _model("ToyTwiceForCausalLM", dtype, **over)
    cache = model.new_cache(256)
    assert cache.k[0].shape[0] == 3 and cache.entry_kv[3] == cache.entry_kv[1]      # four runs, three caches
    seqs = [tokens(4, 70, 256), tokens(5, 33, 256), tokens(6, 66, 256)]
    got = _drive(model, seqs, cut=[64, 3])
    sched = [(0, None), (1, None), (0, None), (1, 1)]
    for i in range(3):
        assert_close(got[i], pl.forward(cfg, w, seqs[i], dtype=torch.float64, schedule=sched), dtype, f"request {i}")


@pytest.mark.parametrize("over", [{}, WIDE], ids=["head16", "head64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_layer_has_storage_of_its_own(cuda, dtype, over):
    """head64 in bfloat16: the tcgen05 prefill kernel (prompts of 200 and 140 rows also take the
    two-block products with the norms inside them) and the fused decode kernel, both with a
    window whose older pages have been given back."""
    _register_toys()
    cfg, model, w = _model("ToyWindowForCausalLM", dtype, **over)
    cache = model.new_cache(1024, max_slots=2)
    assert len(cache.k) == 2 and cache.book.kv_specs[1].window == 70

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        fr = pl.rope_frequencies(cfg)
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        h, _ = pl.decoder_layer(h, w, 0, cfg, pos, fr)
        p = "model.layers.1."
        n = pl.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        T, nH, nKV, hd = len(ids), cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        q = pl.rope((n @ w[p + "self_attn.q_proj.weight"].double().T).view(T, nH, hd), pos, fr)
        k = pl.rope((n @ w[p + "self_attn.k_proj.weight"].double().T).view(T, nKV, hd), pos, fr)
        v = (n @ w[p + "self_attn.v_proj.weight"].double().T).view(T, nKV, hd)
        r = h + pl.attention(q, k, v, window=70).reshape(T, -1) @ w[p + "self_attn.o_proj.weight"].double().T
        n2 = pl.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        r = r + pl.swiglu(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return pl.rms_norm(r, w["model.norm.weight"], cfg["rms_norm_eps"]) @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(7, 300, 256), tokens(8, 150, 256), tokens(9, 200, 256)]
    got = _drive(model, seqs, cut=[200, 140])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"window, request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_that_routes(cuda, dtype):
    _register_toys()
    cfg, model, w = _model("ToyRoutedForCausalLM", dtype, seed=5)
    assert "model.layers.0.moe.router" in w and "model.layers.0.mlp.gate_proj.weight" not in w

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        fr = pl.rope_frequencies(cfg)
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        p = "model.layers.0."
        h = h + pl.attention_block(pl.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"]), w, p, cfg, pos, fr)[0]
        n = pl.rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        if dtype == "bfloat16":
            n = n.to(torch.bfloat16).double()          # the toy reads the normed rows in the compute type
        prob = torch.softmax(n @ w[p + "moe.router"].double().T, dim=-1)
        best = prob.argmax(dim=-1)
        experts = w[p + "moe.experts"].double().view(3, cfg["hidden_size"], cfg["hidden_size"])
        h = h + torch.stack([prob[t, best[t]] * (experts[best[t]] @ n[t]) for t in range(len(ids))])
        h, _ = pl.decoder_layer(h, w, 1, cfg, pos, fr)
        return pl.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]) @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(7, 40, 256), tokens(8, 23, 256), tokens(9, 30, 256)]
    got = _drive(model, seqs, cut=[17, 20])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"routed feed-forward, request {i}")


@pytest.mark.parametrize("over", [{}, WIDE], ids=["head16", "head64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_encoding_of_its_own(cuda, dtype, over):
    _register_toys()
    cfg, model, w = _model("ToyHarmonicForCausalLM", dtype, seed=6, **over)
    rot = cfg["head_dim"] // 2
    fr = (1.0 / (torch.arange(rot // 2, dtype=torch.float32) + 2.0)).numpy()

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        for layer in range(cfg["num_hidden_layers"]):
            h, _ = pl.decoder_layer(h, w, layer, cfg, pos, fr)
        return pl.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]) @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(10, 70, 256), tokens(11, 33, 256), tokens(12, 66, 256)]
    got = _drive(model, seqs, cut=[64, 3])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"harmonic rotary, request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_safe_mixer_from_outside_finds_its_state_by_slot(cuda, dtype):
    """A mixer from outside the library that is safe to capture, keeps state per sequence, reads
    the residual stream and ignores the context's pending sums: stepped by hand (graph path for
    the single tokens), and through the generation loop with two batches of equal size that sit
    in different slots, so that the captured graph and the C++ decode loop must pick up each
    batch's own slots."""
    from camelid_b200 import StepEntry
    from camelid_b200.engine.generate import generate
    from camelid_b200.sampling.options import SamplingOptions
    from camelid_b200.sampling.sampler import Sampler
    _register_toys()
    cfg, model, w = _model("ToyDeviceSumForCausalLM", dtype)
    assert model.use_graphs

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        fr = pl.rope_frequencies(cfg)
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        h, _ = pl.decoder_layer(h, w, 0, cfg, pos, fr)
        p = "model.layers.1."
        n = pl.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        if dtype == "bfloat16":
            n = n.to(torch.bfloat16).double()
        r = h + torch.cumsum(n, 0) * w[p + "toy.w"].double() + 0.1 * h
        n2 = pl.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        r = r + pl.swiglu(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return pl.rms_norm(r, w["model.norm.weight"], cfg["rms_norm_eps"]) @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(21, 40, 256), tokens(22, 23, 256), tokens(23, 30, 256)]
    got = _drive(model, seqs, cut=[17, 20])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"device running sum, request {i}")

    # through the loop: the same two prompts first in slots 0 and 1, then, with slot 0 held by
    # someone else, in slots 1 and 2; teacher-forced against the plain implementation
    cache = model.new_cache(1024, max_slots=4)
    sampler = Sampler(SamplingOptions(), model.vocab_size, model.device)
    prompts = [tokens(31, 9, 256), tokens(32, 14, 256)]
    first = [r.tokens for r in generate(model, cache, sampler, prompts, 12)]
    held = cache.alloc_slot()
    assert held == 0
    again = [r.tokens for r in generate(model, cache, sampler, prompts, 12)]
    cache.free_slot(held)
    assert first == again, "the same prompts gave other tokens in other slots"
    for prompt, gen in zip(prompts, first):
        ref = plain(prompt + gen[:-1])
        scale = float(ref.abs().max())
        for i, tok in enumerate(gen):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) <= (1e-4 if dtype == "float32" else 3e-2) * scale, (i, tok)


@pytest.mark.parametrize("over", [{}, WIDE], ids=["head16", "head64"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_and_block_arrangement_of_their_own(cuda, dtype, over):
    """A norm (mean-subtracting) and a block arrangement (attention and feed-forward in parallel on
    the same normed rows) registered from outside, the norm also as the model's final norm: layer 0
    is the library's own block and leaves its split sums pending, which the outside block and norm
    never hear of."""
    _register_toys()
    cfg, model, w = _model("ToyParallelForCausalLM", dtype, seed=8, **over)
    assert "model.layers.1.post_attention_layernorm.weight" not in w      # the arrangement decides which parts exist

    def layernorm(x, weight):
        return (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + cfg["rms_norm_eps"]) * weight.double()

    def plain(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        fr = pl.rope_frequencies(cfg)
        h = pl.embedding(ids, w["model.embed_tokens.weight"], torch.float64)
        h, _ = pl.decoder_layer(h, w, 0, cfg, pos, fr)
        p = "model.layers.1."
        n = layernorm(h, w[p + "input_layernorm.weight"])
        if dtype == "bfloat16":
            n = n.to(torch.bfloat16).double()
        a, _kv = pl.attention_block(n, w, p, cfg, pos, fr)
        f = pl.swiglu(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        h = h + a + f
        n = layernorm(h, w["model.norm.weight"])
        if dtype == "bfloat16":
            n = n.to(torch.bfloat16).double()
        return n @ pl.output_weight(cfg, w).double().T

    seqs = [tokens(13, 70, 256), tokens(14, 33, 256), tokens(15, 66, 256)]
    got = _drive(model, seqs, cut=[64, 3])
    for i in range(3):
        assert_close(got[i], plain(seqs[i]), dtype, f"layer norm and parallel block, request {i}")
