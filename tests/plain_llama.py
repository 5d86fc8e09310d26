"""Plain, slow implementation of the dense Llama decoder, used only as a test oracle.

It rests on the formulas of karan68/Camelid (a Rust project that cannot be compiled
here: no Rust toolchain), each function citing the file and lines it was written
from. It runs whole sequences without a cache, has one function for each part, and
shares no code with the ``camelid_b200`` package: it reads ``config.json`` as a plain
dict and ``model.safetensors`` with a reader of its own.

Everything is computed in ``dtype`` (float32 as in the reference, or float64 as a tighter
ground truth), on the CPU unless ``forward`` is given a device: the wide shapes of the
benchmark take minutes in float64 on a CPU, so tests of those run these same plain torch
operations on the GPU. Weights are taken as stored (bfloat16 values are exactly
representable in both types).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

# --------------------------------------------------------------------------------------
# files


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


_ST_DTYPES = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
              "I32": (torch.int32, 4), "I64": (torch.int64, 8)}


def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, payload; offsets are relative to
    the payload (src/model_source.rs:818-896)."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    payload = memoryview(raw)[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt, _size = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        if e == b:
            out[name] = torch.empty(info["shape"], dtype=dt)
            continue
        t = torch.frombuffer(bytearray(payload[b:e]), dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def read_model(folder: str) -> tuple[dict, dict[str, torch.Tensor]]:
    return read_config(folder), read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------------------
# configuration helpers (plain dict; defaults as the reference has them)


def head_dim_of(cfg: dict) -> int:
    """head_dim = key_length or hidden / heads (src/model.rs:1405-1456)."""
    hd = cfg.get("head_dim")
    return int(hd) if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


def kv_heads_of(cfg: dict) -> int:
    """kv heads default to the number of heads (src/model.rs:698-705)."""
    return int(cfg.get("num_key_value_heads") or cfg["num_attention_heads"])


# --------------------------------------------------------------------------------------
# parts


def embedding(ids: torch.Tensor, table: torch.Tensor, dtype) -> torch.Tensor:
    """h[t, :] = E[id_t, :], a row gather without scaling; an id beyond the vocabulary is
    an error (src/tensor/mod.rs:2253-2283, error at :2266-2270)."""
    if int(ids.max()) >= table.shape[0] or int(ids.min()) < 0:
        raise ValueError("token id outside the vocabulary")
    return table.to(ids.device, dtype)[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """mean_square = sum(v*v)/cols; scale = 1/sqrt(mean_square + eps);
    out = x * scale * weight, in that order (src/tensor/mod.rs:2086-2096)."""
    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(mean_square + eps)
    return x * scale * weight.to(x.device, x.dtype)


def rope_frequencies(cfg: dict) -> np.ndarray:
    """Per-pair frequency in float32: f_i = theta^(-2i/rope_dim)
    (src/inference/rope.rs:526-537), then the llama3 law when rope_scaling asks for it
    (src/inference/rope.rs:687-711; defaults low 1, high 4, original 8192 at :413-422)."""
    rope_dim = head_dim_of(cfg)
    theta = np.float32(cfg.get("rope_theta", 10000.0))
    out = np.zeros(rope_dim // 2, dtype=np.float32)
    scaling = cfg.get("rope_scaling") or None
    for i in range(rope_dim // 2):
        exponent = np.float32(-(np.float32(i) * np.float32(2.0)) / np.float32(rope_dim))
        f = np.float32(np.power(theta, exponent, dtype=np.float32))
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind == "llama3":
                factor = np.float32(scaling["factor"])
                low = np.float32(scaling.get("low_freq_factor", 1.0))
                high = np.float32(scaling.get("high_freq_factor", 4.0))
                original = np.float32(scaling.get("original_max_position_embeddings", 8192))
                wavelength = np.float32(np.float32(2.0) * np.float32(math.pi)) / f
                low_wavelength = original / low
                high_wavelength = original / high
                if wavelength < high_wavelength:
                    pass
                elif wavelength > low_wavelength:
                    f = np.float32(f / factor)
                else:
                    smooth = np.float32((original / wavelength - low) / (high - low))
                    f = np.float32((np.float32(1.0) - smooth) * f / factor + smooth * f)
            elif kind in (None, "default"):
                pass
            else:
                raise ValueError(f"rope scaling {kind!r} is not part of this architecture")
        out[i] = f
    return out


def rope(x: torch.Tensor, positions: torch.Tensor, freqs: np.ndarray) -> torch.Tensor:
    """x: [T, heads, head_dim]. angle = position (as f32, 0-based) * f_i in float32;
    split-half pairing (i, i + rope_dim/2) for un-permuted weights:
    x0' = x0 cos - x1 sin, x1' = x0 sin + x1 cos
    (src/inference/rope.rs:489-524, pairing at :501-509)."""
    half = freqs.shape[0]
    f = torch.from_numpy(freqs).to(x.device)
    angle = positions.to(torch.float32)[:, None] * f[None, :]        # float32 product
    cos = torch.cos(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    sin = torch.sin(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    x0 = x[..., :half]
    x1 = x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:2 * half] = x0 * sin + x1 * cos
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """q: [T, nH, hd]; k, v: [T, nKV, hd] (the same sequence, causal).
    For query head h the kv head is h // (nH / nKV); the query at position p sees keys
    0..p; score = (q . k) * 1/sqrt(hd) (dot first, then scale); m = max; e = exp(s - m);
    out = sum_j (e_j * (1/Z)) * v_j (src/inference.rs:23945-24025; mapping and scale
    src/inference/diagnostic_config.rs:300-317; causal rows src/inference.rs:23668-23705).
    ``window`` (keys p-window+1..p) is not part of Llama; toy layers in tests use it."""
    T, nH, hd = q.shape
    nKV = k.shape[1]
    group = nH // nKV
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for h in range(nH):
        kvh = h // group
        scores = (q[:, h, :] @ k[:, kvh, :].T) * scale              # [T, T]
        idx = torch.arange(T, device=q.device)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] <= idx[:, None] - window)
        scores = scores.masked_fill(mask, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        z = e.sum(dim=-1, keepdim=True)
        out[:, h, :] = (e * (1.0 / z)) @ v[:, kvh, :]
    return out


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """g = x Wg^T, u = x Wu^T, act = (g / (1 + exp(-g))) * u, d = act Wd^T
    (src/inference.rs:9657-9664, :6654-6706)."""
    g = x @ w_gate.to(x.device, x.dtype).T
    u = x @ w_up.to(x.device, x.dtype).T
    act = (g / (1.0 + torch.exp(-g))) * u
    return act @ w_down.to(x.device, x.dtype).T


class _On:
    """``w[name]`` on a device."""

    def __init__(self, w, device):
        self.w, self.device = w, device

    def __getitem__(self, name):
        return self.w[name].to(self.device)


def attention_block(x: torch.Tensor, w: dict, prefix: str, cfg: dict, positions: torch.Tensor,
                    freqs: np.ndarray, kv_override=None):
    """q, k, v projections without bias (src/inference.rs:6301-6336), RoPE on q and k
    before the keys are kept (src/inference.rs:23244-23281), attention, output
    projection (src/inference.rs:6487-6522). Returns the projected output and (k, v)."""
    T = x.shape[0]
    nH, nKV, hd = cfg["num_attention_heads"], kv_heads_of(cfg), head_dim_of(cfg)
    dt = x.dtype
    w = _On(w, x.device)
    q = (x @ w[prefix + "self_attn.q_proj.weight"].to(dt).T).reshape(T, nH, hd)
    q = rope(q, positions, freqs)
    if kv_override is None:
        k = (x @ w[prefix + "self_attn.k_proj.weight"].to(dt).T).reshape(T, nKV, hd)
        v = (x @ w[prefix + "self_attn.v_proj.weight"].to(dt).T).reshape(T, nKV, hd)
        k = rope(k, positions, freqs)
    else:
        k, v = kv_override
    o = attention(q, k, v).reshape(T, nH * hd)
    return o @ w[prefix + "self_attn.o_proj.weight"].to(dt).T, (k, v)


def decoder_layer(h: torch.Tensor, w: dict, layer: int, cfg: dict, positions: torch.Tensor,
                  freqs: np.ndarray, kv_override=None):
    """r = x + attn(norm(x)); out = r + ffn(norm(r))
    (order of operations: src/inference.rs:6228-6804; residuals :6487-6522, :6654-6706;
    post-attention norm :6539-6544)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    n = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    a, kv = attention_block(n, w, p, cfg, positions, freqs, kv_override)
    r = h + a
    n2 = rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    d = swiglu(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return r + d, kv


def output_weight(cfg: dict, w: dict) -> torch.Tensor:
    """lm_head.weight if present, else the embedding (tied output)
    (src/model.rs:772-775; src/model_source.rs:244-261)."""
    if "lm_head.weight" in w:
        return w["lm_head.weight"]
    if not cfg.get("tie_word_embeddings", False):
        raise ValueError("no lm_head.weight and the embeddings are not tied")
    return w["model.embed_tokens.weight"]


def forward(cfg: dict, w: dict, ids, dtype=torch.float32, schedule=None, rows=None, device="cpu") -> torch.Tensor:
    """Logits [T, V] of one whole sequence: embedding, the layers in order, final norm
    (src/inference.rs:4259-4264), output projection without bias or scaling
    (src/inference.rs:4284-4290). ``rows``: only these positions' logits (the output projection
    of a large vocabulary is most of the work), in the order given.

    ``schedule`` is the order in which layers run, as a list of (layer, source) pairs:
    ``source`` None means the entry makes its own keys and values, an integer means it
    reads those made by that earlier entry of the list. The default is every layer once."""
    ids = torch.as_tensor(ids, dtype=torch.int64).to(device)
    T = ids.shape[0]
    positions = torch.arange(T, device=device)
    freqs = rope_frequencies(cfg)
    h = embedding(ids, w["model.embed_tokens.weight"], dtype)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kept = []
    for layer, source in schedule:
        override = kept[source] if source is not None else None
        h, kv = decoder_layer(h, w, layer, cfg, positions, freqs, override)
        kept.append(kv)
    n = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    if rows is not None:
        n = n[torch.as_tensor(list(rows), dtype=torch.int64).to(device)]
    return (n @ output_weight(cfg, w).to(n.device, dtype).T).cpu()


# --------------------------------------------------------------------------------------
# sampling

_MASK64 = (1 << 64) - 1


def splitmix64(state: int) -> int:
    """SplitMix64 finalizer (src/inference.rs:6160-6166)."""
    z = state & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def unit_draw(seed: int, position: int) -> np.float32:
    """state = seed + (position + 1) * 0x9E3779B97F4A7C15 (wrapping); the draw is the top
    24 bits of splitmix64(state) / 2^24 (src/inference.rs:6168-6180)."""
    state = (seed + ((position + 1) * 0x9E3779B97F4A7C15 & _MASK64)) & _MASK64
    return np.float32((splitmix64(state) >> 40) / float(1 << 24))


def greedy(logits: np.ndarray) -> int:
    """Strict '>', so the first of equal maxima wins; non-finite logits are an error
    (src/inference.rs:5890-5925)."""
    if not np.all(np.isfinite(logits)):
        raise ValueError("non-finite logits")
    best, best_value = 0, -np.inf
    for i, v in enumerate(logits.tolist()):
        if v > best_value:
            best, best_value = i, v
    return best


def adjust_logits(logits: np.ndarray, history, *, logit_bias=(), repeat_penalty=1.0,
                  presence_penalty=0.0, frequency_penalty=0.0) -> np.ndarray:
    """Bias first; then for every token of the history: repeat penalty (divide a positive
    logit, multiply a negative one), presence penalty, frequency penalty times its count
    (src/inference.rs:6093-6157)."""
    out = logits.astype(np.float32).copy()
    for tok, bias in logit_bias:
        if tok >= out.shape[0]:
            raise ValueError("logit_bias token outside the vocabulary")
        out[tok] = np.float32(out[tok] + np.float32(bias))
    if presence_penalty != 0.0 or frequency_penalty != 0.0 or repeat_penalty != 1.0:
        counts: dict[int, int] = {}
        for t in history:
            if t < out.shape[0]:
                counts[t] = counts.get(t, 0) + 1
        for t, c in counts.items():
            v = out[t]
            if repeat_penalty != 1.0:
                v = np.float32(v / np.float32(repeat_penalty)) if v > 0 else np.float32(v * np.float32(repeat_penalty))
            if presence_penalty != 0.0:
                v = np.float32(v - np.float32(presence_penalty))
            if frequency_penalty != 0.0:
                v = np.float32(v - np.float32(frequency_penalty) * np.float32(c))
            out[t] = v
    return out


def sample(logits: np.ndarray, history, *, temperature=0.0, top_k=None, top_p=None, min_p=None,
           seed=0, **adjust) -> int:
    """The reference's sampler (src/inference.rs:5991-6091): adjustments, then greedy if
    temperature is 0; else candidates sorted by logit descending (ties by index), top_k
    truncation, softmax of logit/T - max in float32, min_p filter (p >= min_p * p_max,
    renormalised), top_p prefix (cumulative >= top_p, at least one, renormalised), and
    a walk of the cumulative sum in that order until draw < cumulative, the draw being
    keyed by the seed and the length of the history."""
    adjusted = adjust_logits(logits, history, **adjust)
    if not np.all(np.isfinite(adjusted)):
        raise ValueError("non-finite logits")
    if temperature == 0.0:
        return greedy(adjusted)
    T = np.float32(temperature)
    # the reference orders by total_cmp (src/inference.rs:6004-6006): +0.0 stands before -0.0, then the index
    order = sorted(range(adjusted.shape[0]), key=lambda i: (-float(adjusted[i]), bool(np.signbit(adjusted[i])), i))
    if top_k is not None:
        order = order[:min(top_k, len(order))]
    scaled = np.array([np.float32(adjusted[i] / T) for i in order], dtype=np.float32)
    mx = scaled.max()
    weights = np.exp(scaled - mx, dtype=np.float32)
    total = np.float32(0.0)
    for x in weights:
        total = np.float32(total + x)
    probs = [np.float32(x / total) for x in weights]
    cand = list(zip(order, probs))
    if min_p is not None and min_p > 0.0:
        pmax = max(p for _, p in cand)
        thr = np.float32(np.float32(min_p) * pmax)
        cand = [(i, p) for i, p in cand if p >= thr]
        s = np.float32(0.0)
        for _, p in cand:
            s = np.float32(s + p)
        cand = [(i, np.float32(p / s)) for i, p in cand]
    if top_p is not None and top_p < 1.0:
        cand.sort(key=lambda ip: (-float(ip[1]), ip[0]))
        cum, keep = np.float32(0.0), 0
        for _, p in cand:
            cum = np.float32(cum + p)
            keep += 1
            if cum >= np.float32(top_p):
                break
        cand = cand[:max(keep, 1)]
        s = np.float32(0.0)
        for _, p in cand:
            s = np.float32(s + p)
        cand = [(i, np.float32(p / s)) for i, p in cand]
    draw = unit_draw(seed or 0, len(history))
    cum = np.float32(0.0)
    for i, p in cand:
        cum = np.float32(cum + p)
        if draw < cum:
            return i
    return cand[-1][0]


# --------------------------------------------------------------------------------------
# random weights (the library's generator restated one element at a time)


def _fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & _MASK64
    return h


def random_weight(seed: int, name: str, index: int, kind: str = "linear") -> np.float32:
    """Element ``index`` (row-major) of the random tensor ``name``: Box-Muller on the two halves
    of splitmix64(key + (index + 1) * golden), key = splitmix64(fnv1a64(name) ^ splitmix64(seed)),
    with the logarithm and cosine as written-out polynomials in correctly rounded double
    operations; N(0, 0.02), norm weights 1 + N(0, 0.02). Ours: the reference's only random
    weights are an LCG in its tests (src/cuda_resident/tests.rs:537-553)."""
    key = splitmix64(_fnv1a64(name.encode("utf-8")) ^ splitmix64(seed))
    z = splitmix64(key + (index + 1) * 0x9E3779B97F4A7C15)
    n = float((z >> 32) + 1)
    b = z & 0xFFFFFFFF
    mant, ex = math.frexp(n)
    if mant < 0.7071067811865476:
        mant, ex = mant * 2.0, ex - 1
    s = (mant - 1.0) / (mant + 1.0)
    w = s * s
    p = 1.0 / 21.0
    for k in range(9, -1, -1):
        p = p * w + 1.0 / (2 * k + 1)
    ln_u = float(ex - 32) * 0.6931471805599453 + (2.0 * s) * p
    r = math.sqrt(-2.0 * ln_u)
    octant = b >> 29
    f = float(b & 0x1FFFFFFF) * (1.0 / 536870912.0)
    t = ((1.0 - f) if octant & 1 else f) * 0.7853981633974483
    w = t * t
    if octant in (1, 2, 5, 6):
        p = 1.0 / math.factorial(17)
        for k in range(7, -1, -1):
            p = p * w + (-1.0) ** k / math.factorial(2 * k + 1)
        trig = t * p
    else:
        p = 1.0 / math.factorial(16)
        for k in range(7, -1, -1):
            p = p * w + (-1.0) ** k / math.factorial(2 * k)
        trig = p
    if octant in (2, 3, 4, 5):
        trig = -trig
    return np.float32((1.0 if kind == "norm" else 0.0) + 0.02 * (r * trig))


# --------------------------------------------------------------------------------------
# generation


def generate(cfg: dict, w: dict, prompts, max_tokens: int, *, stop_ids=(), dtype=torch.float32,
             schedule=None, **sampling):
    """The reference's loop, one sequence at a time (src/main.rs:3706-3917): run the
    prompt, sample, append, feed the new token; the stop token is kept and ends the
    sequence (src/main.rs:3731-3733, :3877-3879); the history given to the sampler is
    the prompt plus everything generated so far. Every step here re-runs the whole
    sequence: no cache."""
    outs = []
    for prompt in prompts:
        history = list(prompt)
        gen = []
        while len(gen) < max_tokens:
            logits = forward(cfg, w, history, dtype=dtype, schedule=schedule)[-1].to(torch.float32).numpy()
            tok = sample(logits, history, **sampling)
            gen.append(tok)
            history.append(tok)
            if tok in stop_ids:
                break
        outs.append(gen)
    return outs
