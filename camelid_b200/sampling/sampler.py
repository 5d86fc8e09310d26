"""The sampler on the device: one call per step for the whole batch.

Greedy is an argmax kernel. Otherwise the logits are adjusted in place (bias, repeat,
presence and frequency penalties over each request's history, prompt included, as
src/main.rs:3714-3733 passes it) and the sampling kernel picks a token per row with the
draw of that row's stream position. Only token ids and an error word come back to the host.
This class is the step-by-step form (the histories' token counts are made on the host every
step); the steps that feed themselves on the device keep those counts on the device
(``engine/graphs.py``).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import SamplingError
from .options import SamplingOptions, unit_draw


class Sampler:
    def __init__(self, options: SamplingOptions, vocab_size: int, device):
        self.options = options.validate(vocab_size)
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self._err = torch.zeros(1, dtype=torch.int32, device=self.device)

    @property
    def native_ok(self) -> bool:
        """Whether the C++ decode loop that samples between graph launches can serve this sampler:
        everything but the adjustments (penalties, bias), which it does not know."""
        return not self.options.adjusts

    @property
    def fed_ok(self) -> bool:
        """Whether steps that pick their own token on the device can serve this sampler: all of
        them; adjustments ride along as token counts kept on the device."""
        return True

    @property
    def error_word(self) -> torch.Tensor:
        return self._err

    def _adjust_entries(self, histories: list):
        o = self.options
        entries, biases = [], []
        penalise = o.presence_penalty != 0.0 or o.frequency_penalty != 0.0 or o.repeat_penalty != 1.0
        for row, hist in enumerate(histories):
            counts: dict = {}
            if penalise:
                for t in hist:
                    if 0 <= t < self.vocab_size:
                        counts[t] = counts.get(t, 0) + 1
            bias: dict = {}
            for tok, b in o.logit_bias:
                bias[tok] = bias.get(tok, 0.0) + b
            for tok in set(counts) | set(bias):
                entries.append((row, tok, counts.get(tok, 0)))
                biases.append(bias.get(tok, 0.0))
        return entries, biases

    def sample(self, logits: torch.Tensor, histories: list) -> torch.Tensor:
        """``logits``: float32 [rows, vocab] on the device (adjusted in place when penalties or
        biases are set); ``histories``: per row the tokens so far, prompt included. Returns
        int32 [rows] on the device."""
        rows = logits.shape[0]
        o = self.options
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if o.adjusts:
            entries, biases = self._adjust_entries(histories)
            if entries:
                e = torch.tensor(entries, dtype=torch.int32).to(self.device, non_blocking=True)
                b = torch.tensor(biases, dtype=torch.float32).to(self.device, non_blocking=True)
                ops.adjust_logits(logits, e, b, o.repeat_penalty, o.presence_penalty, o.frequency_penalty)
        if o.greedy:
            ops.argmax_rows(logits, out, self._err)
        else:
            seed = o.seed or 0
            draws = torch.tensor([unit_draw(seed, len(h)) for h in histories], dtype=torch.float32)
            draws = draws.to(self.device, non_blocking=True)
            ops.sample_rows(logits, o.temperature, o.top_k or 0, o.top_p if o.top_p is not None else 1.0,
                            o.min_p or 0.0, draws, out, self._err)
        return out

    def check(self) -> None:
        """Synchronising read of the error word: non-finite logits are an error
        (src/inference.rs:5890-5907)."""
        code = int(self._err.item())
        if code:
            self._err.zero_()
            raise SamplingError("sampler logits contain a non-finite value" if code & 1
                                else "sampler softmax produced an invalid normalisation sum")
