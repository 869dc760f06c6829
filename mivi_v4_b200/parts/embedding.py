"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.needs import StateNeed
from ..ops import kernels as K
from ..ops.linear import linear, norm_link_ok
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("embedding", "table")
class Embedding(Part):
    """x_t = E[token_t], no scaling (crates/mivi-model/src/model.rs:355-366)."""

    emits_norm = True            # forward(step, emit=link) can write the norm that follows it

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def forward(self, step, emit=None) -> torch.Tensor:
        """``emit``: the first layer's first norm as a link (steps of few tokens); its rows and sums
        are then written here and that norm is no kernel of its own."""
        x = step.ws.get("resid", (step.n_tokens, self.hidden), torch.float32)
        return K.embed(self.weight, step.tokens, x, emit)


@register("embedding", "table_scaled_positions")
class ScaledEmbeddingWithPositions(Part):
    """x_t = E[token_t] * scale + P[position_t]: a scaled token embedding plus a learned position vector
    (``positions`` False: no position table; ``max_positions`` None: as many rows as the checkpoint has).  With ``hand_rounded`` the rows are also written in the model's
    dtype and handed to the first block through ``step.handed`` as ("stream", rows): a block whose first
    sublayer reads the stream itself then needs no rounding pass."""

    def __init__(self, vocab: int, hidden: int, scale: float = 1.0, max_positions: Optional[int] = None,
                 hand_rounded: bool = False, positions: bool = True):
        self.vocab, self.hidden, self.scale = int(vocab), int(hidden), float(scale)
        self.max_positions = None if max_positions is None else int(max_positions)
        self.hand_rounded, self.has_positions = bool(hand_rounded), bool(positions)

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {"weight": ParamSpec((self.vocab, self.hidden))}
        if self.has_positions:
            specs["positions"] = ParamSpec((self.max_positions, self.hidden))
        return specs

    def load(self, t) -> None:
        self.weight, self.positions = t["weight"], t.get("positions")
        if self.positions is not None and self.positions.dtype != self.weight.dtype:
            self.weight, self.positions = self.weight.float(), self.positions.float()

    def forward(self, step) -> torch.Tensor:
        N = step.n_tokens
        x = step.ws.get("resid", (N, self.hidden), torch.float32)
        rounded = None
        if self.hand_rounded and step.dtype != torch.float32:
            rounded = step.ws.get("stream_rounded", (N, self.hidden), step.dtype)
        if self.positions is not None and step.max_context > self.positions.shape[0]:
            raise K.KernelError(f"a sequence reaches position {step.max_context - 1}; the position table has "
                                f"{self.positions.shape[0]} rows")
        K.embed_scaled_pos(self.weight, step.tokens, self.scale, self.positions, step.positions, x, rounded)
        step.handed = ("stream", rounded) if rounded is not None else None
        return x


@register("embedding", "table_bigram")
class BigramEmbedding(Part):
    """x_t = E[token_t] + B[r_t]: a token embedding plus a row of a hashed bigram table,
    r_t = (token_(t-1) * mul_prev + token_t * mul_cur) mod buckets, and row ``buckets`` (the table's last) for a
    sequence's first token.  The previous token is part of a sequence's state: one int32 per slot.  With ``keep``
    a second copy of the rows is left in ``step.embedding_output`` for parts that add it to the stream again later."""

    def __init__(self, vocab: int, hidden: int, buckets: int, mul_prev: int, mul_cur: int, keep: bool = False):
        if buckets < 1:
            raise ValueError(f"a bigram table needs at least one bucket, got {buckets}")
        self.vocab, self.hidden, self.buckets = int(vocab), int(hidden), int(buckets)
        self.mul_prev, self.mul_cur, self.keep = int(mul_prev), int(mul_cur), bool(keep)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden)), "bigram": ParamSpec((self.buckets + 1, self.hidden))}

    def load(self, t) -> None:
        self.weight, self.bigram = t["weight"], t["bigram"]
        if self.bigram.dtype != self.weight.dtype:
            self.weight, self.bigram = self.weight.float(), self.bigram.float()

    def cache_need(self):
        return StateNeed((1,), torch.int32)

    def forward(self, step, view) -> torch.Tensor:
        N = step.n_tokens
        x = step.ws.get("resid", (N, self.hidden), torch.float32)
        kept = step.ws.get("embedding_output", (N, self.hidden), torch.float32) if self.keep else None
        K.embed_bigram(self.weight, self.bigram, step.tokens, step.positions, step.seq_of, step.cu, step.slots,
                       view.state.view(-1), x, kept, self.mul_prev, self.mul_cur)
        step.embedding_output = kept
        return x


@register("head", "linear")
class LMHead(Part):
    """logits = f W^T in float32; W is the embedding table when ``tied``
    (crates/mivi-model/src/model.rs:455-473).  ``softcap`` c > 0: logits <- c tanh(logits / c)."""

    def __init__(self, vocab: int, hidden: int, tied: bool, softcap: float = 0.0):
        self.vocab, self.hidden, self.tied, self.softcap = int(vocab), int(hidden), bool(tied), float(softcap or 0.0)

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def carries_norm(self, step, embedding) -> bool:
        """Whether the product can apply the final norm's scale itself (steps of few rows)."""
        w = embedding.weight if self.tied else self.weight
        return norm_link_ok(step.n_out, w, step.dtype)

    def forward(self, f, step, embedding, scale=None) -> torch.Tensor:
        w = embedding.weight if self.tied else self.weight
        logits = step.ws.get("logits", (f.shape[0], self.vocab), torch.float32)
        linear(f, w, logits, scale=scale)
        return K.softcap_(logits, self.softcap) if self.softcap > 0 else logits
