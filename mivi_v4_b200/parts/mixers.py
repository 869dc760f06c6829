"""Mixers: the parts of a layer that move information between tokens."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache.needs import KVNeed, StateNeed
from ..ops import kernels as K
from ..ops.kernels import profile_stage
from ..ops.linear import (conv_rows_grouped, heads_fused_ok, linear, linear_heads, linear_shortconv_decode, norm_link_ok,
                          shortconv_decode_fused_ok)
from .base import Part
from .position import Rope
from .registry import register
from .spec import ParamSpec


@register("mixer", "short_conv")
class ShortConv(Part):
    """Gated short convolution: in_proj to (B, C, x), B*x, causal depthwise
    convolution of width ``kernel``, C*, out_proj
    (crates/mivi-model/src/ssm.rs:51-155).  Its state per sequence is the last
    kernel-1 values of B*x.  With ``bias`` the three linear maps carry one
    (the checkpoint format's conv_bias; the reference has none)."""

    def __init__(self, hidden: int, kernel: int, bias: bool = False):
        if not 1 <= kernel <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {kernel} is outside 1..{K.MAX_CONV_K}")
        self.hidden, self.kernel, self.bias = int(hidden), int(kernel), bool(bias)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, k = self.hidden, self.kernel
        specs = {"in_proj.weight": ParamSpec((3 * H, H)),
                 "conv.weight": ParamSpec((H, 1, k), "vector", "conv"),
                 "out_proj.weight": ParamSpec((H, H))}
        if self.bias:
            specs.update({"in_proj.bias": ParamSpec((3 * H,), "vector", "bias"),
                          "conv.bias": ParamSpec((H,), "vector", "bias"),
                          "out_proj.bias": ParamSpec((H,), "vector", "bias")})
        return specs

    def load(self, t) -> None:
        self.w_in, self.w_out = t["in_proj.weight"], t["out_proj.weight"]
        self.w_in_grouped = None
        self.taps = t["conv.weight"].reshape(self.hidden, self.kernel).contiguous()
        self.b_in, self.b_conv, self.b_out = t.get("in_proj.bias"), t.get("conv.bias"), t.get("out_proj.bias")

    def cache_need(self):
        return StateNeed((self.kernel - 1, self.hidden))

    def carries_norm(self, step):
        n = step.n_tokens
        return norm_link_ok(n, self.w_in, step.dtype), norm_link_ok(n, self.w_out, step.dtype, emits=True)

    def forward(self, u, resid, step, view, scale=None, emit=None) -> None:
        N, H = u.shape
        z = self.scratch(step, "mix", (N, H), step.dtype)
        if step.is_decode and N == step.n_seqs and shortconv_decode_fused_ok(N, u, self.w_in):
            # a few sequences, one token each: the convolution is the projection's epilogue (from 9 sequences
            # on over a copy of the projection whose rows are regrouped, made when first wanted)
            w_in, grouped = self.w_in, conv_rows_grouped(N, self.w_in)
            if grouped:
                if self.w_in_grouped is None:
                    self.w_in_grouped = K.group_conv_rows(self.w_in)
                w_in = self.w_in_grouped
            linear_shortconv_decode(u, w_in, self.b_in, self.taps, self.b_conv, view.state, step.slots, z,
                                    scale=scale, grouped=grouped)
            linear(z, self.w_out, resid, bias=self.b_out, accumulate=True, emit=emit)
            return
        p = self.scratch(step, "proj", (N, 3 * H), torch.float32)
        linear(u, self.w_in, p, bias=self.b_in, scale=scale)
        K.shortconv(p, self.taps, self.b_conv, view.state, step.positions, step.seq_of, step.cu,
                    step.slots, step.starts, step.lens, z, step.n_seqs, decode=step.is_decode)
        linear(z, self.w_out, resid, bias=self.b_out, accumulate=True, emit=emit)


@register("mixer", "gqa")
class GroupedQueryAttention(Part):
    """Grouped-query attention over the cache: q, k, v projections, per-head
    RMSNorm of q and k (``qk_norm_eps`` None: none), the position part's
    rotation, append to the cache, causal softmax attention with scale
    1/sqrt(head_dim) and an optional window, out projection
    (crates/mivi-model/src/transformer.rs:55-110, 114-167, 304-350).
    ``shared_kv``: the layer has no k and v of its own and reads the cache of
    another layer (its schedule entry says which)."""

    nested_roles = {"position": "position"}

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, position,
                 qk_norm_eps: Optional[float] = None, window: int = 0, shared_kv: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if head_dim % 8 or head_dim > K.MAX_HEAD_DIM:
            raise ValueError(f"head size {head_dim} must be a multiple of 8 and at most {K.MAX_HEAD_DIM}")
        self.hidden, self.nh, self.nkv, self.hd = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.position = position
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.window, self.shared_kv = int(window), bool(shared_kv)
        # a position part may put a constant factor on the scores
        self.scale = 1.0 / math.sqrt(self.hd) * float(getattr(position, "score_scale", lambda: 1.0)())

    def nested(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh, nkv, hd = self.hidden, self.nh, self.nkv, self.hd
        specs = {"q_proj.weight": ParamSpec((nh * hd, H))}
        if not self.shared_kv:
            specs["k_proj.weight"] = ParamSpec((nkv * hd, H))
            specs["v_proj.weight"] = ParamSpec((nkv * hd, H))
        specs["out_proj.weight"] = ParamSpec((H, nh * hd))
        if self.qk_norm_eps is not None:
            specs["q_layernorm.weight"] = ParamSpec((hd,), "vector", "norm")
            if not self.shared_kv:
                specs["k_layernorm.weight"] = ParamSpec((hd,), "vector", "norm")
        return specs

    def load(self, t) -> None:
        if self.shared_kv:
            # the fused projection has the rows of k and v left out; the kernel skips them
            self.w_qkv = t["q_proj.weight"]
        else:
            ws = [t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]]
            if len({w.dtype for w in ws}) != 1:
                ws = [w.float() for w in ws]
            self.w_qkv = torch.cat(ws, dim=0).contiguous()
        self.w_o = t["out_proj.weight"]
        self.q_norm, self.k_norm = t.get("q_layernorm.weight"), t.get("k_layernorm.weight")

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    def carries_norm(self, step):
        n = step.n_tokens
        return norm_link_ok(n, self.w_qkv, step.dtype), norm_link_ok(n, self.w_o, step.dtype, emits=True)

    def forward(self, u, resid, step, view, scale=None, emit=None) -> None:
        N = u.shape[0]
        nh, nkv, hd = self.nh, self.nkv, self.hd
        if view.writable == self.shared_kv:
            raise RuntimeError("a shared_kv attention layer must read another layer's cache, and only it may")
        width = (nh + (0 if self.shared_kv else 2 * nkv)) * hd
        q = self.scratch(step, "q", (N, nh * hd), step.dtype)
        rot = self.position.rotary(u.device)
        inv_freq, half_split = rot if rot is not None else (None, False)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        if not self.shared_kv and heads_fused_ok(N, u, self.w_qkv, hd, view.pool, half_split):
            # a few tokens: norm, rotation and the append to the cache are the projection's epilogue
            linear_heads(u, self.w_qkv, self.q_norm, self.k_norm, eps, inv_freq, half_split, step.positions,
                         step.seq_of, view.page_table, view.pool, q, nh, nkv, scale=scale)
        else:
            qkv = self.scratch(step, "proj", (N, width), torch.float32)
            linear(u, self.w_qkv, qkv, scale=scale)
            if self.shared_kv:
                K.qk_prepare_q_only(qkv, self.q_norm, eps, inv_freq, half_split, step.positions, q, nh, hd)
            else:
                K.qk_prepare(qkv, self.q_norm, self.k_norm, eps, inv_freq, half_split, step.positions,
                             step.seq_of, view.page_table, view.pool, q, nh, nkv, hd)
        o = self.scratch(step, "mix", (N, nh * hd), step.dtype)
        # few query tokens, or many sequences with a token or two each: every query token on its own
        few = N <= K.DECODE_ATTENTION_MAX_TOKENS or step.max_len <= K.DECODE_ATTENTION_MAX_QUERIES
        if few and K.attention_decode_tc_supported(step.dtype, hd, view.pool, self.window, nh, nkv):
            # few query tokens, head size 64: flash decoding with both products on tcgen05
            K.attention_decode_tc(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                                  self.scale, step.ws)
        elif few:
            K.attention_decode(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                               self.scale, self.window, step.ws)
        elif (N >= 128 * step.n_seqs and K.attention_prefill_tc_supported(step.dtype, hd, view.pool, self.window)):
            # long chunks: 256 query rows a block, both products on tcgen05
            K.attention_prefill_tc(q, view.pool, view.page_table, step.cu, step.starts, o, step.n_seqs, nh, nkv,
                                   hd, self.scale)
        elif K.attention_prefill_supported(step.dtype, hd):
            K.attention_prefill(q, view.pool, view.page_table, step.cu, step.starts, o, step.n_seqs, nh, nkv, hd,
                                self.scale, self.window)
        else:
            K.attention_generic(q, view.pool, view.page_table, step.positions, step.seq_of, o, nh, nkv, hd,
                                self.scale, self.window)
        if K.profiling_on():
            # keys that the step's queries read (each query its own context), for the attention launch
            pairs = sum(n * s + n * (n + 1) // 2 for s, n in zip(step.host_starts, step.host_lens))
            rows = pairs if few else sum(s + n for s, n in zip(step.host_starts, step.host_lens))
            K.account(2 * nkv * hd * view.pool.element_size() * rows + 2 * N * nh * hd * q.element_size(),
                      4 * nh * hd * pairs)
        linear(o, self.w_o, resid, accumulate=True, emit=emit)


def _fuse_rows(mats, multiple: int = 16) -> torch.Tensor:
    """Several projections of the same input as one matrix, their rows end to end, padded with zero rows to
    a multiple of ``multiple`` (the padding's results are never read)."""
    if len({m.dtype for m in mats}) != 1:
        mats = [m.float() for m in mats]
    rows = sum(m.shape[0] for m in mats)
    pad = -rows % multiple
    if pad:
        mats = list(mats) + [torch.zeros((pad, mats[0].shape[1]), dtype=mats[0].dtype, device=mats[0].device)]
    return torch.cat(mats, dim=0).contiguous()


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """Linear attention with a matrix state per head and a learned decay per key channel:
    q = W_q h / sqrt(dk), k = W_k h, v = W_v h; a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau);
    S <- diag(a) S + k v^T, o = S^T q; each head's o is divided by its root mean square and multiplied by
    ``norm`` [dv] (one weight for all heads), then by silu(W_g h); W_o maps the heads back.  The state
    [heads, dv, dk] is float32 per sequence and starts at zero; decay, state and sums are float32 in every
    run.  ``rank`` is the inner size of the decay's two-step projection; None takes it from the checkpoint."""

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, tau: float, eps: float,
                 rank: Optional[int] = None):
        if not 1 <= key_dim <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"key size {key_dim} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        if tau <= 0:
            raise ValueError(f"tau must be positive, got {tau}")
        self.hidden, self.nh, self.dk, self.dv = int(hidden), int(n_heads), int(key_dim), int(value_dim)
        self.tau, self.eps, self.rank = float(tau), float(eps), None if rank is None else int(rank)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, qk, vv, r = self.hidden, self.nh * self.dk, self.nh * self.dv, self.rank
        return {"q": ParamSpec((qk, H)), "k": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "g": ParamSpec((vv, H)),
                "o": ParamSpec((H, vv)), "norm": ParamSpec((self.dv,), "vector", "norm"),
                "a1": ParamSpec((r, H)), "a2": ParamSpec((qk, r)), "a2.b": ParamSpec((qk,), "vector", "bias")}

    def load(self, t) -> None:
        if t["a1"].shape[0] != t["a2"].shape[1]:
            raise ValueError(f"the decay's two projections disagree: a1 is {tuple(t['a1'].shape)}, a2 {tuple(t['a2'].shape)}")
        self.w_qkvg = _fuse_rows([t["q"], t["k"], t["v"], t["g"]])
        self.w_a1, self.w_a2, self.b_a2 = t["a1"], t["a2"], t["a2.b"]
        self.w_o, self.norm = t["o"], t["norm"]

    def cache_need(self):
        return StateNeed((self.nh, self.dv, self.dk))

    def forward(self, u, resid, step, view) -> None:
        N = u.shape[0]
        qk, vv = self.nh * self.dk, self.nh * self.dv
        proj = self.scratch(step, "proj", (N, self.w_qkvg.shape[0]), torch.float32)
        linear(u, self.w_qkvg, proj)
        low = self.scratch(step, "low", (N, self.w_a1.shape[0]), step.dtype)
        linear(u, self.w_a1, low)
        z = self.scratch(step, "z", (N, qk), torch.float32)
        linear(low, self.w_a2, z, bias=self.b_a2)
        o = self.scratch(step, "o", (N, vv), torch.float32)
        K.decay_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], view.state, step.slots, step.cu, o,
                     step.n_seqs, self.nh, self.dk, self.dv, decay_logits=z, inv_tau=1.0 / self.tau,
                     q_scale=self.dk ** -0.5, max_len=step.max_len, ws=step.ws)
        y = self.scratch(step, "mix", (N, vv), step.dtype)
        K.gated_rmsnorm(o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.norm, self.dv, self.eps, K.GATE_SILU, y)
        linear(y, self.w_o, resid, accumulate=True)


@register("mixer", "lightning_attention")
class LightningAttention(Part):
    """Linear attention with a matrix state per head and one fixed decay per head:
    q = silu(W_q h), k = silu(W_k h), v = silu(W_v h); S <- decay_h S + k v^T, o = S^T q; the heads together
    are divided by their root mean square and multiplied by ``norm`` [heads * dv], then by sigmoid(W_g h);
    W_o maps them back.  The state [heads, dv, dk] is float32 per sequence and starts at zero."""

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, decay, eps: float):
        decay = [float(d) for d in decay]
        if len(decay) != int(n_heads):
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if not 1 <= key_dim <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"key size {key_dim} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        self.hidden, self.nh, self.dk, self.dv = int(hidden), int(n_heads), int(key_dim), int(value_dim)
        self.decay, self.eps = decay, float(eps)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, qk, vv = self.hidden, self.nh * self.dk, self.nh * self.dv
        return {"q": ParamSpec((qk, H)), "k": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "g": ParamSpec((vv, H)),
                "o": ParamSpec((H, vv)), "norm": ParamSpec((vv,), "vector", "norm")}

    def load(self, t) -> None:
        self.w_qkvg = _fuse_rows([t["q"], t["k"], t["v"], t["g"]])
        self.w_o, self.norm = t["o"], t["norm"]
        # the decays as float32, rounded once from the configuration's numbers
        self.decay_t = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def cache_need(self):
        return StateNeed((self.nh, self.dv, self.dk))

    def forward(self, u, resid, step, view) -> None:
        N = u.shape[0]
        qk, vv = self.nh * self.dk, self.nh * self.dv
        proj = self.scratch(step, "proj", (N, self.w_qkvg.shape[0]), torch.float32)
        linear(u, self.w_qkvg, proj)
        o = self.scratch(step, "o", (N, vv), torch.float32)
        K.decay_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], view.state, step.slots, step.cu, o,
                     step.n_seqs, self.nh, self.dk, self.dv, head_decay=self.decay_t, act=K.SCAN_ACT_SILU,
                     max_len=step.max_len, ws=step.ws)
        y = self.scratch(step, "mix", (N, vv), step.dtype)
        K.gated_rmsnorm(o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.norm, vv, self.eps, K.GATE_SIGMOID, y)
        linear(y, self.w_o, resid, accumulate=True)


@register("mixer", "sink_attention")
class SinkAttention(Part):
    """Grouped-query softmax attention over the cache with keys of size ``key_dim`` and values of size
    ``value_dim``: q, k, v projections without bias; a root-mean-square norm over the WHOLE q and the whole
    k projection (all heads at once; ``qk_norm_eps`` None: none) before the rotation; the position part's
    rotation of the first ``position.head_dim`` elements of every head, element i paired with
    i + position.head_dim / 2; scores (q . k) * scale, capped as c tanh(s / c) when ``softcap`` c > 0; a window
    of ``window`` tokens (0: none) that also keeps the sequence's first ``keep_first`` tokens; with ``sink`` a
    learned number per head whose exponential joins the softmax's denominator; with ``gated`` each head's
    output times sigmoid of one projection of the layer's input per head; then the out projection.  Scores
    and softmax are float32.  ``norm_per_head``: the q and k norms run over every head by itself, with one
    weight [key_dim] shared by the heads.  ``chunk`` c > 0 (instead of a window): token i reads token j <= i
    only if i // c == j // c, chunks counted from the sequence's first position.  A position part with an
    ``amplitude()`` has its cos and sin multiplied by it.

    Further options.  ``talk``: the heads' softmax weights are mixed after the softmax, w'_h(i, j) =
    sum_g T[h, g] w_g(i, j) with the tensor ``talk`` [heads, heads], and head h applies w'_h to the values of its own
    kv head (computed as sum_g T[h, g] O[g, kv(h)] from every head's weights applied to every kv head's values).
    ``conv`` k > 0: q and k pass a causal convolution of k taps per channel (``q.conv``, ``k.conv``, no bias, no
    activation, the last tap the current token's) directly after their projections; the last k - 1 projected rows
    are part of a sequence's state.  ``values_are_keys``: there is no value projection, the values are the first
    ``value_dim`` elements of the keys as they are cached.  ``distance_bias``: r1_h ln(1 + r2_h (i - j)) is taken off
    the scores (``r1``, ``r2`` [heads]).  ``sink`` "zero": the sink's score is 0 for every head and there is no
    tensor (the denominator gains 1).  ``gated`` "element": the gate is one projection of the layer's input per
    element of the concatenated heads.  ``split_weights``: steps of many tokens carry 16 instead of 8 bits of a
    softmax weight's mantissa into the value product."""

    nested_roles = {"position": "position"}
    overwrites = True            # forward(..., accumulate=False) writes its result instead of adding it

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 position, softcap: float = 0.0, window: int = 0, keep_first: int = 0,
                 qk_norm_eps: Optional[float] = None, sink=True, gated=True,
                 norm_per_head: bool = False, chunk: int = 0, talk: bool = False, conv: int = 0,
                 values_are_keys: bool = False, distance_bias: bool = False, split_weights: bool = False):
        if n_kv_heads < 1 or n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if not (1 <= key_dim <= K.MAX_HEAD_DIM and 1 <= value_dim <= K.MAX_HEAD_DIM):
            raise ValueError(f"key size {key_dim} and value size {value_dim} must lie in 1..{K.MAX_HEAD_DIM}")
        self.hidden, self.nh, self.nkv = int(hidden), int(n_heads), int(n_kv_heads)
        self.dk, self.dv, self.scale, self.softcap = int(key_dim), int(value_dim), float(scale), float(softcap or 0.0)
        self.window, self.keep_first = int(window), int(keep_first) if window else 0
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        if sink not in (True, False, "zero") or gated not in (True, False, "element"):
            raise ValueError(f"sink {sink!r} (True, False or 'zero'), gated {gated!r} (True, False or 'element')")
        self.sink, self.gated, self.position = sink, gated, position
        self.norm_per_head, self.chunk = bool(norm_per_head), int(chunk)
        self.talk, self.conv, self.values_are_keys = bool(talk), int(conv), bool(values_are_keys)
        self.distance_bias, self.split_weights = bool(distance_bias), bool(split_weights)
        if self.values_are_keys and self.dv > self.dk:
            raise ValueError(f"values of {self.dv} cannot be the first elements of keys of {self.dk}")
        if not 0 <= self.conv <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {self.conv} is outside 0..{K.MAX_CONV_K}")
        if self.conv and not self.values_are_keys:
            raise ValueError("convolved q and k come with values that are the keys (a value projection beside them is not built)")
        if self.chunk < 0 or (self.chunk and self.window):
            raise ValueError("a chunked mask is a size > 0 and comes instead of a window")
        self.rot_dims = 0
        if isinstance(position, Rope):
            if position.style != "half_split" or position.head_dim > self.dk:
                raise ValueError("the rotation pairs element i with i + dims / 2 over at most the key size")
            self.rot_dims = position.head_dim
        elif position.rotary("cpu") is not None:
            raise ValueError("a rotation that is not a Rope part cannot say how many elements it turns")

    def nested(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh, nkv, dk, dv = self.hidden, self.nh, self.nkv, self.dk, self.dv
        specs = {"q": ParamSpec((nh * dk, H)), "k": ParamSpec((nkv * dk, H))}
        if not self.values_are_keys:
            specs["v"] = ParamSpec((nkv * dv, H))
        specs["o"] = ParamSpec((H, nh * dv))
        if self.qk_norm_eps is not None:
            specs["q.norm"] = ParamSpec((dk if self.norm_per_head else nh * dk,), "vector", "norm")
            specs["k.norm"] = ParamSpec((dk if self.norm_per_head else nkv * dk,), "vector", "norm")
        if self.sink is True:
            specs["sink"] = ParamSpec((nh,), "vector", "bias")
        if self.gated:
            specs["g"] = ParamSpec((nh * dv if self.gated == "element" else nh, H))
        if self.talk:
            specs["talk"] = ParamSpec((nh, nh), "vector", "conv")
        if self.conv:
            specs["q.conv"] = ParamSpec((nh * dk, self.conv), "vector", "conv")
            specs["k.conv"] = ParamSpec((nkv * dk, self.conv), "vector", "conv")
        if self.distance_bias:
            specs["r1"] = ParamSpec((nh,), "vector", "norm")
            specs["r2"] = ParamSpec((nh,), "vector", "norm")
        return specs

    def load(self, t) -> None:
        self.w_qkvg = _fuse_rows([t["q"], t["k"]] + ([] if self.values_are_keys else [t["v"]]) + ([t["g"]] if self.gated else []))
        self.w_o = t["o"]
        self.q_norm, self.k_norm, self.sinks = t.get("q.norm"), t.get("k.norm"), t.get("sink")
        if self.sink == "zero":
            self.sinks = torch.zeros(self.nh, dtype=torch.float32, device=self.w_o.device)
        self.w_talk = t["talk"].float().contiguous() if self.talk else None
        self.taps = torch.cat([t["q.conv"], t["k.conv"]], dim=0).contiguous() if self.conv else None
        self.bias = (t["r1"].float().contiguous(), t["r2"].float().contiguous()) if self.distance_bias else None

    def cache_need(self):
        kv = KVNeed(self.nkv, self.dk, self.window, self.dv if self.values_are_keys or self.dv != self.dk else 0,
                    self.keep_first, self.chunk, values_in_keys=self.values_are_keys)
        return [kv, StateNeed((self.conv - 1, (self.nh + self.nkv) * self.dk))] if self.conv > 1 else kv

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, nkv, dk, dv = self.nh, self.nkv, self.dk, self.dv
        conv_state = None
        if self.conv > 1:
            view, conv_state = view[0], view[1].state
        proj = self.scratch(step, "proj", (N, self.w_qkvg.shape[0]), torch.float32)
        linear(u, self.w_qkvg, proj)
        rot = self.position.rotary(u.device) if self.rot_dims else None
        q = self.scratch(step, "q", (N, nh * dk), step.dtype)
        rows = proj
        if self.conv:
            rows = self.scratch(step, "qk", (N, (nh + nkv) * dk), torch.float32)
            K.causal_conv(proj[:, :(nh + nkv) * dk], self.taps, None, conv_state, step.seq_of, step.cu, step.slots, rows,
                          step.n_seqs, one_each=step.is_decode)
        K.qkv_prepare_wide(rows, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, self.rot_dims,
                           rot[0] if rot is not None else None, step.positions, step.seq_of, view.page_table,
                           view.pool, view.page_size, q, nh, nkv, dk, 0 if self.values_are_keys else dv,
                           per_head=self.norm_per_head,
                           amplitude=float(getattr(self.position, "amplitude", lambda: 1.0)()) if self.rot_dims else 1.0)
        o = self.scratch(step, "mix", (N, nh * dv), step.dtype)
        g0 = nh * dk + nkv * dk + (0 if self.values_are_keys else nkv * dv)
        wide = self.gated == "element"
        extras = dict(softcap=self.softcap, window=self.window, keep_first=self.keep_first, sinks=self.sinks,
                      gate=proj[:, g0:g0 + (nh * dv if wide else nh)] if self.gated else None, chunk=self.chunk,
                      distance_bias=self.bias, values_in_keys=self.values_are_keys, gate_wide=wide,
                      out_all=self.scratch(step, "o_all", (N, nh, nkv, dv), torch.float32) if self.talk else None)
        # few query tokens, or many sequences with a token or two each: every query token on its own
        few = N <= K.DECODE_ATTENTION_MAX_TOKENS or step.max_len <= K.DECODE_ATTENTION_MAX_QUERIES
        if not few and K.attention_sink_prefill_supported(step.dtype, dk, dv):
            K.attention_sink_prefill(q, view.pool, view.page_size, view.page_table, step.cu, step.starts, o,
                                     step.n_seqs, nh, nkv, dk, dv, self.scale, split_weights=self.split_weights, **extras)
        else:
            K.attention_sink(q, view.pool, view.page_size, view.page_table, step.positions, step.seq_of, o, nh, nkv,
                             dk, dv, self.scale, **extras)
        if K.profiling_on():
            reach = (self.window + self.keep_first) if self.window else (self.chunk or None)
            pairs = sum(sum(min(s + i + 1, reach) if reach else s + i + 1 for i in range(n))
                        for s, n in zip(step.host_starts, step.host_lens))
            # keys and values: every query reads its own in a step of few tokens, a sequence's tile shares them otherwise
            rows = pairs if few else sum(min(s + n, n + reach) if reach else s + n
                                         for s, n in zip(step.host_starts, step.host_lens))
            vh = nkv if self.talk else 1          # mixed weights: every head's weights meet every kv head's values
            K.account(nkv * (dk + dv) * view.pool.element_size() * rows + N * nh * (dk + dv * vh) * q.element_size(),
                      2 * nh * (dk + dv) * vh * pairs)
        if self.talk:
            K.mix_heads(extras["out_all"], self.w_talk, o, nh, nkv, dv)
        linear(o, self.w_o, resid, accumulate=accumulate)


@register("mixer", "mamba2")
class Mamba2(Part):
    """Selective state space layer in its scalar-decay form (Dao and Gu, "Transformers are SSMs: Generalized
    Models and Efficient Algorithms Through Structured State Space Duality"): one projection of the input, laid
    out [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads] with inner = heads * value_dim;
    x, B and C pass a causal convolution of ``conv`` taps per channel (with bias) and silu;
    dt = softplus(dt + dt_bias); per head (head h reads group h // (heads / groups))
    S <- exp(-exp(A_log_h) dt) S + dt B x^T, y = S^T C + D_h x; y * silu(z) is divided by its root mean
    square in ``norm_groups`` equal parts and multiplied by ``norm``; then the out projection.  The state
    [heads, value_dim, state] and the convolution's last conv - 1 inputs are float32 per sequence and start
    at zero; decay, step size, state and sums are float32 in every run."""

    overwrites = True

    def __init__(self, hidden: int, n_heads: int, value_dim: int, state: int, groups: int, conv: int, norm_groups: int,
                 eps: float):
        if n_heads % groups:
            raise ValueError(f"{n_heads} heads are not a multiple of {groups} groups")
        if (n_heads * value_dim) % norm_groups:
            raise ValueError(f"{n_heads * value_dim} channels do not split into {norm_groups} parts for the norm")
        if not 1 <= conv <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {conv} is outside 1..{K.MAX_CONV_K}")
        if not 1 <= state <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"state size {state} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        self.hidden, self.nh, self.dv, self.state, self.groups = int(hidden), int(n_heads), int(value_dim), int(state), int(groups)
        self.conv, self.norm_groups, self.eps = int(conv), int(norm_groups), float(eps)
        self.inner = self.nh * self.dv
        self.channels = self.inner + 2 * self.groups * self.state

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh = self.hidden, self.nh
        return {"in": ParamSpec((2 * self.inner + 2 * self.groups * self.state + nh, H)),
                "conv": ParamSpec((self.channels, self.conv), "vector", "conv"),
                "conv.b": ParamSpec((self.channels,), "vector", "bias"),
                "dt_bias": ParamSpec((nh,), "vector", "bias"), "A_log": ParamSpec((nh,), "vector", "bias"),
                "D": ParamSpec((nh,), "vector", "norm"), "norm": ParamSpec((self.inner,), "vector", "norm"),
                "o": ParamSpec((H, self.inner))}

    def load(self, t) -> None:
        self.rows = t["in"].shape[0]
        self.w_in = _fuse_rows([t["in"]])
        self.taps, self.b_conv = t["conv"].contiguous(), t["conv.b"]
        self.dt_bias, self.a_log, self.skip, self.norm, self.w_o = t["dt_bias"], t["A_log"], t["D"], t["norm"], t["o"]

    def cache_need(self):
        return [StateNeed((self.nh, self.dv, self.state)), StateNeed((self.conv - 1, self.channels))]

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, inner, gn = self.nh, self.inner, self.groups * self.state
        ssm, conv = view
        proj = self.scratch(step, "proj", (N, self.w_in.shape[0]), torch.float32)
        linear(u, self.w_in, proj)
        xbc = self.scratch(step, "xbc", (N, self.channels), torch.float32)
        log_a = self.scratch(step, "log_a", (N, nh), torch.float32)
        b = self.scratch(step, "b", (N, nh), torch.float32)
        raw_dt = proj[:, inner + self.channels:inner + self.channels + nh]
        if step.is_decode and N == step.n_seqs:
            # one token a sequence: convolution, kept inputs and step size in one kernel
            K.ssm_decode_prepare(proj[:, inner:inner + self.channels], self.taps, self.b_conv, conv.state, step.slots, xbc,
                                 raw_dt, self.dt_bias, self.a_log, log_a, b)
        else:
            K.causal_conv_silu(proj[:, inner:inner + self.channels], self.taps, self.b_conv, conv.state, step.seq_of,
                               step.cu, step.slots, xbc, step.n_seqs)
            K.step_size(raw_dt, self.dt_bias, self.a_log, log_a, b)
        y = self.scratch(step, "y", (N, inner), torch.float32)
        K.scalar_scan(xbc[:, inner + gn:inner + 2 * gn], xbc[:, inner:inner + gn], xbc[:, :inner], log_a, b, ssm.state,
                      step.slots, step.cu, y, step.n_seqs, nh, self.state, self.dv, heads_per_group=nh // self.groups,
                      skip=self.skip, max_len=step.max_len, ws=step.ws)
        g = self.scratch(step, "mix", (N, inner), step.dtype)
        K.gated_rmsnorm(y, proj[:, :inner], self.norm, inner // self.norm_groups, self.eps, K.GATE_SILU_FIRST, g)
        linear(g, self.w_o, resid, accumulate=accumulate)


@register("mixer", "matrix_memory")
class MatrixMemory(Part):
    """Matrix memory with exponential gates (the mLSTM of Beck et al., "xLSTM: Extended Long Short-Term Memory"):
    q = W_q h / sqrt(key_dim), k = W_k h, v = W_v h per head; log gates i = cap tanh((W_i h + b_i) / cap) and
    f = log sigmoid(cap tanh((W_f h + b_f) / cap)) per head; with the running maximum m_t = max(f_t + m_(t-1), i_t)
    (m before the first token is 0) S <- e^(f + m_(t-1) - m_t) S + e^(i - m_t) k v^T, n likewise with k alone,
    o = S^T q / (max(|n . q|, e^(-m_t)) + 1e-6); each head's o is divided by its root mean square, the heads
    together are multiplied by ``norm`` and by sigmoid(W_g h); then the out projection.  S and n
    ([heads, value_dim + 1, key_dim], n as the last column) and m [heads] are float32 per sequence and start at
    zero; gates, maxima, state and sums are float32 in every run."""

    overwrites = True

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, eps: float):
        if not 1 <= key_dim <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"key size {key_dim} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        if gate_cap <= 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.hidden, self.nh, self.dk, self.dv = int(hidden), int(n_heads), int(key_dim), int(value_dim)
        self.cap, self.eps = float(gate_cap), float(eps)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh, qk, vv = self.hidden, self.nh, self.nh * self.dk, self.nh * self.dv
        return {"q": ParamSpec((qk, H)), "k": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "g": ParamSpec((vv, H)),
                "o": ParamSpec((H, vv)), "norm": ParamSpec((vv,), "vector", "norm"),
                "i": ParamSpec((nh, H)), "i.b": ParamSpec((nh,), "vector", "bias"),
                "f": ParamSpec((nh, H)), "f.b": ParamSpec((nh,), "vector", "bias")}

    def load(self, t) -> None:
        self.w_all = _fuse_rows([t["q"], t["k"], t["v"], t["g"], t["i"], t["f"]])
        self.b_i, self.b_f, self.norm, self.w_o = t["i.b"], t["f.b"], t["norm"], t["o"]

    def cache_need(self):
        return [StateNeed((self.nh, self.dv + 1, self.dk)), StateNeed((self.nh,))]

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, qk, vv = self.nh, self.nh * self.dk, self.nh * self.dv
        memory, maxima = view
        proj = self.scratch(step, "proj", (N, self.w_all.shape[0]), torch.float32)
        linear(u, self.w_all, proj)
        g0 = 2 * qk + 2 * vv
        log_a = self.scratch(step, "log_a", (N, nh), torch.float32)
        b = self.scratch(step, "b", (N, nh), torch.float32)
        m_tok = self.scratch(step, "m", (N, nh), torch.float32)
        K.memory_gates(proj[:, g0:g0 + nh], proj[:, g0 + nh:g0 + 2 * nh], self.b_i, self.b_f, self.cap, maxima.state,
                       step.slots, step.cu, log_a, b, m_tok, step.n_seqs, nh)
        o = self.scratch(step, "o", (N, vv), torch.float32)
        K.scalar_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], log_a, b, memory.state, step.slots,
                      step.cu, o, step.n_seqs, nh, self.dk, self.dv, m_tok=m_tok, q_scale=self.dk ** -0.5,
                      max_len=step.max_len, ws=step.ws)
        y = self.scratch(step, "mix", (N, vv), step.dtype)
        K.gated_rmsnorm(o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.norm, self.dv, self.eps, K.GATE_SIGMOID, y)
        linear(y, self.w_o, resid, accumulate=accumulate)


@register("mixer", "parallel")
class ParallelMixers(Part):
    """Two mixers side by side that read the same input; the result is left_scale * left + right_scale * right.
    Each keeps its own cache or state.  A block that can take the two results apart (``forward_sum``) adds them
    inside its next kernel; ``forward`` adds them itself."""

    nested_roles = {"left": "mixer", "right": "mixer"}
    overwrites = True

    def __init__(self, left, right, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        for side in (left, right):
            if not getattr(side, "overwrites", False):
                raise ValueError(f"mixer {getattr(side, 'kind', '?')} cannot write its result apart from the residual stream")

    def nested(self):
        return {"left": self.left, "right": self.right}

    @property
    def graph_safe(self):
        return getattr(self.left, "graph_safe", True) and getattr(self.right, "graph_safe", True)

    def cache_need(self):
        self._split = []
        needs = []
        for side in (self.left, self.right):
            need = side.cache_need()
            many = isinstance(need, (list, tuple))
            mine = list(need) if many else ([] if need is None else [need])
            self._split.append((len(mine), many))
            needs += mine
        return needs

    def _views(self, view):
        if not hasattr(self, "_split"):
            self.cache_need()
        views, out, at = list(view), [], 0
        for n, many in self._split:
            out.append(views[at:at + n] if many else (views[at] if n else None))
            at += n
        return out

    def forward_sum(self, u, step, view):
        """[(result, scale), (result, scale)]: the two mixers' results in buffers of their own (float32)."""
        N = u.shape[0]
        lv, rv = self._views(view)
        yl = self.scratch(step, "left", (N, self.left.hidden), torch.float32)
        yr = self.scratch(step, "right", (N, self.right.hidden), torch.float32)
        with profile_stage("mixer " + getattr(self.left, "kind", "?")):
            self.left.forward(u, yl, step, lv, accumulate=False)
        with profile_stage("mixer " + getattr(self.right, "kind", "?")):
            self.right.forward(u, yr, step, rv, accumulate=False)
        return [(yl, self.left_scale), (yr, self.right_scale)]

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        (yl, sl), (yr, sr) = self.forward_sum(u, step, view)
        if accumulate:
            resid.add_(yl, alpha=sl).add_(yr, alpha=sr)
        else:
            torch.add(yl * sl, yr, alpha=sr, out=resid)


@register("mixer", "latent_attention")
class LatentAttention(Part):
    """Softmax attention over a compressed cache (the multi-head latent attention of DeepSeek-V2): per head q = W_q h
    is [``dim`` unrotated | ``rot_dim`` rotated]; W_dkv h gives ``kv_rank`` numbers, divided by their root mean
    square and multiplied by a weight (the latent c), and ``rot_dim`` more, one rotated key part r shared by all
    heads; per head the unrotated key is W_uk c and the value W_uv c; score = (q_unrotated . k_unrotated +
    q_rotated . r) * scale; a sliding ``window`` (0: none); with ``sink`` a learned number per head joins the softmax's
    denominator; with ``gated`` the concatenated heads are multiplied by sigmoid(W_g h); then W_o.  The position
    part turns the first ``position.head_dim`` of the ``rot_dim`` elements, element i with i + head_dim / 2.

    Only [c | r] is cached, one row a token for all heads.  W_uk is folded into the query
    (qa = [W_uk^T q_unrotated | q_rotated]) and W_uv applied to the weighted sum of the cached c, so keys and values
    are never rebuilt.  Scores, softmax, norm and angles are float32."""

    nested_roles = {"position": "position"}
    overwrites = True

    def __init__(self, hidden: int, n_heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int, scale: float,
                 eps: float, position, window: int = 0, sink: bool = True, gated: bool = True):
        if not 1 <= kv_rank <= K.LATENT_MAX_RANK or not 0 <= rot_dim <= K.LATENT_MAX_ROT:
            raise ValueError(f"latent size {kv_rank} (1..{K.LATENT_MAX_RANK}), rotated size {rot_dim} (0..{K.LATENT_MAX_ROT})")
        self.hidden, self.nh, self.dim, self.rd = int(hidden), int(n_heads), int(dim), int(rot_dim)
        self.dv, self.rank, self.scale, self.eps = int(value_dim), int(kv_rank), float(scale), float(eps)
        self.window, self.sink, self.gated, self.position = int(window), bool(sink), bool(gated), position
        self.rot_dims = 0
        if isinstance(position, Rope):
            if position.style != "half_split" or position.head_dim > self.rd:
                raise ValueError("the rotation pairs element i with i + dims / 2 over at most the rotated size")
            self.rot_dims = position.head_dim
        elif position.rotary("cpu") is not None:
            raise ValueError("a rotation that is not a Rope part cannot say how many elements it turns")

    def nested(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, nh, qd, dv, rank = self.hidden, self.nh, self.dim + self.rd, self.dv, self.rank
        specs = {"q": ParamSpec((nh * qd, H)), "dkv": ParamSpec((rank + self.rd, H)),
                 "dkv.norm": ParamSpec((rank,), "vector", "norm"), "uk": ParamSpec((nh * self.dim, rank)),
                 "uv": ParamSpec((nh * dv, rank)), "o": ParamSpec((H, nh * dv))}
        if self.sink:
            specs["sink"] = ParamSpec((nh,), "vector", "bias")
        if self.gated:
            specs["g"] = ParamSpec((nh * dv, H))
        return specs

    def load(self, t) -> None:
        self.w_in = _fuse_rows([t["q"], t["dkv"]] + ([t["g"]] if self.gated else []))
        self.c_norm, self.sinks, self.w_o = t["dkv.norm"], t.get("sink"), t["o"]
        self.w_uk, self.w_uv = t["uk"].contiguous(), t["uv"].contiguous()
        # steps of many tokens build every head's keys and values from the cached rows with one product
        self.w_kv = None
        if self.w_uk.dtype == torch.bfloat16 and K.latent_prefill_fits(self.dim, self.rd, self.dv, self.rank):
            self.w_kv = _fuse_rows([self.w_uk, self.w_uv])

    def cache_need(self):
        return KVNeed(1, self.rank + self.rd, self.window, self.rank, values_in_keys=True)

    # a step takes the tensor-core path when a sequence brings this many tokens and the cached rows it has to turn
    # into keys and values are at most this many times its tokens
    LONG_STEP, LONG_ROWS = 16, 4

    def _seen_rows(self, step) -> int:
        w = self.window
        return sum(s + n - (max(0, s - w + 1) if w else 0) for s, n in zip(step.host_starts, step.host_lens))

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, dim, rd, dv, rank = self.nh, self.dim, self.rd, self.dv, self.rank
        c0 = nh * (dim + rd)
        g0 = c0 + rank + rd
        proj = self.scratch(step, "proj", (N, self.w_in.shape[0]), torch.float32)
        linear(u, self.w_in, proj)
        rot = self.position.rotary(u.device) if self.rot_dims else None
        inv_freq = rot[0] if rot is not None else None
        gate = proj[:, g0:g0 + nh * dv] if self.gated else None
        y = self.scratch(step, "mix", (N, nh * dv), step.dtype)
        rows = self._seen_rows(step) if step.max_len >= self.LONG_STEP else 0
        if K.profiling_on():
            reach = self.window or None
            pairs = sum(sum(min(s + i + 1, reach) if reach else s + i + 1 for i in range(n))
                        for s, n in zip(step.host_starts, step.host_lens))
        if (self.w_kv is not None and step.dtype == torch.bfloat16 and view.pool.dtype == torch.bfloat16
                and 0 < rows <= self.LONG_ROWS * N):
            K.latent_prepare(proj, 0, c0, self.c_norm, self.eps, inv_freq, step.positions, step.seq_of, view.page_table,
                             view.pool, view.page_size, None, nh, dim, rd, rank, self.rot_dims)
            q = self.scratch(step, "q", (N, nh, dim + rd), torch.bfloat16)
            K.latent_query(proj, 0, inv_freq, step.positions, q, nh, dim, rd, self.rot_dims)
            c = self.scratch(step, "c", (rows, rank), torch.bfloat16)
            r = self.scratch(step, "r", (rows, rd), torch.bfloat16)
            K.latent_gather(view.pool, view.page_size, view.page_table, step.cu, step.starts, step.n_seqs, self.window, c, r)
            kx = self.scratch(step, "kx", (rows, self.w_kv.shape[0]), torch.bfloat16)
            linear(c, self.w_kv, kx)
            K.latent_attention_prefill(q, kx, nh * dim, r, step.cu, step.starts, step.n_seqs, y, nh, dim, rd, dv,
                                       self.scale, window=self.window, sinks=self.sinks, gate=gate)
            if K.profiling_on():
                K.account(N * nh * (dim + rd + dv) * 2 + rows * nh * (dim + dv) * 2 + rows * rd * 2,
                          2 * nh * (dim + rd + 2 * dv) * pairs)
            linear(y, self.w_o, resid, accumulate=accumulate)
            return
        qa = self.scratch(step, "qa", (N, nh, rank + rd), torch.float32)
        K.latent_prepare(proj, 0, c0, self.c_norm, self.eps, inv_freq, step.positions, step.seq_of, view.page_table,
                         view.pool, view.page_size, qa, nh, dim, rd, rank, self.rot_dims)
        K.head_product(proj[:, :c0].unflatten(1, (nh, dim + rd)), self.w_uk, qa, nh, dim, rank, transposed=True)
        o_lat = self.scratch(step, "o_lat", (N, nh, rank), torch.float32)
        # few query tokens with many keys each: the keys in shares.  The number of shares follows from what the page
        # table can hold, not from the lengths of the moment, so that a recorded step stays right as they grow.
        longest = view.page_table.shape[1] * view.page_size
        splits = K.latent_splits(N, nh, min(longest, self.window) if self.window else longest, K.n_sms())
        part = None
        if splits > 1:
            part = (self.scratch(step, "part_o", (N, nh, splits, rank), torch.float32),
                    self.scratch(step, "part_ml", (N, nh, splits, 2), torch.float32))
        K.latent_attention(qa, view.pool, view.page_size, view.page_table, step.positions, step.seq_of, o_lat, nh, rank,
                           rd, self.scale, window=self.window, sinks=self.sinks, splits=splits, part=part)
        if K.profiling_on():
            K.account((rank + rd) * view.pool.element_size() * pairs + N * nh * (2 * rank + rd) * 4,
                      2 * nh * (2 * rank + rd) * pairs)
        K.head_product(o_lat, self.w_uv, y.view(N, nh, dv), nh, rank, dv, gate=gate)
        linear(y, self.w_o, resid, accumulate=accumulate)


def _block_diagonal(a: torch.Tensor, b: torch.Tensor, cols: int, multiple: int = 16) -> torch.Tensor:
    """[[a, 0], [0, b]] with ``cols`` columns (>= the two widths together) and rows padded to ``multiple``: two
    products of different inputs as one product of the inputs side by side."""
    if a.dtype != b.dtype:
        a, b = a.float(), b.float()
    rows = a.shape[0] + b.shape[0]
    out = torch.zeros((rows + (-rows % multiple), cols), dtype=a.dtype, device=a.device)
    out[:a.shape[0], :a.shape[1]] = a
    out[a.shape[0]:rows, a.shape[1]:a.shape[1] + b.shape[1]] = b
    return out.contiguous()


@register("mixer", "channel_delta")
class ChannelDelta(Part):
    """The gated delta rule with a decay per key channel (Yang, Kautz and Hatamizadeh, "Gated Delta Networks:
    Improving Mamba2 with Delta Rule", with the decay of one number a head widened to one a key channel):
    q = W_q h and k = W_k h on ``kv_heads`` heads of ``key_dim``, v = W_v h on ``n_heads`` heads of ``value_dim``
    (head h reads q/k head h // (n_heads / kv_heads)); each passes a causal convolution of ``conv`` taps per
    channel (no bias, the last tap the current token's) and silu; q and k become unit vectors per head
    (x / sqrt(sum x^2 + 1e-6)), q times key_dim^-1/2; beta = sigmoid(W_b h) per head;
    g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel; per head
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; each head's o over its root mean square, times
    ``norm`` [value_dim], times sigmoid(W_g2 (W_g1 h)); then W_o.  The state [heads, value_dim, key_dim] and the
    convolution's last conv - 1 inputs are float32 per sequence and start at zero; decays, gates of the recurrence,
    unit norms, state and sums are float32 in every run.  ``decay_rank`` / ``gate_rank``: the inner sizes of the
    two-step projections; None takes them from the checkpoint."""

    overwrites = True
    UNIT_EPS = 1e-6

    def __init__(self, hidden: int, n_heads: int, kv_heads: int, key_dim: int, value_dim: int, conv: int, eps: float,
                 decay_rank: Optional[int] = None, gate_rank: Optional[int] = None):
        if kv_heads < 1 or n_heads % kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {kv_heads} kv heads")
        if not 1 <= key_dim <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"key size {key_dim} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        if not 1 <= conv <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {conv} is outside 1..{K.MAX_CONV_K}")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = int(hidden), int(n_heads), int(kv_heads), int(key_dim), int(value_dim)
        self.conv, self.eps = int(conv), float(eps)
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.gate_rank = None if gate_rank is None else int(gate_rank)
        self.channels = 2 * self.nkv * self.dk + self.nh * self.dv

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, qk, vv, hk, c = self.hidden, self.nkv * self.dk, self.nh * self.dv, self.nh * self.dk, self.conv
        return {"q": ParamSpec((qk, H)), "q.conv": ParamSpec((qk, c), "vector", "conv"),
                "k": ParamSpec((qk, H)), "k.conv": ParamSpec((qk, c), "vector", "conv"),
                "v": ParamSpec((vv, H)), "v.conv": ParamSpec((vv, c), "vector", "conv"),
                "b": ParamSpec((self.nh, H)), "A_log": ParamSpec((self.nh,), "vector", "bias"),
                "norm": ParamSpec((self.dv,), "vector", "norm"),
                "a1": ParamSpec((self.decay_rank, H)), "a2": ParamSpec((hk, self.decay_rank)),
                "dt_bias": ParamSpec((hk,), "vector", "bias"),
                "g1": ParamSpec((self.gate_rank, H)), "g2": ParamSpec((vv, self.gate_rank)), "o": ParamSpec((H, vv))}

    def load(self, t) -> None:
        for one, two in (("a1", "a2"), ("g1", "g2")):
            if t[one].shape[0] != t[two].shape[1]:
                raise ValueError(f"the two projections disagree: {one} is {tuple(t[one].shape)}, {two} {tuple(t[two].shape)}")
        self.w_in = _fuse_rows([t["q"], t["k"], t["v"], t["b"]])
        self.w_low = _fuse_rows([t["a1"], t["g1"]])
        self.w_up = _block_diagonal(t["a2"], t["g2"], self.w_low.shape[0])
        self.taps = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm, self.w_o = t["A_log"], t["dt_bias"], t["norm"], t["o"]

    def cache_need(self):
        needs = [StateNeed((self.nh, self.dv, self.dk))]
        if self.conv > 1:
            needs.append(StateNeed((self.conv - 1, self.channels)))
        return needs

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, nkv, dk, dv, C = self.nh, self.nkv, self.dk, self.dv, self.channels
        qk, vv, hk = nkv * dk, nh * dv, nh * dk
        memory = view[0]
        conv_state = view[1].state if self.conv > 1 else None
        proj = self.scratch(step, "proj", (N, self.w_in.shape[0]), torch.float32)
        linear(u, self.w_in, proj)
        low = self.scratch(step, "low", (N, self.w_low.shape[0]), step.dtype)
        linear(u, self.w_low, low)
        up = self.scratch(step, "up", (N, self.w_up.shape[0]), torch.float32)
        linear(low, self.w_up, up)
        xbc = self.scratch(step, "xbc", (N, C), torch.float32)
        K.causal_conv_silu(proj[:, :C], self.taps, None, conv_state, step.seq_of, step.cu, step.slots, xbc, step.n_seqs)
        o = self.scratch(step, "o", (N, vv), torch.float32)
        K.delta_scan(xbc[:, :qk], xbc[:, qk:2 * qk], xbc[:, 2 * qk:], proj[:, C:C + nh], up[:, :hk], self.dt_bias,
                     self.a_log, memory.state, step.slots, step.cu, o, step.n_seqs, nh, nkv, dk, dv,
                     q_scale=dk ** -0.5, norm_eps=self.UNIT_EPS, max_len=step.max_len, ws=step.ws)
        y = self.scratch(step, "mix", (N, vv), step.dtype)
        K.gated_rmsnorm(o, up[:, hk:hk + vv], self.norm, dv, self.eps, K.GATE_SIGMOID, y)
        linear(y, self.w_o, resid, accumulate=accumulate)


@register("mixer", "gated_recurrence")
class GatedRecurrence(Part):
    """A recurrent block around a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear
    Recurrences with Local Attention for Efficient Language Models"): two branches of ``width`` channels,
    y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a causal convolution of ``conv`` taps per channel with a
    bias and no activation (the last tap the current token's); u cut into ``blocks`` equal parts, in part b
    r = sigmoid(A_b u_b + a_b) and i = sigmoid(B_b u_b + b_b) with square matrices [out, in];
    log a = -``c`` r softplus(lam), S_t = a S_(t-1) + sqrt(1 - a^2) i u from S = 0 (the first token is no special
    case); the result is W_o (S * y).  S [width] and the convolution's last conv - 1 inputs are float32 per sequence
    and start at zero; gates, decays, state and sums are float32 in every run."""

    overwrites = True

    def __init__(self, hidden: int, width: int, blocks: int, conv: int, c: float = 8.0):
        if blocks < 1 or width % blocks:
            raise ValueError(f"{width} channels do not split into {blocks} equal parts")
        if not 1 <= conv <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {conv} is outside 1..{K.MAX_CONV_K}")
        self.hidden, self.width, self.blocks, self.conv, self.c = int(hidden), int(width), int(blocks), int(conv), float(c)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, C, nb = self.hidden, self.width, self.blocks
        bs = C // nb
        return {"y": ParamSpec((C, H)), "y.b": ParamSpec((C,), "vector", "bias"),
                "x": ParamSpec((C, H)), "x.b": ParamSpec((C,), "vector", "bias"),
                "conv": ParamSpec((C, self.conv), "vector", "conv"), "conv.b": ParamSpec((C,), "vector", "bias"),
                "ra": ParamSpec((nb, bs, bs), "vector", "linear"), "ra.b": ParamSpec((nb, bs), "vector", "bias"),
                "ri": ParamSpec((nb, bs, bs), "vector", "linear"), "ri.b": ParamSpec((nb, bs), "vector", "bias"),
                "lam": ParamSpec((C,), "vector", "norm"), "o": ParamSpec((H, C))}

    def load(self, t) -> None:
        self.w_yx = _fuse_rows([t["y"], t["x"]])
        b = torch.cat([t["y.b"].float(), t["x.b"].float()])
        self.b_yx = torch.cat([b, b.new_zeros(self.w_yx.shape[0] - b.numel())]).contiguous()
        self.taps, self.b_conv = t["conv"].contiguous(), t["conv.b"]
        # the parts' matrices transposed to [in, out]: the gate kernel's threads read consecutive outputs
        self.wa_t = t["ra"].float().transpose(1, 2).contiguous()
        self.wi_t = t["ri"].float().transpose(1, 2).contiguous()
        self.ba, self.bi = t["ra.b"].float().reshape(-1).contiguous(), t["ri.b"].float().reshape(-1).contiguous()
        self.lam, self.w_o = t["lam"], t["o"]

    def cache_need(self):
        needs = [StateNeed((self.width,))]
        if self.conv > 1:
            needs.append(StateNeed((self.conv - 1, self.width)))
        return needs

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N, C = u.shape[0], self.width
        memory = view[0]
        conv_state = view[1].state if self.conv > 1 else None
        proj = self.scratch(step, "proj", (N, self.w_yx.shape[0]), torch.float32)
        linear(u, self.w_yx, proj, bias=self.b_yx)
        uc = self.scratch(step, "u", (N, C), torch.float32)
        K.causal_conv(proj[:, C:2 * C], self.taps, self.b_conv, conv_state, step.seq_of, step.cu, step.slots, uc, step.n_seqs,
                      one_each=step.is_decode)
        a = self.scratch(step, "a", (N, C), torch.float32)
        x = self.scratch(step, "x", (N, C), torch.float32)
        K.block_gates(uc, self.wa_t, self.wi_t, self.ba, self.bi, self.lam, self.c, a, x)
        g = self.scratch(step, "mix", (N, C), step.dtype)
        K.gated_recurrence(a, x, proj[:, :C], memory.state, step.slots, step.cu, g, step.n_seqs, max_len=step.max_len)
        linear(g, self.w_o, resid, accumulate=accumulate)


@register("mixer", "gated_delta")
class GatedDeltaRule(Part):
    """The gated delta rule with one decay per head (Yang, Kautz and Hatamizadeh, "Gated Delta Networks: Improving
    Mamba2 with Delta Rule"): q = W_q h and k = W_k h on ``kv_heads`` heads of ``key_dim``, v = W_v h on ``n_heads``
    heads of ``value_dim`` (head h reads q/k head h // (n_heads / kv_heads)); each passes a causal convolution of
    ``conv`` taps per channel (no bias, the last tap the current token's) and silu; q and k become unit vectors per
    head (x / sqrt(sum x^2 + 1e-6)), q times key_dim^-1/2; beta = sigmoid(W_b h) and
    g = exp(-exp(A_log_h) softplus(W_a h + dt_bias)) per head; per head S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q; each head's o over its root mean square, times ``norm`` [value_dim], times
    silu(W_g h); then W_o.  The state [heads, value_dim, key_dim] and the convolution's last conv - 1 inputs are
    float32 per sequence and start at zero; decays, beta, unit norms, state and sums are float32 in every run."""

    overwrites = True
    UNIT_EPS = 1e-6

    def __init__(self, hidden: int, n_heads: int, kv_heads: int, key_dim: int, value_dim: int, conv: int, eps: float):
        if kv_heads < 1 or n_heads % kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {kv_heads} kv heads")
        if not 1 <= key_dim <= K.MAX_SCAN_KEY_DIM:
            raise ValueError(f"key size {key_dim} is outside 1..{K.MAX_SCAN_KEY_DIM}")
        if not 1 <= conv <= K.MAX_CONV_K:
            raise ValueError(f"convolution width {conv} is outside 1..{K.MAX_CONV_K}")
        self.hidden, self.nh, self.nkv, self.dk, self.dv = int(hidden), int(n_heads), int(kv_heads), int(key_dim), int(value_dim)
        self.conv, self.eps = int(conv), float(eps)
        self.channels = 2 * self.nkv * self.dk + self.nh * self.dv

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, qk, vv, c = self.hidden, self.nkv * self.dk, self.nh * self.dv, self.conv
        return {"q": ParamSpec((qk, H)), "q.conv": ParamSpec((qk, c), "vector", "conv"),
                "k": ParamSpec((qk, H)), "k.conv": ParamSpec((qk, c), "vector", "conv"),
                "v": ParamSpec((vv, H)), "v.conv": ParamSpec((vv, c), "vector", "conv"),
                "b": ParamSpec((self.nh, H)), "a": ParamSpec((self.nh, H)),
                "A_log": ParamSpec((self.nh,), "vector", "bias"), "dt_bias": ParamSpec((self.nh,), "vector", "bias"),
                "norm": ParamSpec((self.dv,), "vector", "norm"), "g": ParamSpec((vv, H)), "o": ParamSpec((H, vv))}

    def load(self, t) -> None:
        # one product: [q | k | v | gate | beta | decay]
        self.w_in = _fuse_rows([t["q"], t["k"], t["v"], t["g"], t["b"], t["a"]])
        self.taps = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm, self.w_o = t["A_log"], t["dt_bias"], t["norm"], t["o"]

    def cache_need(self):
        needs = [StateNeed((self.nh, self.dv, self.dk))]
        if self.conv > 1:
            needs.append(StateNeed((self.conv - 1, self.channels)))
        return needs

    def forward(self, u, resid, step, view, accumulate: bool = True) -> None:
        N = u.shape[0]
        nh, nkv, dk, dv, C = self.nh, self.nkv, self.dk, self.dv, self.channels
        qk, vv = nkv * dk, nh * dv
        memory = view[0]
        conv_state = view[1].state if self.conv > 1 else None
        proj = self.scratch(step, "proj", (N, self.w_in.shape[0]), torch.float32)
        linear(u, self.w_in, proj)
        xbc = self.scratch(step, "xbc", (N, C), torch.float32)
        K.causal_conv_silu(proj[:, :C], self.taps, None, conv_state, step.seq_of, step.cu, step.slots, xbc, step.n_seqs,
                           one_each=step.is_decode)
        b0 = C + vv
        o = self.scratch(step, "o", (N, vv), torch.float32)
        K.delta_scan(xbc[:, :qk], xbc[:, qk:2 * qk], xbc[:, 2 * qk:], proj[:, b0:b0 + nh], proj[:, b0 + nh:b0 + 2 * nh],
                     self.dt_bias, self.a_log, memory.state, step.slots, step.cu, o, step.n_seqs, nh, nkv, dk, dv,
                     q_scale=dk ** -0.5, norm_eps=self.UNIT_EPS, max_len=step.max_len, ws=step.ws, head_decay=True)
        y = self.scratch(step, "mix", (N, vv), step.dtype)
        K.gated_rmsnorm(o, proj[:, C:C + vv], self.norm, dv, self.eps, K.GATE_SILU, y)
        linear(y, self.w_o, resid, accumulate=accumulate)
