"""Arrangements of a layer's parts."""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops.kernels import profile_stage
from .base import Part
from .norm import LayerNorm, RMSNorm
from .registry import register


@register("block", "prenorm")
class PreNormBlock(Part):
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the arrangement of both
    layer kinds of the reference (crates/mivi-model/src/ssm.rs:65,155-166;
    transformer.rs:317,338; ffn.rs:64,106).  The residual stream stays in
    float32; the normed activations are in the model's dtype."""

    nested_roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def nested(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def cache_need(self):
        """The mixer's needs, followed by the feed-forward's if it keeps something too (the block's need is
        then a list, and ``forward`` deals the views out again)."""
        need = self.mixer.cache_need()
        extra = self.ffn.cache_need() if hasattr(self.ffn, "cache_need") else None
        if extra is None:
            self._views = None
            return need
        mixer_list = isinstance(need, (list, tuple))
        mine = list(need) if mixer_list else ([] if need is None else [need])
        ffn_list = isinstance(extra, (list, tuple))
        self._views = (len(mine), mixer_list, ffn_list)
        return mine + (list(extra) if ffn_list else [extra])

    def entry_link(self, step):
        """The first norm of this block as a link that the block before may fill, or None."""
        if step.carry_norms and hasattr(self.mixer_norm, "link") and self.mixer.carries_norm(step)[0]:
            return self.mixer_norm.link(step, "entry")
        return None

    def forward(self, resid, step, view, after=None) -> None:
        """``after``: the block that runs next in this step, if any.  In a step of few tokens the two
        norms are not kernels of their own where the parts allow it: the product that completes the
        residual stream writes the next norm's rows, the product that reads them applies its scale."""
        N, H = resid.shape
        ffn_kw = {}
        if getattr(self, "_views", None) is not None:
            n_mixer, mixer_list, ffn_list = self._views
            views = list(view)
            view = views[:n_mixer] if mixer_list else (views[0] if n_mixer else None)
            ffn_kw["view"] = views[n_mixer:] if ffn_list else views[n_mixer]
        carry = step.carry_norms
        _, mixer_emits = self.mixer.carries_norm(step) if carry else (False, False)
        ffn_accepts, ffn_emits = self.ffn.carries_norm(step) if carry else (False, False)
        entry = step.take_link(self.mixer_norm)
        mid = self.ffn_norm.link(step, "mid") if mixer_emits and ffn_accepts and hasattr(self.ffn_norm, "link") else None
        leave = after.entry_link(step) if ffn_emits and after is not None and hasattr(after, "entry_link") else None
        kw = {}
        if entry is not None:
            u, kw["scale"] = entry.xg, entry
        else:
            u = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.mixer_norm.forward(resid, u)
        if mid is not None:
            kw["emit"] = mid
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            self.mixer.forward(u, resid, step, view, **kw)
        kw = dict(ffn_kw)
        if mid is not None:
            g, kw["scale"] = mid.xg, mid
        else:
            g = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.ffn_norm.forward(resid, g)
        if leave is not None:
            kw["emit"] = leave
        with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
            self.ffn.forward(g, resid, step, **kw)
        step.leave_link(leave)


@register("block", "prenorm_optional")
class PreNormOptionalBlock(Part):
    """x += mixer(norm(x)); then, if the layer has a feed-forward, x += feed_forward(norm(x)); then, if it has
    a per-layer token input, that adds to x.  The residual stream stays in float32; the normed activations
    are in the model's dtype.  Norms are kernels of their own here (no product carries them)."""

    nested_roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward",
                    "token_input": "token_input"}

    def __init__(self, mixer_norm, mixer, ffn_norm=None, ffn=None, token_input=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.token_input = mixer_norm, mixer, ffn_norm, ffn, token_input

    def nested(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn,
                 "token_input": self.token_input}
        return {k: v for k, v in parts.items() if v is not None}

    def cache_need(self):
        return self.mixer.cache_need()

    def entry_link(self, step):
        """No product carries this block's norms; the method is there so that the model tells ``forward`` which
        block runs next (``after``)."""
        return None

    def forward(self, resid, step, view, after=None) -> None:
        """``after``: the block that runs next in this step, if any.  Where this block ends with a token input and
        the next one is of this kind with a layer norm first, that norm runs inside the token input's last kernel
        and its rows are handed over through the step (``step.handed``)."""
        N, H = resid.shape
        handed, step.handed = getattr(step, "handed", None), None
        if handed is not None and handed[0] is self.mixer_norm:
            u = handed[1]
        else:
            u = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.mixer_norm.forward(resid, u)
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            self.mixer.forward(u, resid, step, view)
        if self.ffn is not None:
            g = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.ffn_norm.forward(resid, g)
            with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
                self.ffn.forward(g, resid, step)
        if self.token_input is not None:
            nxt = after.mixer_norm if isinstance(after, PreNormOptionalBlock) and isinstance(after.mixer_norm, LayerNorm) \
                and not after.mixer_norm.has_bias and getattr(self.token_input, "takes_norm", False) else None
            with profile_stage("token_input " + getattr(self.token_input, "kind", "?")):
                if nxt is not None:
                    # another buffer than "normed": this block's rows there are done with, the next block's
                    # second norm will write there while its first norm's rows are still read
                    out = self.scratch(step, "normed_entry", (N, H), step.dtype)
                    self.token_input.forward(resid, step, then_norm=(nxt, out))
                    step.handed = (nxt, out)
                else:
                    self.token_input.forward(resid, step)


@register("block", "prenorm_scaled")
class PreNormScaledBlock(Part):
    """x += m * s1 * mixer(norm1(x)); then, if the layer has a feed-forward, x += m * s2 * feed_forward(norm2(x)):
    every sublayer's result is multiplied element by element by a learned vector of the stream's width (``scale1``,
    ``scale2``) and by the constant ``residual_mult`` m before it joins the stream.  The norms are root-mean-square
    norms.  A sublayer writes its result into a float32 buffer of its own (a mixer with ``forward_sum`` gives its two
    branches apart, with their factors); ONE kernel then adds it, times m * s, to the float32 stream and norms the
    completed row for the sublayer that reads it next, this block's feed-forward or the next block's mixer."""

    nested_roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def __init__(self, hidden: int, mixer_norm, mixer, ffn_norm=None, ffn=None, residual_mult: float = 1.0):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not isinstance(norm, RMSNorm):
                raise ValueError("the norms of a prenorm_scaled block are rmsnorm parts")
        for part in (mixer, ffn):
            if part is not None and not (getattr(part, "overwrites", False) or hasattr(part, "forward_sum")):
                raise ValueError(f"{getattr(part, 'kind', '?')} cannot write its result apart from the residual stream")
        self.hidden, self.mult = int(hidden), float(residual_mult)
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def nested(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}
        return {k: v for k, v in parts.items() if v is not None}

    def param_specs(self):
        from .spec import ParamSpec
        specs = {"scale1": ParamSpec((self.hidden,), "vector", "norm")}
        if self.ffn is not None:
            specs["scale2"] = ParamSpec((self.hidden,), "vector", "norm")
        return specs

    def load(self, t) -> None:
        # m * s as one float32 vector a sublayer
        self.vec1 = (t["scale1"].float() * self.mult).contiguous()
        self.vec2 = (t["scale2"].float() * self.mult).contiguous() if self.ffn is not None else None

    def cache_need(self):
        return self.mixer.cache_need()

    def entry_link(self, step):
        """No product carries this block's norms; the method is there so that the model tells ``forward`` which
        block runs next (``after``)."""
        return None

    def _run(self, part, name, u, step, *args):
        """The sublayer's result in a buffer of its own, as a list of (rows, factor)."""
        if hasattr(part, "forward_sum"):
            return part.forward_sum(u, step, *args)
        y = self.scratch(step, name, (u.shape[0], self.hidden), torch.float32)
        part.forward(u, y, step, *args, accumulate=False)
        return [(y, 1.0)]

    def _join(self, branches, vec, resid, norm, out):
        (y1, s1), rest = branches[0], branches[1:]
        if len(rest) > 1:
            raise ValueError("at most two branches are summed in the joining kernel")
        y2, s2 = rest[0] if rest else (None, 1.0)
        if norm is None:
            K.scaled_add_norm(y1, vec, resid, s1=s1, y2=y2, s2=s2)
        else:
            K.scaled_add_norm(y1, vec, resid, s1=s1, y2=y2, s2=s2, w=norm.weight, eps=norm.eps, out=out)

    def forward(self, resid, step, view, after=None) -> None:
        N, H = resid.shape
        handed, step.handed = getattr(step, "handed", None), None
        if handed is not None and handed[0] is self.mixer_norm:
            u = handed[1]
        else:
            u = self.scratch(step, "normed", (N, H), step.dtype)
            with profile_stage("norm"):
                self.mixer_norm.forward(resid, u)
        # the block after this one, if it is of this kind, gets its first norm's rows from this block's last kernel
        nxt = after.mixer_norm if isinstance(after, PreNormScaledBlock) else None
        # (into the buffer that held this block's own: its mixer is done with them by then)
        nxt_out = self.scratch(step, "normed", (N, H), step.dtype) if nxt is not None else None
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            branches = self._run(self.mixer, "y", u, step, view)
        if self.ffn is None:
            with profile_stage("norm"):
                self._join(branches, self.vec1, resid, nxt, nxt_out)
        else:
            g = self.scratch(step, "normed_mid", (N, H), step.dtype)
            with profile_stage("norm"):
                self._join(branches, self.vec1, resid, self.ffn_norm, g)
            with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
                branches = self._run(self.ffn, "y", g, step)
            with profile_stage("norm"):
                self._join(branches, self.vec2, resid, nxt, nxt_out)
        if nxt is not None:
            step.handed = (nxt, nxt_out)


@register("block", "postnorm")
class PostNormBlock(Part):
    """x += norm1(mixer(x)); then, if the layer has a feed-forward, x += norm2(feed_forward(x)): the norms sit on
    the sublayers' OUTPUTS and the sublayers read the stream itself (rounded to the model's dtype where that is
    narrower).  The norms are root-mean-square norms.  One kernel per sublayer adds a mixer's branches (a mixer
    with ``forward_sum`` gives them apart, with their factors), norms the sum, adds it to the float32 stream and
    writes the rounded rows that the next sublayer multiplies."""

    nested_roles = {"mixer": "mixer", "mixer_norm": "norm", "ffn": "feed_forward", "ffn_norm": "norm"}

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together or not at all")
        for norm in (mixer_norm, ffn_norm):
            if norm is not None and not isinstance(norm, RMSNorm):
                raise ValueError("the norms of a postnorm block are rmsnorm parts")
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm

    def nested(self):
        parts = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "ffn": self.ffn, "ffn_norm": self.ffn_norm}
        return {k: v for k, v in parts.items() if v is not None}

    def cache_need(self):
        return self.mixer.cache_need()

    def entry_link(self, step):
        """No product carries this block's norms; the method is there so that the model tells ``forward`` which
        block runs next (``after``)."""
        return None

    def _run(self, part, u, step, *args):
        """The sublayer's result in a buffer of its own, as a list of (rows, factor)."""
        N = u.shape[0]
        if hasattr(part, "forward_sum"):
            return part.forward_sum(u, step, *args)
        y = self.scratch(step, "y", (N, self.mixer_norm.dim), torch.float32)
        if getattr(part, "overwrites", False):
            part.forward(u, y, step, *args, accumulate=False)
        else:
            y.zero_()                                 # a part that can only add
            part.forward(u, y, step, *args)
        return [(y, 1.0)]

    def _add(self, branches, norm, resid, rounded):
        (y1, s1), rest = branches[0], branches[1:]
        if len(rest) > 1:
            raise ValueError("at most two branches are summed in the norm's kernel")
        y2, s2 = rest[0] if rest else (None, 1.0)
        K.rmsnorm_add_sum(y1, norm.weight, norm.eps, resid, s1=s1, y2=y2, s2=s2, rounded=rounded)

    def forward(self, resid, step, view, after=None) -> None:
        N, H = resid.shape
        narrow = step.dtype != torch.float32
        handed, step.handed = getattr(step, "handed", None), None
        if not narrow:
            u = resid                                   # the sublayers multiply the stream itself
        elif handed is not None and handed[0] == "stream":
            u = handed[1]
        else:
            u = K.round_rows(resid, step.ws.get("stream_rounded", (N, H), step.dtype))
        rounded = step.ws.get("stream_rounded", (N, H), step.dtype) if narrow else None
        last = self.ffn is None
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            branches = self._run(self.mixer, u, step, view)
        with profile_stage("norm"):
            # the rounded rows are wanted by this block's feed-forward, or by the next block of this kind
            want = narrow and (not last or isinstance(after, PostNormBlock))
            self._add(branches, self.mixer_norm, resid, rounded if want else None)
        if not last:
            with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
                branches = self._run(self.ffn, rounded if narrow else resid, step)
            with profile_stage("norm"):
                want = narrow and isinstance(after, PostNormBlock)
                self._add(branches, self.ffn_norm, resid, rounded if want else None)
        if narrow and isinstance(after, PostNormBlock):
            step.handed = ("stream", rounded)


@register("block", "parallel_prenorm")
class ParallelPreNormBlock(Part):
    """x += mixer(h) + feed_forward(h) with h = norm(x): ONE norm whose output both sublayers read (the feed-forward
    is optional).  The residual stream stays in float32; the normed activations are in the model's dtype.  Both
    sublayers add their results into the stream themselves."""

    nested_roles = {"norm": "norm", "mixer": "mixer", "ffn": "feed_forward"}

    def __init__(self, norm, mixer, ffn=None):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn

    def nested(self):
        parts = {"norm": self.norm, "mixer": self.mixer, "ffn": self.ffn}
        return {k: v for k, v in parts.items() if v is not None}

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, resid, step, view) -> None:
        N, H = resid.shape
        u = self.scratch(step, "normed", (N, H), step.dtype)
        with profile_stage("norm"):
            self.norm.forward(resid, u)
        with profile_stage("mixer " + getattr(self.mixer, "kind", "?")):
            self.mixer.forward(u, resid, step, view)
        if self.ffn is not None:
            with profile_stage("feed_forward " + getattr(self.ffn, "kind", "?")):
                self.ffn.forward(u, resid, step)


@register("block", "stream_restart")
class StreamRestart(Part):
    """What stands before a pass over a run of layers that is walked several times with the same weights:
    x += embedding output (with ``add_embedding``: every pass but the first) + steps[row], one learned vector a pass.
    The embedding leaves its output for this through ``step.embedding_output``.  No mixer, no cache."""

    def __init__(self, hidden: int, n_rows: int, row: int, add_embedding: bool):
        if not 0 <= int(row) < int(n_rows):
            raise ValueError(f"pass {row} of {n_rows}")
        self.hidden, self.n_rows, self.row, self.add_embedding = int(hidden), int(n_rows), int(row), bool(add_embedding)

    def param_specs(self):
        from .spec import ParamSpec
        return {"steps": ParamSpec((self.n_rows, self.hidden), "vector", "bias")}

    def load(self, t) -> None:
        self.vec = t["steps"][self.row].contiguous()

    def forward(self, resid, step, view) -> None:
        rows = None
        if self.add_embedding:
            rows = getattr(step, "embedding_output", None)
            if rows is None:
                raise RuntimeError("the embedding of this model does not keep its output for later passes")
        with profile_stage("restart"):
            K.add_rows_vector(resid, rows, self.vec)
