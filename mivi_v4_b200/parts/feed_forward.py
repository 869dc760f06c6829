"""Feed-forwards: the parts of a layer that work on each token alone."""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, linear_swiglu, norm_link_ok, tensor_core_ok
from .base import Part
from .registry import register
from .spec import ParamSpec


@register("feed_forward", "swiglu")
class SwiGLU(Part):
    """x + (silu(g W1^T) * (g W3^T)) W2^T without biases
    (crates/mivi-model/src/ffn.rs:56-108).  W1 and W3 are merged at load time
    so that one product yields gate and up: in alternating groups of 16 rows
    (16 of W1, then the 16 of W3 for the same features) when the width allows,
    which lets the tensor-core kernels apply the activation in their
    epilogue; else end to end."""

    overwrites = True            # forward(..., accumulate=False) writes its result instead of adding it

    def __init__(self, hidden: int, ff: int):
        self.hidden, self.ff = int(hidden), int(ff)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, F = self.hidden, self.ff
        return {"w1.weight": ParamSpec((F, H)), "w3.weight": ParamSpec((F, H)), "w2.weight": ParamSpec((H, F))}

    def load(self, t) -> None:
        w1, w3 = t["w1.weight"], t["w3.weight"]
        if w1.dtype != w3.dtype:
            w1, w3 = w1.float(), w3.float()
        G = K.SWIGLU_GROUP
        self.group = G if self.ff % G == 0 else 0
        if self.group:
            F, H = w1.shape
            self.w13 = torch.stack([w1.view(F // G, G, H), w3.view(F // G, G, H)], dim=1).reshape(2 * F, H).contiguous()
        else:
            self.w13 = torch.cat([w1, w3], dim=0).contiguous()
        self.w2 = t["w2.weight"]

    def carries_norm(self, step):
        n = step.n_tokens
        return (bool(self.group) and norm_link_ok(n, self.w13, step.dtype)), norm_link_ok(n, self.w2, step.dtype, emits=True)

    def forward(self, g, resid, step, scale=None, emit=None, accumulate: bool = True) -> None:
        N = g.shape[0]
        h = self.scratch(step, "ffh", (N, self.ff), step.dtype)
        if self.group and tensor_core_ok(g, self.w13):
            linear_swiglu(g, self.w13, h, scale=scale)
        else:
            gu = self.scratch(step, "proj", (N, 2 * self.ff), torch.float32)
            linear(g, self.w13, gu, scale=scale)
            K.swiglu(gu, h, self.group)
        linear(h, self.w2, resid, accumulate=accumulate, emit=emit)


@register("feed_forward", "clamped_glu")
class ClampedGLU(Part):
    """x + (g * sigmoid(alpha g) * (u + 1)) W_down^T with g = min(h W_gate^T, limit) and
    u = clamp(h W_up^T, -limit, limit); no biases.  ``alpha`` is the constant of the sigmoid approximation of
    gelu (1.702).  Gate and up are one product (the two matrices end to end); the activation is computed in
    float32 from its float32 results."""

    overwrites = True            # forward(..., accumulate=False) writes its result instead of adding it

    def __init__(self, hidden: int, ff: int, limit: float, alpha: float = 1.702):
        self.hidden, self.ff, self.limit, self.alpha = int(hidden), int(ff), float(limit), float(alpha)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, F = self.hidden, self.ff
        return {"gate": ParamSpec((F, H)), "up": ParamSpec((F, H)), "down": ParamSpec((H, F))}

    def load(self, t) -> None:
        wg, wu = t["gate"], t["up"]
        if wg.dtype != wu.dtype:
            wg, wu = wg.float(), wu.float()
        self.w_gu = torch.cat([wg, wu], dim=0).contiguous()
        self.w_down = t["down"]

    def forward(self, g, resid, step, accumulate: bool = True) -> None:
        N = g.shape[0]
        gu = self.scratch(step, "proj", (N, 2 * self.ff), torch.float32)
        linear(g, self.w_gu, gu)
        h = self.scratch(step, "ffh", (N, self.ff), step.dtype)
        K.glu_clamped(gu, h, self.limit, self.alpha)
        linear(h, self.w_down, resid, accumulate=accumulate)


@register("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """Mixture of experts: every expert is W_down (silu(W_gate h) * (W_up h)) without
    biases; router logits z = W_router h in float32, scores s = sigmoid(z), or with ``score`` "softmax" softmax(z)
    over all routed entries; with ``correction`` a learned number per entry is added to the scores for the CHOICE
    only (the weights use the scores themselves); the weights are multiplied by ``out_scale``; the last
    ``n_identity`` routed entries (after the ``n_experts`` experts with matrices) are identity experts whose output
    is the input itself times the weight.  The entries form ``n_groups`` equal
    groups of neighbours, a group's score is the sum of its two largest scores, and only experts of the
    ``keep_groups`` best groups can be chosen; the ``top`` largest scores among them are chosen and weigh their
    experts by s / (sum of the chosen s + 1e-20).  With ``shared_ff`` > 0 a shared expert of that width runs for
    every token and is added times sigmoid(w_sg . h).

    All experts' gate and up matrices are laid end to end (the shared expert's last), so that one product yields
    every expert's pre-activations; the gated activation is multiplied by the router's weight before it is
    rounded (zero where an expert was not chosen: nothing is computed there), and one product with the down
    matrices side by side sums the chosen experts.  Long bfloat16 steps instead sort the (token, choice) entries by
    expert on the device and run grouped products over the sorted rows, so every expert multiplies its own tokens
    only.  No decision is taken on the host."""

    overwrites = True

    SCORES = {"sigmoid": K.ROUTE_SIGMOID, "softmax": K.ROUTE_SOFTMAX}

    def __init__(self, hidden: int, n_experts: int, ff: int, top: int, n_groups: int = 1, keep_groups: int = 1,
                 shared_ff: int = 0, score: str = "sigmoid", correction: bool = False, out_scale: float = 1.0,
                 n_identity: int = 0):
        routed = int(n_experts) + int(n_identity)
        if n_experts < 1 or n_identity < 0 or routed > K.MAX_EXPERTS or n_groups < 1 or routed % n_groups:
            raise ValueError(f"{routed} routed entries do not form {n_groups} equal groups (at most {K.MAX_EXPERTS})")
        if not 1 <= keep_groups <= n_groups or not 1 <= top <= min(32, keep_groups * (routed // n_groups)):
            raise ValueError(f"{top} experts cannot be chosen from {keep_groups} of {n_groups} groups of "
                             f"{routed // n_groups} (at most 32)")
        if score not in self.SCORES:
            raise ValueError(f"router score {score!r}; known: {', '.join(sorted(self.SCORES))}")
        self.hidden, self.E, self.ff, self.top = int(hidden), int(n_experts), int(ff), int(top)
        self.n_groups, self.keep, self.shared_ff = int(n_groups), int(keep_groups), int(shared_ff)
        self.score, self.has_correction, self.out_scale = score, bool(correction), float(out_scale)
        self.I, self.routed = int(n_identity), routed

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, F = self.hidden, self.ff
        specs = {"router": ParamSpec((self.routed, H))}
        if self.has_correction:
            specs["correction"] = ParamSpec((self.routed,), "vector", "bias")
        for e in range(self.E):
            specs.update({f"e{e}.gate": ParamSpec((F, H)), f"e{e}.up": ParamSpec((F, H)), f"e{e}.down": ParamSpec((H, F))})
        if self.shared_ff:
            S = self.shared_ff
            specs.update({"shared.gate": ParamSpec((S, H)), "shared.up": ParamSpec((S, H)), "shared.down": ParamSpec((H, S)),
                          "shared.sg": ParamSpec((1, H))})
        return specs

    def active_matrix_elements(self) -> int:
        """Matrix elements that one token is multiplied with: the router, its chosen experts, the shared one."""
        H = self.hidden
        return self.routed * H + 3 * self.top * self.ff * H + (3 * self.shared_ff * H + H if self.shared_ff else 0)

    def load(self, t) -> None:
        names = [f"e{e}." for e in range(self.E)] + (["shared."] if self.shared_ff else [])
        mats = [t[n + "gate"] for n in names] + [t[n + "up"] for n in names] + [t[n + "down"] for n in names]
        if len({m.dtype for m in mats}) != 1:
            t = {k: v.float() for k, v in t.items()}
        G = K.SWIGLU_GROUP

        def gate_up(n, width):
            """An expert's gate and up rows together: alternating in groups of 16 where the width allows (the
            tensor-core products then apply the activation themselves), else the gates, then the ups."""
            wg, wu = t[n + "gate"], t[n + "up"]
            if width % G:
                return torch.cat([wg, wu], dim=0)
            H = wg.shape[1]
            return torch.stack([wg.view(width // G, G, H), wu.view(width // G, G, H)], dim=1).reshape(2 * width, H)
        self.group = G if self.ff % G == 0 else 0
        self.shared_group = G if self.shared_ff and self.shared_ff % G == 0 else 0
        self.w_gu = torch.cat([gate_up(n, self.shared_ff if n == "shared." else self.ff) for n in names], dim=0).contiguous()
        self.w_down = torch.cat([t[n + "down"] for n in names], dim=1).contiguous()
        rows = [t["router"]] + ([t["shared.sg"]] if self.shared_ff else [])
        pad = -sum(r.shape[0] for r in rows) % 16
        if pad:
            rows.append(torch.zeros((pad, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.correction = t.get("correction")
        # the shared expert's down matrix by itself, for the steps that sort the tokens by expert (kept in a list,
        # beside the weights that every step reads: a copy of columns that those steps read from it instead)
        self._shared_down = [self.w_down[:, self.E * self.ff:].contiguous()] if self.shared_ff else []

    # Steps that bring an expert this many rows on average (never a decode step) sort the (token, choice) entries
    # by expert and run ONE grouped product over the sorted rows for the experts' gate and up matrices and one for
    # their down matrices: every expert multiplies its own tokens only.  Shorter steps multiply every token with
    # every expert (three products whatever was chosen), which is what a step of few tokens wants anyway: it
    # streams the experts' matrices once, and nearly all of them are chosen by some token.  Measured with 16 experts
    # of which 4 are chosen (width 2,048, experts of 1,024): 256 tokens 5.2 ms a prefill sorted against 3.9, 512 tokens
    # 6.0 against 5.6, 1,024 tokens 9.4 against 9.6, 2,048 tokens 15.5 against 16.6: runs of fewer rows than two
    # tiles are mostly padding.
    SORTED_ROWS_AN_EXPERT = 256
    # steps of more rows than this let the first product gate its own results (and round them) before the router's
    # weights are put on them; shorter steps round once, after the weights
    GATED_IN_PRODUCT_FROM = 65

    def _sorted_ok(self, g, step, N: int) -> bool:
        return (N * self.top >= self.SORTED_ROWS_AN_EXPERT * self.E and not step.is_decode and self.top < self.E
                and self.I == 0 and self.group == K.SWIGLU_GROUP and self.ff % 8 == 0 and g.shape[1] % 8 == 0
                and tensor_core_ok(g, self.w_gu) and self.w_down.dtype == torch.bfloat16)

    def forward(self, g, resid, step, accumulate: bool = True) -> None:
        N = g.shape[0]
        E, F, I = self.E, self.E * self.ff + self.shared_ff, self.I
        sg = 1 if self.shared_ff else 0
        cols = self.routed + sg                  # a dense row: [experts | the shared gate | identity experts]
        z = self.scratch(step, "z", (N, self.w_router.shape[0]), torch.float32)
        linear(g, self.w_router, z)
        dense = self.scratch(step, "route", (N, cols), torch.float32)
        pick = self.scratch(step, "pick", (N, self.top), torch.int32)
        pick_w = self.scratch(step, "pick_w", (N, self.top), torch.float32)
        K.route(z[:, :cols], dense, pick, pick_w, self.routed, self.n_groups, self.keep, self.top, bool(self.shared_ff),
                mode=self.SCORES[self.score], correction=self.correction, out_scale=self.out_scale, n_identity=I)
        if self._sorted_ok(g, step, N):
            return self._forward_sorted(g, resid, step, accumulate, dense, pick, pick_w)
        h = self.scratch(step, "ffh", (N, F), step.dtype)
        if (N >= self.GATED_IN_PRODUCT_FROM and self.group and (self.shared_group or not self.shared_ff)
                and tensor_core_ok(g, self.w_gu)):
            # long steps: gate and up never reach memory; the weights go on the rounded activations
            linear_swiglu(g, self.w_gu, h)
            K.scale_expert_columns(h, dense, E, self.ff, self.shared_ff, extra_cols=I)
        else:
            gu = self.scratch(step, "proj", (N, 2 * F), torch.float32)
            linear(g, self.w_gu, gu)
            K.routed_glu(gu, dense, h, E, self.ff, self.shared_ff, self.group, self.shared_group, extra_cols=I)
        linear(h, self.w_down, resid, accumulate=accumulate)
        if I:
            K.identity_experts(g, dense, E + sg, I, resid)

    def _forward_sorted(self, g, resid, step, accumulate, dense, pick, pick_w) -> None:
        N, H = g.shape
        E, ff, top = self.E, self.ff, self.top
        tiles = K.grouped_tiles(N * top, E)
        rows = tiles * K.GROUPED_TILE_ROWS
        rank = self.scratch(step, "rank", (N * top,), torch.int32)
        counts = self.scratch(step, "counts", (E,), torch.int32)
        offsets = self.scratch(step, "offsets", (E,), torch.int32)
        tile_group = self.scratch(step, "tile_group", (tiles,), torch.int32)
        place = self.scratch(step, "place", (N * top,), torch.int32)
        xs = self.scratch(step, "sorted", (rows, H), g.dtype)
        K.expert_sort(pick, E, g, rank, counts, place, xs, offsets, tile_group)
        hs = self.scratch(step, "sorted_h", (rows, ff), step.dtype)
        K.gemm_tc_grouped(xs, self.w_gu, hs, tile_group, 2 * ff, H, row_step=2 * ff, swiglu=True, active_rows=N * top)
        ys = self.scratch(step, "sorted_y", (rows, H), torch.float32)
        K.gemm_tc_grouped(hs, self.w_down, ys, tile_group, H, ff, k_step=ff, active_rows=N * top)
        shared = None
        if self.shared_ff:
            hsh = self.scratch(step, "shared_h", (N, self.shared_ff), step.dtype)
            w_gu = self.w_gu[E * 2 * ff:]
            if self.shared_group and tensor_core_ok(g, w_gu):
                linear_swiglu(g, w_gu, hsh)
            else:
                gu = self.scratch(step, "proj", (N, w_gu.shape[0]), torch.float32)
                linear(g, w_gu, gu)
                K.swiglu(gu, hsh, self.shared_group)
            shared = self.scratch(step, "shared_y", (N, H), torch.float32)
            linear(hsh, self._shared_down[0], shared)
        # the shared expert's gate is the last column of the router's dense weights
        K.expert_combine(ys, place, pick_w, shared, dense[:, E:E + 1] if shared is not None else None, resid, accumulate)
