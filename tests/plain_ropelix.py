"""A plain, slow implementation of the Ropelix decoder: whole sequences, float64, one function per mechanism,
written from the design's equations and sharing no code with the package.

``rnd`` is a hook that the caller may set to a rounding function (for instance to bfloat16 and back): it is applied
where a narrower run rounds (the operands of matrix products), so that two runs with and without it estimate that
run's rounding noise.  Everything that the design computes in 32-bit is left alone.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F = torch.float64
Round = Optional[Callable[[torch.Tensor], torch.Tensor]]


def _r(x: torch.Tensor, rnd: Round) -> torch.Tensor:
    return x if rnd is None else rnd(x)


def _lin(x: torch.Tensor, w: torch.Tensor, rnd: Round, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = _r(x, rnd) @ w.to(F).T
    return y if b is None else y + b.to(F)


# ---- small functions -------------------------------------------------------------------------------------------
def rms_norm(x, w, eps, one_plus: bool = False):
    """x / sqrt(mean(x^2) + eps) over the last dimension, times w (or 1 + w)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * ((1.0 + w.to(F)) if one_plus else w.to(F))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x, taps, bias=None):
    """x [T, C], taps [C, K] with the last column the current token's; zeros before the start; no activation."""
    T, C = x.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=F), x], dim=0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(K):
        y = y + pad[j:j + T] * taps.to(F)[:, j][None, :]
    return y if bias is None else y + bias.to(F)[None, :]


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: the first ``dims`` elements of every head turn, element i with i + dims/2, by
    positions * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = (positions.to(F)[:, None] * f[None, :])[:, None, :]
    cs, sn = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cs - v * sn, v * cs + u * sn, x[..., dims:]], dim=-1)


def window_mask(T: int, window: int):
    """seen[i, j]: 0 <= i - j (< window, if there is one)."""
    pos = torch.arange(T)
    i, j = pos[:, None], pos[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    return seen


# ---- softmax weights of grouped heads -----------------------------------------------------------------------------
def attention_weights(q, k, scale, positions=None, window=0, cap=0.0, bias=None, sink=False, rnd: Round = None):
    """q [N, H, d] at ``positions`` (None: 0 .. N-1) over the keys k [T, G, d] at positions 0 .. T-1 (head h reads
    key head h // (H / G)): weights [H, N, T].  score = (q . k) * scale; capped as cap tanh(score / cap) if cap > 0;
    minus bias[0]_h ln(1 + bias[1]_h (i - j)) if there is a bias; key j is seen from i if 0 <= i - j (< window, if
    there is one); softmax over the seen keys, with ``sink`` one more term exp(0) in the denominator."""
    N, H, _ = q.shape
    T, G, _ = k.shape
    pos = torch.arange(N) if positions is None else torch.as_tensor(positions)
    kv_of = torch.arange(H) // (H // G)
    s = torch.einsum("nhd,shd->hns", _r(q, rnd), _r(k, rnd)[:, kv_of]) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    dist = pos[:, None] - torch.arange(T)[None, :]
    if bias is not None:
        r1, r2 = bias[0].to(F)[:, None, None], bias[1].to(F)[:, None, None]
        s = s - r1 * torch.log1p(r2 * dist.clamp(min=0).to(F)[None])
    seen = dist >= 0
    if window:
        seen = seen & (dist < window)
    s = s.masked_fill(~seen[None], -math.inf)
    mx = s.max(-1).values
    if sink:
        mx = torch.clamp(mx, min=0.0)
    e = torch.exp(s - mx[..., None])
    den = e.sum(-1)
    if sink:
        den = den + torch.exp(-mx)
    return e / den[..., None]


def apply_weights(w, v, rnd: Round = None):
    """w [H, N, T], v [T, G, dv]: every head's weighted sum of the values of its own key/value head, [N, H * dv]."""
    H, N, _ = w.shape
    G = v.shape[1]
    kv_of = torch.arange(H) // (H // G)
    return torch.einsum("hns,shd->nhd", w, _r(v, rnd)[:, kv_of]).reshape(N, -1)


def mix_heads(w, talk):
    """w'_h(i, j) = sum_g talk[h, g] w_g(i, j)."""
    return torch.einsum("hg,gns->hns", talk.to(F), w)


# ---- attention with mixed heads (the left side of a parallel mixer) ---------------------------------------------
def talking_attention(h, p: Dict[str, torch.Tensor], m: dict, eps: float, rnd: Round = None):
    """h [T, width] of one sequence from position 0.  Norm over the whole q and k projections, rotation of a part
    of every head, capped scores, window, softmax, then the heads' weights mixed by ``talk``; every head applies
    its mixed weights to the values of its own key/value head."""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms_norm(_lin(h, p["q"], rnd), p["q.norm"], eps).view(T, H, d)
    k = rms_norm(_lin(h, p["k"], rnd), p["k.norm"], eps).view(T, G, d)
    v = _lin(h, p["v"], rnd).view(T, G, vd)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = rotate_half(q, pos, rot["base"], rot["dims"])
    k = rotate_half(k, pos, rot["base"], rot["dims"])
    w = attention_weights(q, k, m["scale"], window=(m.get("mask") or {}).get("size", 0), cap=m.get("softcap") or 0.0, rnd=rnd)
    if "talk" in p:
        w = mix_heads(w, p["talk"])
    return _lin(apply_weights(w, v, rnd), p["o"], rnd)


# ---- the recurrent block with a real-gated linear recurrent unit (the right side) -------------------------------
def gated_recurrence(u, r_gate, i_gate, lam, c: float = 8.0):
    """u, r_gate, i_gate [T, C]: log a = -c r softplus(lam); S_t = a S_(t-1) + sqrt(1 - a^2) i u from S = 0."""
    T, C = u.shape
    S = torch.zeros(C, dtype=F)
    out = torch.zeros(T, C, dtype=F)
    sp = softplus(lam.to(F))
    for t in range(T):
        log_a = -c * r_gate[t] * sp
        a = torch.exp(log_a)
        S = a * S + torch.sqrt(1.0 - a * a) * i_gate[t] * u[t]
        out[t] = S
    return out


def block_gates(u, w, b):
    """u [T, C] cut into w.shape[0] equal parts; part n is multiplied by the square matrix w[n] ([out, in]) and b[n] added."""
    T, C = u.shape
    nb = w.shape[0]
    ub = u.view(T, nb, C // nb)
    return (torch.einsum("tbi,boi->tbo", ub, w.to(F)) + b.to(F)[None]).reshape(T, C)


def recurrent_block(h, p: Dict[str, torch.Tensor], m: dict, rnd: Round = None):
    y = gelu_tanh(_lin(h, p["y"], rnd, p["y.b"]))
    u = causal_conv(_lin(h, p["x"], rnd, p["x.b"]), p["conv"], p["conv.b"])
    r = torch.sigmoid(block_gates(u, p["ra"], p["ra.b"]))
    i = torch.sigmoid(block_gates(u, p["ri"], p["ri.b"]))
    S = gated_recurrence(u, r, i, p["lam"])
    return _lin(S * y, p["o"], rnd)


def parallel_mixer(h, p, m, eps, rnd: Round = None):
    left = talking_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, m["left"], eps, rnd)
    right = recurrent_block(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, m["right"], rnd)
    return m["left_scale"] * left + m["right_scale"] * right


# ---- attention with convolved q and k, values = keys, a distance bias and a sink --------------------------------
def distance_attention(h, p: Dict[str, torch.Tensor], m: dict, rnd: Round = None):
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(_lin(h, p["q"], rnd), p["q.conv"]).view(T, H, d)
    k = causal_conv(_lin(h, p["k"], rnd), p["k.conv"]).view(T, G, d)
    w = attention_weights(q, k, m["scale"], window=(m.get("mask") or {}).get("size", 0), bias=(p["r1"], p["r2"]), sink=True,
                          rnd=rnd)
    o = apply_weights(w, k[..., :vd], rnd) * torch.sigmoid(_lin(h, p["g"], rnd))
    return _lin(o, p["o"], rnd)


# ---- gated delta rule with one decay per head -------------------------------------------------------------------
def delta_rule(q, k, v, beta, g):
    """q, k [T, H, dk]; v [T, H, dv]; beta, g [T, H].  Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def unit(x, eps: float = 1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def head_decay(a, dt_bias, a_log):
    """g = exp(-exp(A_log) softplus(a + dt_bias)), one a head."""
    return torch.exp(-torch.exp(a_log.to(F)) * softplus(a + dt_bias.to(F)))


def delta_mixer(h, p: Dict[str, torch.Tensor], m: dict, eps: float, rnd: Round = None):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(_lin(h, p["q"], rnd), p["q.conv"])).view(T, G, dk)
    k = silu(causal_conv(_lin(h, p["k"], rnd), p["k.conv"])).view(T, G, dk)
    v = silu(causal_conv(_lin(h, p["v"], rnd), p["v.conv"])).view(T, H, dv)
    q, k = unit(q) * dk ** -0.5, unit(k)
    kv_of = torch.arange(H) // (H // G)
    beta = torch.sigmoid(_lin(h, p["b"], rnd))
    g = head_decay(_lin(h, p["a"], rnd), p["dt_bias"], p["A_log"])
    o = delta_rule(q[:, kv_of], k[:, kv_of], v, beta, g)
    o = rms_norm(o, p["norm"], eps) * silu(_lin(h, p["g"], rnd)).view(T, H, dv)
    return _lin(o.reshape(T, H * dv), p["o"], rnd)


# ---- feed-forward -------------------------------------------------------------------------------------------------
def clamped_glu(h, p: Dict[str, torch.Tensor], mlp: dict, rnd: Round = None):
    lim = mlp["limit"]
    g = torch.clamp(_lin(h, p["gate"], rnd), max=lim)
    u = torch.clamp(_lin(h, p["up"], rnd), min=-lim, max=lim)
    return _lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), p["down"], rnd)


# ---- the model ----------------------------------------------------------------------------------------------------
def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(h, layer: dict, p, eps, rnd: Round = None):
    kind = layer["type"]
    if kind == "parallel":
        return parallel_mixer(h, p, layer["mixer"], eps, rnd)
    if kind == "attention":
        return distance_attention(h, p, layer["mixer"], rnd)
    if kind == "delta":
        return delta_mixer(h, p, layer["mixer"], eps, rnd)
    raise ValueError(kind)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], rnd: Round = None, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the stream after
    every layer."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    E = weights["embed"].to(F)
    x = E[torch.tensor(list(tokens))] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        w = _sub(weights, f"l{i}.")
        h = rms_norm(x, w["norm1"], eps, one_plus=True)
        x = x + mult * w["ls1"].to(F) * mixer(h, layer, _sub(w, "mix."), eps, rnd)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w["norm2"], eps, one_plus=True)
            x = x + mult * w["ls2"].to(F) * clamped_glu(h, _sub(w, "mlp."), layer["mlp"], rnd)
        if layers_out is not None:
            layers_out.append(x.clone())
    f = rms_norm(x, weights["final.norm"], eps, one_plus=True)
    return _r(f, rnd) @ E.T


def greedy(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], n: int) -> List[int]:
    """The n tokens that follow ``tokens`` when the largest logit is taken each time (the whole sequence is run
    again for every token: the slow form)."""
    seq, out = list(tokens), []
    for _ in range(n):
        t = int(forward(cfg, weights, seq)[-1].argmax())
        seq.append(t)
        out.append(t)
    return out
