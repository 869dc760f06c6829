"""A plain, slow implementation of the Puzorax decoder: whole sequences, float64, one function per mechanism,
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


def _lin(x: torch.Tensor, w: torch.Tensor, rnd: Round) -> torch.Tensor:
    return _r(x, rnd) @ w.to(F).T


# ---- norms ---------------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(F) + b.to(F)


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(F)


# ---- embedding -----------------------------------------------------------------------------------------------
def bigram_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """The row of the bigram table for every token of a sequence: a hash of (previous, current), or the table's
    last row for the first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embedding(tokens, embed, bigram, cfg):
    bg = cfg["embedding"]["bigram"]
    rows = bigram_rows(list(tokens), bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    return embed.to(F)[torch.tensor(list(tokens))] + bigram.to(F)[torch.tensor(rows)]


# ---- rotation ------------------------------------------------------------------------------------------------
def rotate_half(x, positions, base, dims):
    """x [T, ..., d]: the first ``dims`` elements turn, element i with i + dims/2, by positions * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = positions.to(F)[:, None] * f[None, :]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    cs, sn = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cs - v * sn, v * cs + u * sn, x[..., dims:]], dim=-1)


# ---- latent attention ----------------------------------------------------------------------------------------
def latent_attention(h, p: Dict[str, torch.Tensor], m: dict, eps: float, rnd: Round = None):
    """h [T, width] of one sequence from position 0.  Keys and values are rebuilt from the latent row per head
    (nothing is folded into the queries): the slow form."""
    T = h.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = _lin(h, p["q"], rnd).view(T, H, dim + rd)
    dkv = _lin(h, p["dkv"], rnd)
    c = rms_norm(dkv[:, :rank], p["dkv.norm"], eps)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    k_rot = rotate_half(dkv[:, rank:], pos, rot["base"], rot["dims"])                    # [T, rd], one for all heads
    q_rot = rotate_half(q[..., dim:], pos, rot["base"], rot["dims"])
    k_un = _lin(c, p["uk"], rnd).view(T, H, dim)
    v = _lin(c, p["uv"], rnd).view(T, H, vd)
    s = torch.einsum("thd,shd->hts", _r(q[..., :dim], rnd), _r(k_un, rnd)) + torch.einsum("thd,sd->hts", _r(q_rot, rnd), _r(k_rot, rnd))
    s = s * m["scale"]
    i, j = pos[:, None], pos[None, :]
    window = (m.get("mask") or {}).get("size", 0)
    seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
    s = s.masked_fill(~seen[None], -math.inf)
    sink = p["sink"].to(F)                                                               # [H]
    mx = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - mx[..., None])
    den = e.sum(-1) + torch.exp(sink[:, None] - mx)
    w = e / den[..., None]
    o = torch.einsum("hts,shd->thd", _r(w, rnd), _r(v, rnd)).reshape(T, H * vd)
    o = o * torch.sigmoid(_lin(h, p["g"], rnd))
    return _lin(o, p["o"], rnd)


# ---- gated delta rule with a decay per key channel -------------------------------------------------------------
def causal_conv_silu(x, taps):
    """x [T, C], taps [C, K] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=F), x], dim=0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(K):
        y = y + pad[j:j + T] * taps.to(F)[:, j][None, :]
    return y * torch.sigmoid(y)


def delta_rule(q, k, v, beta, g):
    """q, k, g [T, H, dk]; v [T, H, dv]; beta [T, H].  Per head: S <- diag(g) S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * g[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def channel_delta(h, p: Dict[str, torch.Tensor], m: dict, eps: float, rnd: Round = None):
    T = h.shape[0]
    H, KV, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(_lin(h, p["q"], rnd), p["q.conv"]).view(T, KV, dk)
    k = causal_conv_silu(_lin(h, p["k"], rnd), p["k.conv"]).view(T, KV, dk)
    v = causal_conv_silu(_lin(h, p["v"], rnd), p["v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // KV
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(_lin(h, p["b"], rnd))                                            # [T, H]
    a = _lin(_lin(h, p["a1"], rnd), p["a2"], rnd) + p["dt_bias"].to(F)
    g = torch.exp(-torch.exp(p["A_log"].to(F))[None, :, None] * torch.nn.functional.softplus(a).view(T, H, dk))
    o = delta_rule(q, k, v, beta, g)
    o = rms_norm(o, p["norm"], eps)
    o = o.reshape(T, H * dv) * torch.sigmoid(_lin(_lin(h, p["g1"], rnd), p["g2"], rnd))
    return _lin(o, p["o"], rnd)


# ---- mixture of experts ----------------------------------------------------------------------------------------
def route(z, correction, top, scale, margins: Optional[list] = None):
    """z [T, E]: scores softmax(z); the ``top`` largest of score + correction are chosen; their weights are
    the scores themselves over their sum, times ``scale``.  Returns a dense [T, E] matrix of weights.
    ``margins``: a list that gets, per token, how far the last chosen entry lies above the first one left out."""
    s = torch.softmax(z, dim=-1)
    pick = torch.topk(s + correction.to(F), top, dim=-1).indices
    if margins is not None and top < s.shape[-1]:
        ranked = torch.sort(s + correction.to(F), dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top])
    w = torch.gather(s, 1, pick)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * scale
    return torch.zeros_like(s).scatter(1, pick, w)


def moe(h, p: Dict[str, torch.Tensor], mlp: dict, rnd: Round = None, margins: Optional[list] = None):
    r = mlp["router"]
    E, I = r["experts"], r.get("identity", 0)
    dense = route(_lin(h, p["router"], rnd), p["correction"], r["top"], r["scale"], margins)
    y = torch.zeros_like(h)
    for e in range(E):
        a = _lin(h, p[f"e{e}.gate"], rnd)
        act = a * torch.sigmoid(a) * _lin(h, p[f"e{e}.up"], rnd)
        y = y + dense[:, e:e + 1] * _lin(act, p[f"e{e}.down"], rnd)
    for e in range(E, E + I):
        y = y + dense[:, e:e + 1] * _r(h, rnd)
    return y


# ---- the model -------------------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer(x, i: int, tensors, cfg, rnd: Round = None, margins: Optional[list] = None):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    h = layer_norm(x, tensors[f"l{i}.norm1"], tensors[f"l{i}.norm1.b"], eps)
    mix = sub(tensors, f"l{i}.mix.")
    if L["type"] == "latent_attention":
        y = latent_attention(h, mix, L["mixer"], eps, rnd)
    elif L["type"] == "channel_delta":
        y = channel_delta(h, mix, L["mixer"], eps, rnd)
    else:
        raise ValueError(L["type"])
    if L.get("mlp") is not None:
        y = y + moe(h, sub(tensors, f"l{i}.mlp."), L["mlp"], rnd, margins)
    return x + y


def layer_runs(cfg) -> List[tuple]:
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def forward(tokens, tensors, cfg, rnd: Round = None, keep_layers: bool = False, margins: Optional[list] = None):
    """Logits [T, vocab] of one sequence from its first token; with ``keep_layers`` also the stream after every
    layer run; ``margins`` collects the routers' margins (see ``route``)."""
    x0 = embedding(tokens, tensors["embed"], tensors["bigram"], cfg)
    x = x0
    kept = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + tensors["loop.step"].to(F)[t]
        x = layer(x, i, tensors, cfg, rnd, margins)
        if keep_layers:
            kept.append(x)
    f = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], cfg["norm"]["eps"])
    logits = _lin(f, tensors["head"], rnd)
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy(tokens, tensors, cfg, n_new: int) -> List[int]:
    """``n_new`` tokens, each the largest logit after everything before it (the whole sequence is run again)."""
    seq, out = list(tokens), []
    for _ in range(n_new):
        nxt = int(forward(seq, tensors, cfg)[-1].argmax())
        seq.append(nxt)
        out.append(nxt)
    return out
