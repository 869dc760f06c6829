"""Small Puzorax configurations for the tests, the weights they run with, and the rounding-noise estimate.

The configurations differ from one another in every size, in the order of the layers and in which options are on:
latent sizes of 24 to 72, one head and ten heads (more than a block of the attention kernel takes), a rotation of
the whole rotated part, of a part of it, and no rotated part at all, windows smaller than a page, of one page
exactly, of more than two pages and no window, delta-rule layers with one and several q/k heads a value head, keys
and values that agree and differ in size, 1 to 4 taps, mixtures with and without identity experts, 1 to 3 chosen,
layers without a feed-forward, a repeated run of layers at the start, in the middle and at the end of the model,
walked once, twice and three times, and no repeated run.  Weights are drawn by the library's random-weights writer
with its "loud" distributions and then sharpened where a fault would otherwise hide: decays slow and fast, sinks and
corrections of size one, loud vectors between the passes."""
import json
import os

import torch
from safetensors.torch import load_file, save_file

from votavik_configs import assert_rows, prompts, read_folder, rel_rms, LIMIT_F32, NOISE_FACTOR  # noqa: F401  (generic helpers)


def _latent(heads, dim, rot_dim, vdim, rank, window, rot_dims, base, scale, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dim:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, mlp=None):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                      "decay_rank": decay_rank, "gate_rank": gate_rank}}


def _moe(experts, identity, ff, top, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}


def _bigram(buckets, mul_prev, mul_cur):
    return {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


# A: the delta rule first; the last two layers are walked three times; a window of 10 (smaller than a page); ten
#    heads; a rotation of 8 of the 12 rotated elements; two q/k heads for four value heads
PUZ_A = {"architecture": "Puzorax", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": _bigram(53, 5, 3),
         "loop": {"start": 1, "stop": 3, "times": 3},
         "layers": [_delta(4, 2, 16, 8, 3, 6, 10, _moe(6, 1, 24, 2, 1.5)),
                    _latent(10, 8, 12, 6, 24, 10, 8, 100.0, 0.3, _moe(5, 3, 16, 3, 0.7)),
                    _delta(2, 2, 24, 24, 2, 4, 4, None)]}

# B: one head everywhere, sizes that are no multiples of 8, no rotated part, no window (plain causal attention), no
#    identity experts, one expert chosen, a convolution of one tap (no kept inputs), no repeated run
PUZ_B = {"architecture": "Puzorax", "vocab": 131, "width": 48, "norm": {"eps": 1e-3}, "embedding": _bigram(17, 1, 1),
         "layers": [_latent(1, 20, 0, 20, 36, 0, 0, 0.0, 0.25, _moe(5, 0, 20, 1, 1.0)),
                    _delta(1, 1, 20, 12, 1, 3, 5, None),
                    _latent(3, 4, 6, 10, 40, 70, 6, 10000.0, 0.4, None)]}

# C: wider heads (keys of 72 and 136: more than 64 and 128 channels a thread group), a window of one page exactly
#    and one of more than two pages, values wider than keys, the first two layers walked twice, a latent of 72
PUZ_C = {"architecture": "Puzorax", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "embedding": _bigram(1009, 131, 17),
         "loop": {"start": 0, "stop": 2, "times": 2},
         "layers": [_latent(4, 32, 16, 40, 72, 64, 16, 500.0, 0.15, _moe(8, 2, 32, 2, 2.0)),
                    _delta(2, 1, 72, 40, 4, 16, 8, _moe(4, 1, 48, 3, 1.0)),
                    _delta(1, 1, 136, 17, 2, 8, 16, None),
                    _latent(2, 64, 32, 32, 64, 150, 32, 50000.0, 0.125, _moe(6, 0, 16, 2, 3.0))]}

# D: no attention layer at all (a cache without pages: states only); one pass over a "repeated" run (the vector of
#    the pass is still added)
PUZ_D = {"architecture": "Puzorax", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "embedding": _bigram(7, 2, 9),
         "loop": {"start": 1, "stop": 2, "times": 1},
         "layers": [_delta(2, 2, 16, 8, 3, 4, 4, _moe(4, 2, 16, 2, 2.5)),
                    _delta(4, 1, 8, 8, 4, 2, 6, _moe(3, 1, 24, 4, 1.0))]}

CONFIGS = {"A": (PUZ_A, 31), "B": (PUZ_B, 32), "C": (PUZ_C, 33), "D": (PUZ_D, 34)}

ROUTE_PUSH = 6.0


def route_direction(cfg, seed):
    """The unit vector of the stream that "two_way" routers read."""
    u = torch.randn(cfg["width"], generator=torch.Generator().manual_seed(1000 + seed))
    return u / u.norm()


def token_sign(vocab):
    """+1 or -1 for every token id, changing every three ids."""
    return 1.0 - 2.0 * ((torch.arange(vocab) // 3) % 2)


def sharpen(weights, cfg, seed, router="random"):
    """Values of size one where the random-weights writer draws small ones.  ``router`` = "random" leaves the
    routers' rows as drawn.  "two_way": every router's rows are multiples of ONE direction u of the stream, with
    unevenly spaced factors, and the token embedding carries ``ROUTE_PUSH`` u with a sign that depends on the token
    id: u . h stays far from zero in every layer, so the order of the scores depends on its sign only, and a
    bfloat16 run (whose activations carry a relative noise of 2^-9) chooses the experts that the plain
    implementation chooses, while tokens still take one of two routes.  The corrections are small beside the
    scores' gaps there."""
    gen = torch.Generator().manual_seed(seed)
    out = dict(weights)
    u = route_direction(cfg, seed)

    def rand(shape):
        return torch.randn(shape, generator=gen)
    if router == "two_way":
        emb = weights["embed"].float()
        out["embed"] = (emb + ROUTE_PUSH * token_sign(emb.shape[0])[:, None] * u[None, :]).to(weights["embed"].dtype)
    for name, w in weights.items():
        if name.endswith(".A_log"):           # decays from e^-0.02 dt to e^-dt
            out[name] = torch.log(0.02 + 0.98 * torch.rand(w.shape, generator=gen)).to(w.dtype)
        elif name.endswith(".dt_bias"):
            out[name] = (-1.0 + rand(w.shape)).to(w.dtype)
        elif name.endswith(".sink"):          # sinks that take a share of the softmax
            out[name] = (1.0 + rand(w.shape)).to(w.dtype)
        elif name == "loop.step":
            out[name] = rand(w.shape).to(w.dtype)
        elif name.endswith(".norm1.b") or name == "final.norm.b":
            out[name] = (0.5 * rand(w.shape)).to(w.dtype)
        elif name.endswith(".correction"):
            # "random": as large as the scores themselves (the choice differs from the largest scores);
            # "two_way": well below the gaps that the factors make
            out[name] = ((0.3 if router == "random" else 0.002) * rand(w.shape)).to(w.dtype)
        elif name.endswith(".router") and router == "two_way":
            E = w.shape[0]
            factors = (4.0 * torch.linspace(0.0, 1.0, E) ** 1.5 - 1.5)[torch.randperm(E, generator=gen)]
            out[name] = (factors[:, None] * (1.8 / ROUTE_PUSH) * u[None, :]).to(w.dtype)
    return out


def write_puzorax(tmpdir, cfg, seed, store="bfloat16", change=None, tag="", router="random"):
    """A model folder for ``cfg``: loud random weights, sharpened; ``change(weights) -> weights`` edits them."""
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"puzorax_s{seed}_{store}_{router}{tag}")
    if os.path.isdir(d):
        return d
    write_random_model(d, cfg, seed, store, "loud")
    path = os.path.join(d, "model.safetensors")
    weights = sharpen(load_file(path), cfg, seed, router)
    if change is not None:
        weights = change(weights)
    save_file({k: v.contiguous() for k, v in weights.items()}, path)
    return d


def router_for(dtype):
    return "random" if dtype in (torch.float32, "float32") else "two_way"


def round_to(dtype):
    return lambda x: x.to(dtype).to(torch.float64)


def noise(cfg, weights, tokens, want, dtype=torch.bfloat16):
    """What rounding alone does to each row of the logits in a run of ``dtype``, on ``rel_rms``'s scale, and never
    less than twice the median of that over the rows.  Two samples of every row's sensitivity are taken, the plain
    implementation with the operands of its products rounded to float32 and to bfloat16 (whose unit is 2^15 times
    larger), and the larger one counts."""
    import plain_puzorax as P
    in32 = rel_rms(P.forward(list(tokens), weights, cfg, rnd=round_to(torch.float32)), want)
    in16 = rel_rms(P.forward(list(tokens), weights, cfg, rnd=round_to(torch.bfloat16)), want)
    if dtype == torch.float32:
        own, other = in32, in16 * 2.0 ** -15
    else:
        own, other = in16, (in32 * 2.0 ** 15).clamp(max=1.0)
    return torch.maximum(torch.maximum(own, other), 2.0 * own.median())
