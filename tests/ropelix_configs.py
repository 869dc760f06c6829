"""Small Ropelix configurations for the tests, the weights they run with, and the rounding-noise estimate.

The configurations differ from one another in every size, in the order of the layers and in which options are on:
heads of 8 to 64 elements (multiples of 16, which the tensor-core kernel of long steps takes, and sizes that are no
multiple of 8), one kv head for all heads, one for each, and groups; values narrower and wider than keys; a rotation
of a part of a head, of all of it, and none; capped and uncapped scores; windows smaller than a page, of one page
exactly, of more than two pages, and no window; recurrent blocks of one part and of several, of widths that are no
multiple of 32; 1 to 4 taps; layers without a feed-forward; a residual constant of 1; models without one or two of the
three mixers.  Weights are drawn by the library's random-weights writer with its "loud" distributions and then
sharpened where a fault would otherwise hide: decays slow and fast, a recurrence that remembers, a distance bias
of size one, mixing matrices far from the identity, norm weights and layer scales far from their defaults."""
import os

import torch
from safetensors.torch import load_file, save_file

from votavik_configs import assert_rows, prompts, read_folder, rel_rms, LIMIT_F32, NOISE_FACTOR  # noqa: F401  (generic helpers)


def _left(heads, kv_heads, dim, vdim, window, rot_dims, base, scale, softcap):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dims is not None:
        m["rot"] = {"dims": rot_dims, "base": base}
    if softcap:
        m["softcap"] = softcap
    return m


def _parallel(left, width, blocks, conv, left_scale, right_scale, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
                      "left_scale": left_scale, "right_scale": right_scale}}


def _attention(heads, kv_heads, dim, window, conv, scale, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# A: delta first; heads of 16 and 32 (the tensor-core kernel of long steps); a window of 10 (smaller than a page) and
#    one of 150 (more than two pages); six heads on three kv heads; values wider than keys; two parts of 24 channels
ROP_A = {"architecture": "Ropelix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
         "residual_mult": 0.8,
         "layers": [_delta(4, 2, 16, 8, 3, _dense(48, 1.0)),
                    _parallel(_left(6, 3, 16, 32, 10, 8, 100.0, 0.3, 5.0), 48, 2, 4, 0.7, 0.4, _dense(32, 2.0)),
                    _attention(4, 2, 32, 150, 2, 0.2, None),
                    _parallel(_left(2, 1, 32, 16, 150, 32, 5000.0, 0.2, 0.0), 40, 5, 2, 1.2, 0.9, _dense(40, 0.7))]}

# B: sizes that are no multiples of 8; one head; no rotation, no cap, no window (plain causal attention); a
#    convolution of one tap (no kept inputs); a recurrent block of one part; a residual constant of 1
ROP_B = {"architecture": "Ropelix", "vocab": 131, "width": 48, "norm": {"eps": 1e-3}, "embedding": {"scale": 1.0},
         "residual_mult": 1.0,
         "layers": [_attention(1, 1, 20, 0, 1, 0.25, _dense(20, 1.5)),
                    _parallel(_left(1, 1, 12, 20, 0, None, 0.0, 0.35, 0.0), 30, 1, 1, 1.0, 1.0, None),
                    _delta(1, 1, 20, 12, 1, None),
                    _attention(3, 3, 12, 7, 4, 0.4, _dense(24, 3.0))]}

# C: wider heads (keys of 64 and 48 on the tensor cores, a delta rule of 72 and 136 key channels), a window of one
#    page exactly, eight heads on two and on eight kv heads, a rotation of all of a head, 3 taps
ROP_C = {"architecture": "Ropelix", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.5},
         "residual_mult": 0.5,
         "layers": [_parallel(_left(8, 2, 64, 48, 64, 64, 30000.0, 0.11, 30.0), 96, 3, 3, 0.5, 0.65, _dense(64, 1.75)),
                    _delta(2, 1, 72, 40, 4, _dense(96, 1.2)),
                    _attention(8, 8, 48, 64, 3, 0.15, _dense(32, 2.5)),
                    _delta(1, 1, 136, 17, 2, None),
                    _parallel(_left(4, 4, 16, 16, 70, 4, 50.0, 0.25, 0.0), 64, 64, 4, 0.9, 0.3, None)]}

# D: no attention of either kind with a cache of pages but the left sides' (a model of recurrent layers mostly);
#    a window of 1 (a token sees itself only)
ROP_D = {"architecture": "Ropelix", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
         "residual_mult": 1.3,
         "layers": [_delta(2, 2, 16, 8, 3, _dense(16, 1.0)),
                    _parallel(_left(2, 1, 8, 8, 1, 2, 10.0, 0.5, 2.0), 24, 3, 2, 0.2, 1.5, _dense(24, 1.0)),
                    _delta(4, 1, 8, 8, 4, _dense(24, 0.5))]}

# E: the attention with convolved keys first; eight heads on four kv heads beside a recurrence of four parts; heads of
#    80 without a window; windows of 48, 100 and 300; a rotation of no element; long prompts run on it
ROP_E = {"architecture": "Ropelix", "vocab": 311, "width": 192, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
         "residual_mult": 0.6,
         "layers": [_attention(6, 2, 32, 100, 4, 0.18, _dense(160, 2.0)),
                    _parallel(_left(8, 4, 32, 64, 48, 16, 10000.0, 0.18, 40.0), 96, 4, 2, 0.8, 0.7, _dense(224, 1.5)),
                    _delta(4, 4, 64, 32, 2, _dense(96, 4.0)),
                    _attention(2, 1, 80, 0, 2, 0.11, None),
                    _parallel(_left(3, 3, 48, 48, 300, 0, 0.0, 0.14, 0.0), 120, 3, 3, 0.4, 1.1, _dense(64, 1.0))]}

CONFIGS = {"A": (ROP_A, 41), "B": (ROP_B, 42), "C": (ROP_C, 43), "D": (ROP_D, 44)}


def sharpen(weights, cfg, seed):
    """Values of size one where the random-weights writer draws small ones."""
    gen = torch.Generator().manual_seed(seed)
    out = dict(weights)

    def rand(shape):
        return torch.randn(shape, generator=gen)

    def unif(shape, lo, hi):
        return lo + (hi - lo) * torch.rand(shape, generator=gen)
    for name, w in weights.items():
        if name.endswith(".A_log"):           # decays from e^-0.02 dt to e^-dt
            out[name] = torch.log(0.02 + 0.98 * torch.rand(w.shape, generator=gen)).to(w.dtype)
        elif name.endswith(".dt_bias"):
            out[name] = (-1.0 + rand(w.shape)).to(w.dtype)
        elif name.endswith(".lam"):           # a = exp(-8 r softplus(lam)) between about 0.5 and 0.99 at r = 1/2
            out[name] = unif(w.shape, -6.0, -1.5).to(w.dtype)
        elif name.endswith(".r1"):
            out[name] = unif(w.shape, 0.3, 1.5).to(w.dtype)
        elif name.endswith(".r2"):
            out[name] = unif(w.shape, 0.05, 2.0).to(w.dtype)
        elif name.endswith(".talk"):
            out[name] = (torch.eye(w.shape[0]) + 0.4 * rand(w.shape)).to(w.dtype)
        elif name.endswith((".norm1", ".norm2")) or name == "final.norm":
            out[name] = (0.3 * rand(w.shape)).to(w.dtype)
        elif name.endswith((".ls1", ".ls2")):
            out[name] = unif(w.shape, 0.3, 1.2).to(w.dtype)
    return out


def write_ropelix(tmpdir, cfg, seed, store="bfloat16", change=None, tag=""):
    """A model folder for ``cfg``: loud random weights, sharpened; ``change(weights) -> weights`` edits them."""
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"ropelix_s{seed}_{store}{tag}")
    if os.path.isdir(d):
        return d
    write_random_model(d, cfg, seed, store, "loud")
    path = os.path.join(d, "model.safetensors")
    weights = sharpen(load_file(path), cfg, seed)
    if change is not None:
        weights = change(weights)
    save_file({k: v.contiguous() for k, v in weights.items()}, path)
    return d


def round_to(dtype):
    return lambda x: x.to(dtype).to(torch.float64)


def noise(cfg, weights, tokens, want, dtype=torch.bfloat16):
    """What rounding alone does to each row of the logits in a run of ``dtype``, on ``rel_rms``'s scale, and never
    less than twice the median of that over the rows.  Two samples of every row's sensitivity are taken, the plain
    implementation with the operands of its products rounded to float32 and to bfloat16 (whose unit is 2^15 times
    larger), and the larger one counts."""
    import plain_ropelix as P
    in32 = rel_rms(P.forward(cfg, weights, list(tokens), rnd=round_to(torch.float32)), want)
    in16 = rel_rms(P.forward(cfg, weights, list(tokens), rnd=round_to(torch.bfloat16)), want)
    if dtype == torch.float32:
        own, other = in32, in16 * 2.0 ** -15
    else:
        own, other = in16, (in32 * 2.0 ** 15).clamp(max=1.0)
    return torch.maximum(torch.maximum(own, other), 2.0 * own.median())
