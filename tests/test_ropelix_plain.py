"""The plain Ropelix implementation against closed forms (no GPU), and the parts of the package that need no GPU:
the configuration reader, the name table, the cache's plan, and the command line."""
import json
import math

import pytest
import torch

import plain_ropelix as P
import ropelix_configs as RC
from ropelix_configs import CONFIGS, ROP_A, ROP_B, ROP_C, ROP_D, prompts, read_folder, rel_rms, write_ropelix

F64 = torch.float64


def _rand(seed):
    g = torch.Generator().manual_seed(seed)
    return lambda *s: torch.randn(*s, generator=g, dtype=F64)


def test_norm_with_a_weight_around_zero():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    y = P.rms_norm(x, torch.tensor([0.5, -1.0], dtype=F64), 0.0, one_plus=True)
    assert torch.allclose(y, torch.tensor([[3.0 / math.sqrt(12.5) * 1.5, 0.0]], dtype=F64))
    assert torch.allclose(P.rms_norm(x, torch.tensor([2.0, 1.0], dtype=F64), 0.0), x / math.sqrt(12.5) * torch.tensor([2.0, 1.0]))


def test_rotation_pairs_element_i_with_i_plus_half_of_the_turned_part():
    x = _rand(1)(3, 2, 12)
    y = P.rotate_half(x, torch.tensor([0, 5, 9]), 100.0, 8)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])          # position 0 and the part that passes
    a = 5 * 100.0 ** (-2 * 1 / 8)
    assert torch.allclose(y[1, :, 1], x[1, :, 1] * math.cos(a) - x[1, :, 5] * math.sin(a))
    assert torch.allclose(y[1, :, 5], x[1, :, 5] * math.cos(a) + x[1, :, 1] * math.sin(a))
    assert torch.equal(P.rotate_half(x, torch.tensor([1, 2, 3]), 100.0, 0), x)


def test_causal_taps_last_column_is_the_current_token_and_bias():
    x = torch.arange(1.0, 6.0, dtype=F64)[:, None]
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)
    assert P.causal_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    assert P.causal_conv(x, taps, torch.tensor([0.5], dtype=F64))[0, 0].item() == 1.5


def _left_weights(H, G, d, vd, W, seed=3):
    r = _rand(seed)
    return {"q": r(H * d, W), "k": r(G * d, W), "v": r(G * vd, W), "q.norm": 1.0 + 0.1 * r(H * d), "k.norm": 1.0 + 0.1 * r(G * d),
            "talk": torch.eye(H, dtype=F64) + 0.5 * r(H, H), "o": r(W, H * vd)}


def test_mixed_heads_window_edge_and_what_the_mixing_does():
    H, G, d, vd, W, T, win = 4, 2, 6, 5, 8, 12, 5
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": vd, "scale": 0.4, "softcap": 3.0, "mask": {"size": win},
         "rot": {"dims": 4, "base": 100.0}}
    p = _left_weights(H, G, d, vd, W)
    h = _rand(4)(T, W)
    base = P.talking_attention(h, p, m, 1e-6)
    # token i must not depend on token i - window, must depend on token i - window + 1
    for j in (3, 6):
        h2 = h.clone()
        h2[j] += 1.0
        moved = (P.talking_attention(h2, p, m, 1e-6) - base).abs().sum(-1) > 1e-9
        assert moved.tolist() == [j <= i < j + win for i in range(T)]
    # with the identity the mixing changes nothing; with a permutation of heads that share a kv head the heads'
    # outputs change places; with a matrix of zeros but one row of ones every head but one is silent
    ident = dict(p, talk=torch.eye(H, dtype=F64), o=torch.eye(H * vd, dtype=F64))
    plain_heads = P.talking_attention(h, ident, m, 1e-6).view(T, H, vd)
    swap = torch.eye(H, dtype=F64)[[1, 0, 3, 2]]
    swapped = P.talking_attention(h, dict(ident, talk=swap), m, 1e-6).view(T, H, vd)
    assert torch.allclose(swapped[:, 0], plain_heads[:, 1]) and torch.allclose(swapped[:, 3], plain_heads[:, 2])
    # head 0 of kv head 0 takes the weights of head 2 (kv head 1) but reads the values of its OWN kv head
    t = torch.zeros(H, H, dtype=F64)
    t[0, 2] = 1.0
    crossed = P.talking_attention(h, dict(ident, talk=t), m, 1e-6).view(T, H, vd)
    assert crossed[:, 1:].abs().max() == 0
    same_values = dict(ident, v=torch.cat([p["v"][:vd], p["v"][:vd]]))       # both kv heads hold kv head 0's values
    want = P.talking_attention(h, same_values, m, 1e-6).view(T, H, vd)[:, 2]
    assert torch.allclose(crossed[:, 0], want)
    # the cap bounds the scores: with huge queries every visible key of a head gets a weight of e^(+-cap) at most apart
    loud = P.talking_attention(h * 1e3, ident, dict(m, scale=1e3), 1e-6)
    assert torch.isfinite(loud).all()


def test_recurrence_from_zero_and_its_memory():
    C, T = 3, 6
    u, lam = _rand(5)(T, C), torch.tensor([-4.0, -2.0, 0.5], dtype=F64)
    r, i = torch.full((T, C), 0.5, dtype=F64), torch.full((T, C), 0.25, dtype=F64)
    S = P.gated_recurrence(u, r, i, lam)
    a = torch.exp(-8.0 * 0.5 * torch.log1p(torch.exp(lam)))
    # the first token is no special case: S_0 = sqrt(1 - a^2) i u_0
    assert torch.allclose(S[0], torch.sqrt(1 - a * a) * 0.25 * u[0])
    assert torch.allclose(S[3], a * S[2] + torch.sqrt(1 - a * a) * 0.25 * u[3])
    # r = 0: a = 1, nothing is written and nothing forgotten
    assert P.gated_recurrence(u, torch.zeros(T, C, dtype=F64), i, lam).abs().max() == 0


def test_block_gates_parts_do_not_mix():
    r = _rand(6)
    u, w, b = r(4, 6), r(3, 2, 2), r(3, 2)
    z = P.block_gates(u, w, b)
    assert torch.allclose(z[:, 2:4], u[:, 2:4] @ w[1].T + b[1])
    u2 = u.clone()
    u2[:, 0] += 1.0
    assert torch.equal(P.block_gates(u2, w, b)[:, 2:], z[:, 2:])


def test_distance_attention_sink_bias_window_and_values_that_are_keys():
    H, G, d, W, T, win = 2, 1, 4, 6, 10, 4
    r = _rand(7)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "conv": 2, "scale": 0.5, "mask": {"size": win}}
    p = {"q": r(H * d, W), "k": r(G * d, W), "q.conv": r(H * d, 2), "k.conv": r(G * d, 2), "r1": torch.tensor([0.7, 1.1], dtype=F64),
         "r2": torch.tensor([0.5, 2.0], dtype=F64), "g": r(H * d, W), "o": torch.eye(H * d, dtype=F64)}
    h = r(T, W)
    base = P.distance_attention(h, p, m)
    # the convolution widens the reach by its taps - 1: token j moves keys j and j + 1, which queries up to
    # j + 1 + win - 1 read
    h2 = h.clone()
    h2[3] += 1.0
    moved = (P.distance_attention(h2, p, m) - base).abs().sum(-1) > 1e-12
    assert moved.tolist() == [3 <= i < 3 + win + 1 for i in range(T)]
    # the first token: one key with score s (no distance), weight e^s / (1 + e^s), value = the key itself
    q0 = (p["q"] @ h[0]) * p["q.conv"][:, -1]
    k0 = (p["k"] @ h[0]) * p["k.conv"][:, -1]
    gate = torch.sigmoid(p["g"] @ h[0])
    for hh in range(H):
        s = (q0[hh * d:(hh + 1) * d] @ k0) * 0.5
        want = torch.sigmoid(s) * k0 * gate[hh * d:(hh + 1) * d]
        assert torch.allclose(base[0, hh * d:(hh + 1) * d], want)
    # a larger r1 moves weight from far keys to the sink and the near keys: the output changes from the second token on
    other = P.distance_attention(h, dict(p, r1=p["r1"] * 3), m)
    assert torch.allclose(other[0], base[0]) and (other[1:] - base[1:]).abs().max() > 1e-3


def test_delta_rule_writes_then_reads_and_forgets_by_head():
    H, dk, dv = 2, 4, 3
    k = torch.zeros(3, H, dk, dtype=F64)
    k[0, :, 0] = 1.0
    k[1, :, 1] = 1.0
    k[2, :, 0] = 1.0
    v = _rand(8)(3, H, dv)
    beta = torch.ones(3, H, dtype=F64)
    g = torch.tensor([[1.0, 1.0], [1.0, 0.5], [0.5, 1.0]], dtype=F64)
    o = P.delta_rule(k.clone(), k, v, beta, g)
    assert torch.allclose(o[0], v[0])                     # the read-out sees the token's own write
    assert torch.allclose(o[1], v[1])
    assert torch.allclose(o[2], v[2])                     # beta = 1 replaces what the key held, whatever was forgotten
    half = P.delta_rule(k.clone(), k, v, 0.5 * beta, g)
    # head 0 forgets half of its first write before the third token, head 1 forgot it before the second
    assert torch.allclose(half[2, 0], 0.5 * (0.5 * 0.5 * v[0, 0]) + 0.5 * v[2, 0])
    assert torch.allclose(half[2, 1], 0.5 * (0.5 * 0.5 * v[0, 1]) + 0.5 * v[2, 1])


def test_feed_forward_clamps_before_the_activation():
    W, Fd = 4, 3
    p = {"gate": torch.eye(Fd, W, dtype=F64), "up": torch.eye(Fd, W, dtype=F64), "down": torch.eye(W, Fd, dtype=F64)}
    h = torch.tensor([[5.0, -5.0, 0.5, 0.0]], dtype=F64)
    y = P.clamped_glu(h, p, {"limit": 2.0})
    sig = lambda z: 1.0 / (1.0 + math.exp(-1.702 * z))   # noqa: E731
    assert math.isclose(y[0, 0].item(), 2.0 * sig(2.0) * 3.0)               # both clamped from above
    assert math.isclose(y[0, 1].item(), -5.0 * sig(-5.0) * (-2.0 + 1.0))    # the gate has no lower clamp, the other has
    assert math.isclose(y[0, 2].item(), 0.5 * sig(0.5) * 1.5)


def test_config_reader_name_table_and_cache_plan():
    from mivi_v4_b200.cache import KVNeed, StateNeed
    from mivi_v4_b200.config import ConfigError, RopelixConfig
    from mivi_v4_b200.engine.model import Model, describe_config, expected_tensors
    for cfg, _ in CONFIGS.values():
        c = RopelixConfig.from_dict(cfg)
        assert len(c.layers) == len(cfg["layers"]) and c.residual_mult == cfg["residual_mult"]
    names = expected_tensors(ROP_A)
    assert names["embed"].shape == (97, 64) and names["final.norm"].shape == (64,) and "head" not in names
    assert names["l0.mix.q"].shape == (32, 64) and names["l0.mix.v"].shape == (32, 64) and names["l0.mix.b"].shape == (4, 64)
    assert names["l0.mix.a"].shape == (4, 64) and names["l0.mix.dt_bias"].shape == (4,) and names["l0.mix.g"].shape == (32, 64)
    assert names["l0.mix.k.conv"].shape == (32, 3) and names["l0.mix.norm"].shape == (8,)
    assert names["l0.mlp.gate"].shape == (48, 64) and names["l0.mlp.down"].shape == (64, 48) and names["l0.ls2"].shape == (64,)
    assert names["l1.mix.left.q"].shape == (96, 64) and names["l1.mix.left.k"].shape == (48, 64)
    assert names["l1.mix.left.v"].shape == (96, 64) and names["l1.mix.left.q.norm"].shape == (96,)
    assert names["l1.mix.left.talk"].shape == (6, 6) and names["l1.mix.left.o"].shape == (64, 192)
    assert names["l1.mix.right.ra"].shape == (2, 24, 24) and names["l1.mix.right.ri.b"].shape == (2, 24)
    assert names["l1.mix.right.conv"].shape == (48, 4) and names["l1.mix.right.lam"].shape == (48,)
    assert names["l2.mix.q"].shape == (128, 64) and names["l2.mix.k"].shape == (64, 64) and names["l2.mix.k.conv"].shape == (64, 2)
    assert names["l2.mix.r1"].shape == (4,) and names["l2.mix.g"].shape == (128, 64) and "l2.mix.v" not in names
    assert "l2.mlp.gate" not in names and "l2.ls2" not in names and "l2.norm2" not in names

    config, spec = describe_config(ROP_A)
    model = Model(spec, config)
    assert [type(model.blocks[e.block]).__name__ for e in model.schedule] == 4 * ["PreNormScaledBlock"]
    plan = model.cache_plan()
    kv = {(g.need.n_kv_heads, g.need.head_dim, g.need.value_dim, g.need.window, g.need.values_in_keys): g.n_layers
          for g in plan.groups if isinstance(g.need, KVNeed)}
    assert kv == {(3, 16, 32, 10, False): 1, (2, 32, 32, 150, True): 1, (1, 32, 16, 150, False): 1}
    states = {g.need.shape: g.n_layers for g in plan.groups if isinstance(g.need, StateNeed)}
    assert states[(4, 8, 16)] == 1 and states[(2, 2 * 2 * 16 + 4 * 8)] == 1           # the delta rule and its kept inputs
    assert states[(48,)] == 1 and states[(3, 48)] == 1 and states[(40,)] == 1 and states[(1, 40)] == 1
    assert states[(1, (4 + 2) * 32)] == 1                                              # the kept projections of q and k
    # one tap keeps no inputs
    shapes_b = [g.need.shape for g in Model(describe_config(ROP_B)[1]).cache_plan().groups if isinstance(g.need, StateNeed)]
    assert sorted(shapes_b) == [(1, 12, 20), (3, 72), (30,)]

    def broken(edit):
        c = json.loads(json.dumps(ROP_A))
        edit(c)
        with pytest.raises(ConfigError):
            RopelixConfig.from_dict(c)
    broken(lambda c: c["layers"][0].update(type="mamba2"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18))
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][1]["mixer"]["right"].update(blocks=5))
    broken(lambda c: c["layers"][1]["mixer"].pop("left_scale"))
    broken(lambda c: c["layers"][2]["mixer"].update(vdim=40))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda c: c["layers"][0]["mlp"].pop("limit"))
    broken(lambda c: c.pop("embedding"))
    broken(lambda c: c.update(layers=[]))


def test_a_window_edge_a_lost_state_or_another_constant_would_show(tmp_path):
    """The comparisons of the engine's tests can fail: the plain logits with one mechanism changed lie outside the
    float32 and the bfloat16 limit."""
    cfg, seed = CONFIGS["A"]
    folder = write_ropelix(tmp_path, cfg, seed)
    toks = prompts(cfg["vocab"], [60], 5)[0]
    _, weights = read_folder(folder)
    want = P.forward(cfg, weights, toks)
    limit_bf16 = RC.NOISE_FACTOR * float(RC.noise(cfg, weights, toks, want).min())          # of the quiet rows: the rule of most

    def off(change_cfg=None, change_w=None):
        c = json.loads(json.dumps(cfg))
        w = dict(weights)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(w)
        return rel_rms(P.forward(c, w, toks), want)[20:].max().item()

    def window_one_more(c): c["layers"][1]["mixer"]["left"]["mask"]["size"] += 1
    def window_one_less(c): c["layers"][1]["mixer"]["left"]["mask"]["size"] -= 1
    def rotate_all(c): c["layers"][1]["mixer"]["left"]["rot"]["dims"] = 16
    def other_base(c): c["layers"][1]["mixer"]["left"]["rot"]["base"] = 10000.0
    def other_scale(c): c["layers"][2]["mixer"]["scale"] = 0.3
    def other_cap(c): c["layers"][1]["mixer"]["left"]["softcap"] = 2.0
    def other_side_scale(c): c["layers"][1]["mixer"]["right_scale"] = 0.8
    def other_limit(c): c["layers"][0]["mlp"]["limit"] = 0.5
    def other_mult(c): c["residual_mult"] = 1.0
    def other_embedding_scale(c): c["embedding"]["scale"] = 1.0
    def no_talk(w): w["l1.mix.left.talk"] = torch.eye(6).to(w["l1.mix.left.talk"].dtype)
    def talk_transposed(w): w["l1.mix.left.talk"] = w["l1.mix.left.talk"].T.contiguous()
    def no_distance(w): w["l2.mix.r1"] = torch.zeros_like(w["l2.mix.r1"])
    def other_distance(w): w["l2.mix.r2"] = w["l2.mix.r2"] * 16
    def no_layer_scale(w): w["l1.ls1"] = torch.ones_like(w["l1.ls1"])
    def plain_norm_weight(w): w["l3.norm1"] = w["l3.norm1"] - 1.0
    def other_decay(w): w["l0.mix.A_log"] = w["l0.mix.A_log"] + 1.0
    def other_memory(w): w["l1.mix.right.lam"] = w["l1.mix.right.lam"] + 2.0
    def gates_swapped(w): w["l1.mix.right.ra"], w["l1.mix.right.ri"] = w["l1.mix.right.ri"], w["l1.mix.right.ra"]
    def parts_swapped(w): w["l1.mix.right.ra"] = w["l1.mix.right.ra"].flip(0)
    def taps_reversed(w): w["l2.mix.k.conv"] = w["l2.mix.k.conv"].flip(-1)
    def no_conv_bias(w): w["l1.mix.right.conv.b"] = torch.zeros_like(w["l1.mix.right.conv.b"])
    def no_gate(w): w["l2.mix.g"] = torch.zeros_like(w["l2.mix.g"])
    for change in (dict(change_cfg=window_one_more), dict(change_cfg=window_one_less), dict(change_cfg=rotate_all),
                   dict(change_cfg=other_base), dict(change_cfg=other_scale), dict(change_cfg=other_cap),
                   dict(change_cfg=other_side_scale), dict(change_cfg=other_limit), dict(change_cfg=other_mult),
                   dict(change_cfg=other_embedding_scale), dict(change_w=no_talk), dict(change_w=talk_transposed),
                   dict(change_w=no_distance), dict(change_w=other_distance), dict(change_w=no_layer_scale),
                   dict(change_w=plain_norm_weight), dict(change_w=other_decay), dict(change_w=other_memory),
                   dict(change_w=gates_swapped), dict(change_w=parts_swapped), dict(change_w=taps_reversed),
                   dict(change_w=no_conv_bias), dict(change_w=no_gate)):
        assert off(**change) > 2 * limit_bf16, (change.get("change_cfg") or change.get("change_w"), off(**change), limit_bf16)


def test_command_line_writes_and_describes_a_model_folder(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(ROP_C))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "1", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Ropelix" in text
    assert "l0.mix.left.talk" in text and "l0.mix.right.lam" in text and "l2.mix.r1" in text and "l1.mix.dt_bias" in text
