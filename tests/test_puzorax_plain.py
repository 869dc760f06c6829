"""The plain Puzorax implementation against closed forms (no GPU), and the parts of the package that need no GPU:
the configuration reader, the name table, the order of the layer runs, the cache's plan, and the command line."""
import json
import math

import pytest
import torch

import plain_puzorax as P
from puzorax_configs import CONFIGS, PUZ_A, PUZ_B, PUZ_C, PUZ_D

F64 = torch.float64


def test_bigram_rows_first_token_and_hash():
    assert P.bigram_rows([4, 9, 9, 0], 7, 2, 3) == [7, (4 * 2 + 9 * 3) % 7, (9 * 2 + 9 * 3) % 7, (9 * 2) % 7]
    assert P.bigram_rows([5], 11, 1, 1) == [11]
    cfg = {"embedding": {"bigram": {"buckets": 3, "mul_prev": 1, "mul_cur": 1}}}
    embed, bigram = torch.eye(4, dtype=F64), 10.0 * torch.arange(4, dtype=F64)[:, None].expand(4, 4)
    x = P.embedding([2, 3, 1], embed, bigram, cfg)
    assert torch.equal(x[0], embed[2] + 30.0) and torch.equal(x[1], embed[3] + 10.0 * ((2 + 3) % 3))
    assert torch.equal(x[2], embed[1] + 10.0 * ((3 + 1) % 3))


def test_rotation_pairs_element_i_with_i_plus_half_of_the_turned_part():
    x = torch.randn(3, 2, 12, dtype=F64)
    y = P.rotate_half(x, torch.tensor([0, 5, 9]), 100.0, 8)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])          # position 0 and the part that passes
    a = 5 * 100.0 ** (-2 * 1 / 8)
    assert torch.allclose(y[1, :, 1], x[1, :, 1] * math.cos(a) - x[1, :, 5] * math.sin(a))
    assert torch.allclose(y[1, :, 5], x[1, :, 5] * math.cos(a) + x[1, :, 1] * math.sin(a))
    assert torch.equal(P.rotate_half(x, torch.tensor([1, 2, 3]), 100.0, 0), x)


def _latent_weights(H, dim, rd, vd, rank, W, sink):
    g = torch.Generator().manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)   # noqa: E731
    return {"q": r(H * (dim + rd), W), "dkv": r(rank + rd, W), "dkv.norm": 1.0 + 0.1 * r(rank), "uk": r(H * dim, rank),
            "uv": r(H * vd, rank), "sink": torch.full((H,), sink, dtype=F64), "g": r(H * vd, W), "o": r(W, H * vd)}


def test_latent_attention_window_edge_and_sink():
    """Token i must not depend on token i - window, must depend on token i - window + 1; a sink of minus infinity
    changes nothing beside plain softmax, a large one silences the layer."""
    H, dim, rd, vd, rank, W, T, win = 2, 4, 4, 3, 6, 8, 12, 5
    m = {"heads": H, "dim": dim, "rot_dim": rd, "vdim": vd, "kv_rank": rank, "scale": 0.4, "mask": {"size": win},
         "rot": {"dims": rd, "base": 100.0}}
    p = _latent_weights(H, dim, rd, vd, rank, W, -1.0)
    h = torch.randn(T, W, generator=torch.Generator().manual_seed(4), dtype=F64)
    base = P.latent_attention(h, p, m, 1e-6)
    for j in (3, 6):
        h2 = h.clone()
        h2[j] += 1.0
        moved = (P.latent_attention(h2, p, m, 1e-6) - base).abs().sum(-1) > 1e-9
        assert moved.tolist() == [j <= i < j + win for i in range(T)]
    silent = P.latent_attention(h, dict(p, sink=torch.full((H,), 80.0, dtype=F64)), m, 1e-6)
    assert silent.abs().max() < 1e-20 * base.abs().max() + 1e-25
    # without a window and with the sink far below: the first token's output is its own value through gate and W_o
    m0 = {k: v for k, v in m.items() if k != "mask"}
    p0 = dict(p, sink=torch.full((H,), -700.0, dtype=F64))
    y = P.latent_attention(h, p0, m0, 1e-6)
    c = P.rms_norm((h[:1] @ p["dkv"].T)[:, :rank], p["dkv.norm"], 1e-6)
    v0 = (c @ p["uv"].T) * torch.sigmoid(h[:1] @ p["g"].T)
    assert torch.allclose(y[0], (v0 @ p["o"].T)[0])


def test_delta_rule_writes_then_reads_and_forgets_by_channel():
    # one head, two key channels: k = e0 writes v into row 0; q = e0 reads it back at once (the read-out sees the
    # token's own write); a decay on channel 0 alone shrinks it, one on channel 1 leaves it
    e0, e1 = torch.tensor([1.0, 0.0], dtype=F64), torch.tensor([0.0, 1.0], dtype=F64)
    k = torch.stack([e0, e1, e0])[:, None, :]
    q = torch.stack([e0, e0, e0])[:, None, :]
    v = torch.tensor([[[2.0, 4.0]], [[1.0, 1.0]], [[0.0, 0.0]]], dtype=F64)
    beta = torch.tensor([[1.0], [1.0], [0.5]], dtype=F64)
    g = torch.tensor([[[1.0, 1.0]], [[0.5, 1.0]], [[1.0, 0.25]]], dtype=F64)
    o = P.delta_rule(q, k, v, beta, g)
    assert torch.allclose(o[0, 0], torch.tensor([2.0, 4.0], dtype=F64))
    assert torch.allclose(o[1, 0], torch.tensor([1.0, 2.0], dtype=F64))             # row 0 halved; the write went to row 1
    # token 2: u = 0.5 (0 - S^T e0) = -0.5 (1, 2): row 0 is halved again
    assert torch.allclose(o[2, 0], torch.tensor([0.5, 1.0], dtype=F64))


def test_causal_taps_last_column_is_the_current_token():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=F64)
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)
    y = P.causal_conv_silu(x, taps)
    pre = torch.tensor([[1.0], [12.0], [124.0]], dtype=F64)
    assert torch.allclose(y, pre * torch.sigmoid(pre))


def test_router_correction_moves_the_choice_and_not_the_weights():
    z = torch.tensor([[2.0, 1.0, 0.0, -1.0]], dtype=F64)
    s = torch.softmax(z, -1)[0]
    dense = P.route(z, torch.zeros(4), 2, 1.0)
    assert torch.allclose(dense[0], torch.stack([s[0], s[1], s[0] * 0, s[0] * 0]) / (s[0] + s[1]))
    dense = P.route(z, torch.tensor([0.0, 0.0, 0.0, 5.0]), 2, 3.0)                 # entry 3 is chosen by its correction alone
    assert torch.allclose(dense[0], 3.0 * torch.stack([s[0], s[0] * 0, s[0] * 0, s[3]]) / (s[0] + s[3]))


def test_identity_experts_pass_the_input_on():
    W = 6
    mlp = {"expert": {"ff": 4}, "router": {"experts": 1, "identity": 2, "top": 2, "scale": 2.0}}
    g = torch.Generator().manual_seed(5)
    p = {"router": torch.zeros(3, W, dtype=F64), "correction": torch.tensor([-1.0, 0.0, 0.0], dtype=F64),
         "e0.gate": torch.randn(4, W, generator=g, dtype=F64), "e0.up": torch.randn(4, W, generator=g, dtype=F64),
         "e0.down": torch.randn(W, 4, generator=g, dtype=F64)}
    h = torch.randn(3, W, generator=g, dtype=F64)
    assert torch.allclose(P.moe(h, p, mlp), 2.0 * h)              # both identity experts, half of the weight each


def test_layer_runs_follow_the_repeated_run():
    assert [r[:2] for r in P.layer_runs(PUZ_A)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2)]
    assert [r[2] for r in P.layer_runs(PUZ_A)] == [False, True, False, True, False, True, False]
    assert [r[:2] for r in P.layer_runs(PUZ_C)] == [(0, 0), (1, 0), (0, 1), (1, 1), (2, None), (3, None)]
    assert [r[:2] for r in P.layer_runs(PUZ_B)] == [(0, None), (1, None), (2, None)]


def test_config_reader_name_table_schedule_and_cache_plan():
    from mivi_v4_b200.cache import KVNeed, StateNeed
    from mivi_v4_b200.config import ConfigError, PuzoraxConfig
    from mivi_v4_b200.engine.model import Model, describe_config, expected_tensors
    for cfg, _ in CONFIGS.values():
        c = PuzoraxConfig.from_dict(cfg)
        assert len(c.layers) == len(cfg["layers"]) and c.buckets == cfg["embedding"]["bigram"]["buckets"]
    names = expected_tensors(PUZ_A)
    assert names["embed"].shape == (97, 64) and names["bigram"].shape == (54, 64) and names["loop.step"].shape == (3, 64)
    assert names["l0.norm1.b"].shape == (64,) and names["final.norm.b"].shape == (64,)
    assert names["l0.mix.q"].shape == (32, 64) and names["l0.mix.v"].shape == (32, 64) and names["l0.mix.b"].shape == (4, 64)
    assert names["l0.mix.a1"].shape == (6, 64) and names["l0.mix.a2"].shape == (64, 6) and names["l0.mix.g2"].shape == (32, 10)
    assert names["l0.mix.k.conv"].shape == (32, 3) and names["l0.mix.norm"].shape == (8,)
    assert names["l0.mlp.router"].shape == (7, 64) and names["l0.mlp.correction"].shape == (7,)
    assert names["l0.mlp.e5.down"].shape == (64, 24) and "l0.mlp.e6.down" not in names
    assert names["l1.mix.q"].shape == (200, 64) and names["l1.mix.dkv"].shape == (36, 64) and names["l1.mix.uk"].shape == (80, 24)
    assert names["l1.mix.uv"].shape == (60, 24) and names["l1.mix.sink"].shape == (10,) and names["l1.mix.g"].shape == (60, 64)
    assert "l2.mlp.router" not in names
    assert "loop.step" not in expected_tensors(PUZ_B)
    without = json.loads(json.dumps(PUZ_A))
    for k in ("decay_rank", "gate_rank"):
        without["layers"][0]["mixer"].pop(k)              # the inner sizes are then the checkpoint's to say
    assert expected_tensors(without)["l0.mix.a1"].shape == (None, 64) and expected_tensors(without)["l0.mix.g2"].shape == (32, None)

    config, spec = describe_config(PUZ_A)
    model = Model(spec, config)
    kinds = [type(model.blocks[e.block]).__name__ for e in model.schedule]
    assert kinds == ["ParallelPreNormBlock"] + 3 * ["StreamRestart", "ParallelPreNormBlock", "ParallelPreNormBlock"]
    assert [e.block for e in model.schedule if kinds[model.schedule.index(e)] != "StreamRestart"][:3] == [0, 1, 2]
    plan = model.cache_plan()
    # every pass over the repeated run has pages and states of its own; the embedding keeps the previous token
    kv = [g for g in plan.groups if isinstance(g.need, KVNeed)]
    assert len(kv) == 1 and kv[0].n_layers == 3 and kv[0].need.window == 10 and kv[0].need.head_dim == 24 + 12
    assert kv[0].need.values_in_keys and kv[0].need.value_dim == 24
    states = {g.need.shape: g.n_layers for g in plan.groups if isinstance(g.need, StateNeed)}
    assert states[(4, 8, 16)] == 1 and states[(2, 24, 24)] == 3 and states[(1,)] == 1
    assert states[(2, 2 * 2 * 16 + 4 * 8)] == 1 and states[(1, 2 * 2 * 24 + 2 * 24)] == 3
    assert all(Model(describe_config(PUZ_D)[1]).cache_plan().groups[i].need.__class__ is StateNeed for i in range(3))

    def broken(edit):
        c = json.loads(json.dumps(PUZ_A))
        edit(c)
        with pytest.raises(ConfigError):
            PuzoraxConfig.from_dict(c)
    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=8))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda c: c["loop"].update(stop=4))
    broken(lambda c: c["loop"].update(times=0))
    broken(lambda c: c["embedding"]["bigram"].update(buckets=0))
    broken(lambda c: c.pop("embedding"))


def test_two_way_routers_stay_far_from_a_close_call(tmp_path):
    """The weights of the bfloat16 engine tests: in every mixture layer the last chosen entry lies well above the
    first one left out, and both routes are taken."""
    from puzorax_configs import prompts, read_folder, write_puzorax
    for name, (cfg, seed) in CONFIGS.items():
        c, w = read_folder(write_puzorax(tmp_path, cfg, seed, router="two_way"))
        margins = []
        P.forward(prompts(cfg["vocab"], [150], seed)[0], w, c, margins=margins)
        assert margins, name
        assert min(float(m.min()) for m in margins) > 5e-3, (name, [float(m.min()) for m in margins])


def test_command_line_writes_and_describes_a_model_folder(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(PUZ_A))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "1", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Puzorax" in text
    assert "l1.mix.dkv.norm" in text and "l0.mix.dt_bias" in text and "l0.mlp.correction" in text and "loop.step" in text
