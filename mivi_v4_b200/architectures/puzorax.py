"""The Puzorax decoder described in parts.

x = embed[token] + bigram[hash(previous token, token)]; every layer is x += mixer(h) + feed_forward(h) with
h = layer_norm(x) (one norm with weight and bias that both sublayers read); a final layer norm and an untied head
follow.  A layer's mixer is one of

  latent_attention  softmax attention over a compressed cache (one normed low-rank row and one rotated key part a
                    token for all heads), with a sliding window, a sink per head and an output gate
  channel_delta     the gated delta rule with a decay per key channel, short causal convolutions on q, k and v,
                    unit-norm q and k, a gated root-mean-square norm on the read-out

and its feed-forward a mixture of experts with softmax scores, a correction that only the choice sees, a factor on
the weights, and identity experts.  Layers may come in any order, each with its own sizes.  A run of layers may be
walked several times with the same weights (``loop``): every pass has caches and states of its own; before every
pass but the first the embedding's output is added to the stream again, and before every pass one learned vector of
``loop.step`` [times, width].  Checkpoint names:

  embed [vocab, width]; bigram [buckets + 1, width]; loop.step [times, width]; final.norm, final.norm.b; head
  l<i>.norm1, l<i>.norm1.b [width]
  l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,g,o}                                         (latent_attention)
  l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,A_log,norm,a1,a2,dt_bias,g1,g2,o}         (channel_delta)
  l<i>.mlp.router, l<i>.mlp.correction, l<i>.mlp.e<j>.{gate,up,down}
"""
from __future__ import annotations

from ..config.puzorax import PuzoraxConfig
from ..config.registry import register_architecture
from ..parts.spec import ModelSpec, PartSpec, ScheduleEntry

NAME = "Puzorax"


def _mixer(cfg: PuzoraxConfig, layer, prefix: str) -> PartSpec:
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "latent_attention":
        rot = m.get("rot") or {}
        dims = int(rot.get("dims", 0))
        position = PartSpec("rope", dict(head_dim=dims, theta=rot["base"], style="half_split")) if dims else PartSpec("none")
        return PartSpec("latent_attention",
                        dict(hidden=W, n_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
                             kv_rank=m["kv_rank"], scale=m["scale"], eps=eps, window=int((m.get("mask") or {}).get("size", 0)),
                             sink=True, gated=True), prefix=prefix, parts={"position": position})
    return PartSpec("channel_delta",
                    dict(hidden=W, n_heads=m["heads"], kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                         conv=m["conv"], eps=eps, decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank")),
                    prefix=prefix)


def _mlp(cfg: PuzoraxConfig, mlp: dict, prefix: str) -> PartSpec:
    r = mlp["router"]
    return PartSpec("routed_experts",
                    dict(hidden=cfg.width, n_experts=r["experts"], ff=mlp["expert"]["ff"], top=r["top"], score="softmax",
                         correction=True, out_scale=float(r.get("scale", 1.0) if r.get("scale") is not None else 1.0),
                         n_identity=int(r.get("identity") or 0)), prefix=prefix)


def describe(cfg: PuzoraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    blocks = []
    for i, layer in enumerate(cfg.layers):
        pre = f"l{i}."
        parts = {"norm": PartSpec("layernorm", dict(dim=W, eps=eps, bias=True),
                                  names={"weight": pre + "norm1", "bias": pre + "norm1.b"}),
                 "mixer": _mixer(cfg, layer, pre + "mix.")}
        if layer.mlp is not None:
            parts["ffn"] = _mlp(cfg, layer.mlp, pre + "mlp.")
        blocks.append(PartSpec("parallel_prenorm", prefix=pre, parts=parts))
    n = len(blocks)
    if cfg.loop is None:
        schedule = [ScheduleEntry(i) for i in range(n)]
    else:
        # one restart block a pass (they share the tensor of the passes' vectors), then the run's layers again:
        # a block that appears again in the schedule has a cache or state of its own there
        lp = cfg.loop
        schedule = [ScheduleEntry(i) for i in range(lp.start)]
        for t in range(lp.times):
            blocks.append(PartSpec("stream_restart", dict(hidden=W, n_rows=lp.times, row=t, add_embedding=t > 0),
                                   names={"steps": "loop.step"}))
            schedule.append(ScheduleEntry(len(blocks) - 1))
            schedule += [ScheduleEntry(i) for i in range(lp.start, lp.stop)]
        schedule += [ScheduleEntry(i) for i in range(lp.stop, n)]
    return ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("table_bigram",
                           dict(vocab=cfg.vocab, hidden=W, buckets=cfg.buckets, mul_prev=cfg.mul_prev, mul_cur=cfg.mul_cur,
                                keep=cfg.loop is not None and cfg.loop.times > 1),
                           names={"weight": "embed", "bigram": "bigram"}),
        blocks=blocks, schedule=schedule,
        final_norm=PartSpec("layernorm", dict(dim=W, eps=eps, bias=True), names={"weight": "final.norm", "bias": "final.norm.b"}),
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False), names={"weight": "head"}),
        ignorable=("loop.step",) if cfg.loop is None else (),
        stop_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,),
    )


register_architecture(NAME, PuzoraxConfig.from_dict, describe, replace=True)
