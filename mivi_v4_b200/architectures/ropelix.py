"""The Ropelix decoder described in parts.

x = embed[token] * scale; every layer is x += m * s1 * mixer(norm1(x)), then (where the layer has one)
x += m * s2 * feed_forward(norm2(x)): root-mean-square norms whose weights are stored around zero (the factor is
1 + weight), a learned vector per sublayer on its result, one constant m for all.  The final norm is of the same
kind, and the head is the embedding table itself (without its factor).  A layer's mixer is one of

  parallel   two mixers that read the same input, summed with a factor each: grouped-query softmax attention with a
             norm over the whole q and k projections, a rotation of part of each head, capped scores, a sliding
             window and softmax weights mixed between the heads (left); a recurrent block with a real-gated linear
             recurrent unit (right)
  attention  grouped-query attention whose q and k pass a short causal convolution, whose values are the keys,
             with a logarithmic distance bias on the scores, a sliding window, a sink of score 0 in the softmax's
             denominator and a gate per output element
  delta      the gated delta rule with one decay per head

and its feed-forward a clamped gated one.  Layers may come in any order, each with its own sizes.  Checkpoint names:

  embed [vocab, width]; final.norm [width]
  l<i>.norm1, l<i>.norm2, l<i>.ls1, l<i>.ls2 [width]
  l<i>.mix.left.{q,k,v,o,q.norm,k.norm,talk}, l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}   (parallel)
  l<i>.mix.{q,k,q.conv,k.conv,r1,r2,g,o}                                                                    (attention)
  l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,a,A_log,dt_bias,norm,g,o}                                          (delta)
  l<i>.mlp.{gate,up,down}
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.ropelix import RopelixConfig
from ..parts.spec import ModelSpec, PartSpec, ScheduleEntry

NAME = "Ropelix"
GATE_CONSTANT = 8.0          # log a = -8 r softplus(lam) in the recurrent block
GLU_ALPHA = 1.702            # the sigmoid's factor in the feed-forward's activation


def _window(m: dict) -> int:
    return int((m.get("mask") or {}).get("size", 0))


def _mixer(cfg: RopelixConfig, layer, prefix: str) -> PartSpec:
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "parallel":
        l, r = m["left"], m["right"]
        rot = l.get("rot") or {}
        dims = int(rot.get("dims", 0))
        position = PartSpec("rope", dict(head_dim=dims, theta=rot["base"], style="half_split")) if dims else PartSpec("none")
        left = PartSpec("sink_attention",
                        dict(hidden=W, n_heads=l["heads"], n_kv_heads=l["kv_heads"], key_dim=l["dim"], value_dim=l["vdim"],
                             scale=l["scale"], softcap=float(l.get("softcap") or 0.0), window=_window(l), qk_norm_eps=eps,
                             sink=False, gated=False, talk=True, split_weights=True),
                        prefix=prefix + "left.", parts={"position": position})
        right = PartSpec("gated_recurrence", dict(hidden=W, width=r["width"], blocks=r["blocks"], conv=r["conv"],
                                                  c=GATE_CONSTANT), prefix=prefix + "right.")
        return PartSpec("parallel", dict(left_scale=m["left_scale"], right_scale=m["right_scale"]), prefix=prefix,
                        parts={"left": left, "right": right})
    if layer.type == "attention":
        return PartSpec("sink_attention",
                        dict(hidden=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                             scale=m["scale"], window=_window(m), sink="zero", gated="element", conv=m["conv"],
                             values_are_keys=True, distance_bias=True, split_weights=True),
                        prefix=prefix, parts={"position": PartSpec("none")})
    return PartSpec("gated_delta", dict(hidden=W, n_heads=m["heads"], kv_heads=m["kv_heads"], key_dim=m["dim"],
                                        value_dim=m["vdim"], conv=m["conv"], eps=eps), prefix=prefix)


def describe(cfg: RopelixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(dim=W, eps=eps, one_plus=True), names={"weight": name})

    blocks = []
    for i, layer in enumerate(cfg.layers):
        pre = f"l{i}."
        parts = {"mixer_norm": norm(pre + "norm1"), "mixer": _mixer(cfg, layer, pre + "mix.")}
        names = {"scale1": pre + "ls1"}
        if layer.mlp is not None:
            parts["ffn_norm"] = norm(pre + "norm2")
            parts["ffn"] = PartSpec("clamped_glu", dict(hidden=W, ff=layer.mlp["ff"], limit=layer.mlp["limit"],
                                                        alpha=GLU_ALPHA), prefix=pre + "mlp.")
            names["scale2"] = pre + "ls2"
        blocks.append(PartSpec("prenorm_scaled", dict(hidden=W, residual_mult=cfg.residual_mult), prefix=pre, parts=parts,
                               names=names))
    return ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("table_scaled_positions", dict(vocab=cfg.vocab, hidden=W, scale=cfg.embedding_scale, positions=False),
                           names={"weight": "embed"}),
        blocks=blocks, schedule=[ScheduleEntry(i) for i in range(len(blocks))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=True)),
        # a layer without a feed-forward may still carry the tensors of its second sublayer's norm and vector
        ignorable=tuple(f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for n in ("norm2", "ls2")),
        stop_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,),
    )


register_architecture(NAME, RopelixConfig.from_dict, describe, replace=True)
