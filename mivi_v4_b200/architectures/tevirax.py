"""The Tevirax decoder described in parts.

x = embed[token] * scale + pos[position]; every layer is x += norm1(mixer(x)), then (where the layer has one)
x += norm2(feed_forward(x)): root-mean-square norms on the sublayers' outputs, the sublayers read the stream
itself; a final norm, an untied head and a smooth cap on the logits follow.  A layer's mixer is one of

  mamba2    a selective state space layer (scalar decay per head and token, short causal convolution, gate
            before a grouped norm)
  parallel  two mixers that read the same input, summed with a factor each: grouped-query softmax attention
            with a per-head q/k norm, a rotation of part of each head with stretched frequencies, and a chunked
            mask (left); a matrix memory with exponential gates (right)

and its feed-forward a gated one (``dense``) or a mixture of experts with sigmoid scores, groups of experts and a
shared expert (``moe``).  Layers may come in any order, each with its own sizes.  Checkpoint names:

  embed [vocab, width]; pos [max_positions, width]; final.norm [width]; head [vocab, width]
  l<i>.norm1, l<i>.norm2 [width]
  l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}                               (mamba2)
  l<i>.mix.left.{q,k,v,o,q.norm,k.norm}, l<i>.mix.right.{q,k,v,g,o,norm,i,i.b,f,f.b}  (parallel)
  l<i>.mlp.{gate,up,down}                                                        (dense)
  l<i>.mlp.router, l<i>.mlp.e<j>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down,sg}    (moe)
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tevirax import TeviraxConfig
from ..parts.spec import ModelSpec, PartSpec, ScheduleEntry

NAME = "Tevirax"


def _position(rot) -> PartSpec:
    dims = int((rot or {}).get("dims", 0))
    if not dims:
        return PartSpec("none")
    sc = rot.get("scaling")
    if sc:
        return PartSpec("rope_yarn", dict(head_dim=dims, theta=rot["base"], factor=sc["factor"], original=sc["original"],
                                          fast=sc["fast"], slow=sc["slow"], style="half_split"))
    return PartSpec("rope", dict(head_dim=dims, theta=rot["base"], style="half_split"))


def _mixer(cfg: TeviraxConfig, layer, prefix: str) -> PartSpec:
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "mamba2":
        return PartSpec("mamba2", dict(hidden=W, n_heads=m["heads"], value_dim=m["vdim"], state=m["state"], groups=m["groups"],
                                       conv=m["conv"], norm_groups=m["norm_groups"], eps=eps), prefix=prefix)
    l, r = m["left"], m["right"]
    left = PartSpec("sink_attention",
                    dict(hidden=W, n_heads=l["heads"], n_kv_heads=l["kv_heads"], key_dim=l["dim"], value_dim=l["vdim"],
                         scale=l["scale"], chunk=int((l.get("mask") or {}).get("size", 0)), qk_norm_eps=eps,
                         norm_per_head=True, sink=False, gated=False),
                    prefix=prefix + "left.", parts={"position": _position(l.get("rot"))})
    right = PartSpec("matrix_memory", dict(hidden=W, n_heads=r["heads"], key_dim=r["dim"], value_dim=r["vdim"],
                                           gate_cap=r["gate_cap"], eps=eps), prefix=prefix + "right.")
    return PartSpec("parallel", dict(left_scale=m["left_scale"], right_scale=m["right_scale"]), prefix=prefix,
                    parts={"left": left, "right": right})


def _mlp(cfg: TeviraxConfig, mlp: dict, prefix: str) -> PartSpec:
    W = cfg.width
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden=W, ff=mlp["ff"]), prefix=prefix,
                        names={"w1.weight": prefix + "gate", "w3.weight": prefix + "up", "w2.weight": prefix + "down"})
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("routed_experts",
                    dict(hidden=W, n_experts=r["experts"], ff=mlp["expert"]["ff"], top=r["top"], n_groups=groups["count"],
                         keep_groups=groups["keep"], shared_ff=(mlp.get("shared") or {}).get("ff", 0)), prefix=prefix)


def describe(cfg: TeviraxConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    blocks = []
    for i, layer in enumerate(cfg.layers):
        pre = f"l{i}."
        parts = {"mixer": _mixer(cfg, layer, pre + "mix."),
                 "mixer_norm": PartSpec("rmsnorm", dict(dim=W, eps=eps), names={"weight": pre + "norm1"})}
        if layer.mlp is not None:
            parts["ffn"] = _mlp(cfg, layer.mlp, pre + "mlp.")
            parts["ffn_norm"] = PartSpec("rmsnorm", dict(dim=W, eps=eps), names={"weight": pre + "norm2"})
        blocks.append(PartSpec("postnorm", prefix=pre, parts=parts))
    return ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("table_scaled_positions",
                           dict(vocab=cfg.vocab, hidden=W, scale=cfg.embedding_scale, max_positions=cfg.max_positions,
                                hand_rounded=True), names={"weight": "embed", "positions": "pos"}),
        blocks=blocks, schedule=[ScheduleEntry(i) for i in range(len(blocks))],
        final_norm=PartSpec("rmsnorm", dict(dim=W, eps=eps), names={"weight": "final.norm"}),
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False, softcap=cfg.logit_softcap), names={"weight": "head"}),
        stop_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,), max_positions=cfg.max_positions,
    )


register_architecture(NAME, TeviraxConfig.from_dict, describe, replace=True)
