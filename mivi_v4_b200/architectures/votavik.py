"""The Votavik decoder described in parts.

Every layer is a pre-norm residual block, x += mixer(norm1(x)), then (where the layer has one)
x += feed_forward(norm2(x)), then (where the model has one) the per-layer token input.  The norm is a
layer norm with a weight and no bias; a final one and an untied head follow.  A layer's mixer is one of

  gla        gated linear attention: a matrix state per head with a learned decay per key channel
  attention  grouped-query softmax attention with a norm over the whole q and k projections, a rotation
             of part of each head, capped scores, a sliding window that keeps the first tokens, a sink
             in the softmax and a gate per head
  lightning  linear attention with one fixed decay per head

and layers may come in any order, each with its own sizes.  Checkpoint names:

  embed [vocab, width]; side.embed [vocab, layers * side_dim]; final.norm [width]; head [vocab, width]
  l<i>.norm1, l<i>.norm2 [width]
  l<i>.mix.{q,k,v,g,o}, and by mixer: norm, a1, a2, a2.b (gla); q.norm, k.norm, sink (attention); norm (lightning)
  l<i>.mlp.{gate,up,down}
  l<i>.side.{gate,proj,norm}
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.votavik import VotavikConfig
from ..parts.spec import ModelSpec, PartSpec, ScheduleEntry

NAME = "Votavik"


def _mixer(cfg: VotavikConfig, layer, prefix: str) -> PartSpec:
    m, W, eps = layer.mixer, cfg.width, cfg.norm_eps
    if layer.type == "gla":
        return PartSpec("gated_linear_attention",
                        dict(hidden=W, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], tau=m["tau"], eps=eps,
                             rank=m.get("rank")), prefix=prefix)
    if layer.type == "lightning":
        return PartSpec("lightning_attention",
                        dict(hidden=W, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], decay=list(m["decay"]),
                             eps=eps), prefix=prefix)
    rot, mask = m.get("rot") or {}, m.get("mask") or {}
    dims = int(rot.get("dims", 0))
    position = PartSpec("rope", dict(head_dim=dims, theta=rot["base"], style="half_split")) if dims else PartSpec("none")
    return PartSpec("sink_attention",
                    dict(hidden=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                         scale=m["scale"], softcap=m.get("softcap") or 0.0, window=int(mask.get("size", 0)),
                         keep_first=int(mask.get("keep_first") or 0), qk_norm_eps=eps, sink=True, gated=True),
                    prefix=prefix, parts={"position": position})


def describe(cfg: VotavikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    n = len(cfg.layers)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        pre = f"l{i}."
        parts = {"mixer_norm": PartSpec("layernorm", dict(dim=W, eps=eps), names={"weight": pre + "norm1"}),
                 "mixer": _mixer(cfg, layer, pre + "mix.")}
        if layer.mlp is not None:
            parts["ffn_norm"] = PartSpec("layernorm", dict(dim=W, eps=eps), names={"weight": pre + "norm2"})
            parts["ffn"] = PartSpec("clamped_glu", dict(hidden=W, ff=layer.mlp["ff"], limit=layer.mlp["limit"]),
                                    prefix=pre + "mlp.")
        if cfg.side_dim:
            parts["token_input"] = PartSpec(
                "gated_table", dict(hidden=W, vocab=cfg.vocab, dim=cfg.side_dim, index=i, table_width=n * cfg.side_dim,
                                    eps=eps), prefix=pre + "side.", names={"table": "side.embed"})
        blocks.append(PartSpec("prenorm_optional", prefix=pre, parts=parts))
    return ModelSpec(
        hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("table", dict(vocab=cfg.vocab, hidden=W), names={"weight": "embed"}),
        blocks=blocks, schedule=[ScheduleEntry(i) for i in range(n)],
        final_norm=PartSpec("layernorm", dict(dim=W, eps=eps), names={"weight": "final.norm"}),
        head=PartSpec("linear", dict(vocab=cfg.vocab, hidden=W, tied=False), names={"weight": "head"}),
        stop_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,), max_positions=cfg.max_positions,
    )


register_architecture(NAME, VotavikConfig.from_dict, describe, replace=True)
