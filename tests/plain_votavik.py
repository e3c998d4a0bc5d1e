"""A plain, slow implementation of the Votavik decoder: whole sequences, no
cache, no batching, one function per mechanism, in float64 unless asked
otherwise.  It shares no code with the package; the tests compare the package
against it.

``rnd`` (default: nothing) is applied where a run in a narrower dtype stores an activation between two
kernels (a product's operand, the cached keys and values); with ``round_to(torch.bfloat16)`` the
difference to the unrounded result estimates the rounding noise of such a run.

Notation: x is the residual stream [T, W] of one sequence, h a sublayer's
normed input, ``w`` a dict of tensors by checkpoint name, ``c`` a layer's
entry of config.json's ``layers``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def same(x):
    return x


def round_to(dtype):
    return lambda x: x.to(dtype).to(x.dtype)


def layer_norm(x, weight, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight


def rms_unit(x, eps):
    """x divided by its root mean square over the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def decayed_outer_scan(q, k, v, decay):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for one head.
    q, k [T, dk]; v [T, dv]; decay [T, dk] (a row per token, a factor per key channel).
    Returns o [T, dv] and the last state [dk, dv]."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out) if out else torch.zeros(0, v.shape[1], dtype=q.dtype), S


def gla_mixer(h, w, pre, c, eps, rnd=same):
    """Gated linear attention with a learned decay per key channel."""
    m = c["mixer"]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (h @ w[pre + "q"].T) * dk ** -0.5
    k = h @ w[pre + "k"].T
    v = h @ w[pre + "v"].T
    z = rnd(h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    q, k, alpha, v = q.view(T, H, dk), k.view(T, H, dk), alpha.view(T, H, dk), v.view(T, H, dv)
    heads = []
    for a in range(H):
        o, _ = decayed_outer_scan(q[:, a], k[:, a], v[:, a], alpha[:, a])
        heads.append(rms_unit(o, eps) * w[pre + "norm"])
    o = torch.cat(heads, dim=-1)
    return rnd(o * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def lightning_mixer(h, w, pre, c, eps, rnd=same):
    """Linear attention with one fixed decay per head."""
    m = c["mixer"]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[pre + "q"].T).view(T, H, dk)
    k = silu(h @ w[pre + "k"].T).view(T, H, dk)
    v = silu(h @ w[pre + "v"].T).view(T, H, dv)
    heads = []
    for a in range(H):
        decay = torch.full((T, dk), float(m["decay"][a]), dtype=h.dtype)
        o, _ = decayed_outer_scan(q[:, a], k[:, a], v[:, a], decay)
        heads.append(o)
    o = rms_unit(torch.cat(heads, dim=-1), eps) * w[pre + "norm"]
    return rnd(o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def rotate_partial(x, positions, dims, base):
    """x [T, heads, d]: the first ``dims`` elements of every head turn, element i paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    freq = float(base) ** (-2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def attention_mixer(h, w, pre, c, eps, rnd=same, positions=None):
    """Softmax attention: grouped heads, norm over the whole q and k projections, partial rotation,
    capped scores, a window that keeps the first tokens, a sink in the denominator, a gate per head."""
    m = c["mixer"]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = torch.arange(T) if positions is None else positions
    q = rms_unit(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    k = rms_unit(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = rnd(h @ w[pre + "v"].T).view(T, G, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rnd(rotate_partial(q.view(T, H, dk), pos, int(rot["dims"]), rot["base"]))
    k = rnd(rotate_partial(k.view(T, G, dk), pos, int(rot["dims"]), rot["base"]))
    cap = float(m.get("softcap") or 0.0)
    size, keep = int(m["mask"]["size"]), int(m["mask"]["keep_first"])
    mask = torch.tensor([[visible(int(pos[i]), int(pos[j]), size, keep) for j in range(T)] for i in range(T)])
    gate = torch.sigmoid(h @ w[pre + "g"].T)                      # [T, H]
    heads = []
    for a in range(H):
        kv = a // (H // G)
        s = (q[:, a] @ k[:, kv].T) * float(m["scale"])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~mask, float("-inf"))
        sink = w[pre + "sink"][a].to(s.dtype)
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
        heads.append((p @ v[:, kv]) * gate[:, a:a + 1])
    return rnd(torch.cat(heads, dim=-1)) @ w[pre + "o"].T


def dense_ff(h, w, pre, c, rnd=same):
    limit = float(c["mlp"]["limit"])
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def token_side(x, tokens, w, layer: int, dim: int, eps, rnd=same):
    """The per-layer token input: returns what is added to x."""
    pre = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(rnd(x) @ w[pre + "gate"].T) * e
    y = rnd(g) @ w[pre + "proj"].T
    return rms_unit(y, eps) * w[pre + "norm"]


MIXERS = {"gla": gla_mixer, "lightning": lightning_mixer, "attention": attention_mixer}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=F64,
            return_layers: bool = False, rnd=same):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    side_dim = int((cfg.get("token_side") or {}).get("dim", 0))
    toks = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][toks]
    layers = []
    for i, c in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = rnd(layer_norm(x, w[pre + "norm1"], eps))
        x = x + MIXERS[c["type"]](h, w, pre + "mix.", c, eps, rnd)
        if c.get("mlp") is not None:
            x = x + dense_ff(rnd(layer_norm(x, w[pre + "norm2"], eps)), w, pre + "mlp.", c, rnd)
        if side_dim:
            x = x + token_side(x, toks, w, i, side_dim, eps, rnd)
        layers.append(x)
    logits = rnd(layer_norm(x, w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def greedy(cfg: dict, weights, prompt: List[int], n_new: int, dtype=F64) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks, dtype)[-1].argmax()))
    return toks[len(prompt):]
