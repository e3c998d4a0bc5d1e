"""A plain, slow implementation of the Tevirax decoder: whole sequences, no cache, no batching, one
function per mechanism, in float64 unless asked otherwise.  It shares no code with the package; the
tests compare the package against it.

``rnd`` (default: nothing) is applied where a run in a narrower dtype stores an activation between two
kernels (a product's operand, the cached keys and values); with ``round_to(torch.bfloat16)`` the
difference to the unrounded result estimates the rounding noise of such a run.

Notation: x is the residual stream [T, W] of one sequence, h a sublayer's input (the stream itself:
the norms sit on the sublayers' outputs), ``w`` a dict of tensors by checkpoint name, ``c`` a layer's
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


def rms_unit(x, eps):
    """x divided by its root mean square over the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return torch.minimum(z, torch.zeros_like(z)) - torch.log1p(torch.exp(-z.abs()))


# ---------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot: dict):
    """(frequency of every pair [dims/2] in float64, the factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: Optional[dict]):
    """x [T, heads, dim]: element i < dims/2 of every head is paired with i + dims/2; the rest passes."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    f, amp = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * amp).to(x.dtype)[:, None, :], (torch.sin(ang) * amp).to(x.dtype)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------- softmax side
def visible(T: int, mask: Optional[dict]):
    """[T, T] bool: query i sees key j <= i, and with a chunk size only inside its own chunk."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask and mask.get("size"):
        ok = ok & (i // int(mask["size"]) == j // int(mask["size"]))
    return ok


def chunked_attention(h, w, pre, m, eps, rnd=same):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, dk)
    k = (h @ w[pre + "k"].T).view(T, G, dk)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    q = rms_unit(q, eps) * w[pre + "q.norm"]
    k = rms_unit(k, eps) * w[pre + "k.norm"]
    pos = torch.arange(T)
    q, k, v = rnd(rotate(q, pos, m.get("rot"))), rnd(rotate(k, pos, m.get("rot"))), rnd(v)
    ok = visible(T, m.get("mask"))
    outs = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~ok, float("-inf"))
        outs.append(torch.softmax(s, dim=-1) @ v[:, g])
    return rnd(torch.cat(outs, dim=-1)) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------- matrix memory
def matrix_memory_scan(q, k, v, i_log, f_log):
    """One head.  m_t = max(f_t + m_(t-1), i_t) with m_0 = 0; S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) +
    e^(i_t - m_t) k_t v_t^T; n_t the same with k alone; o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=q.dtype)
    n = torch.zeros(dk, dtype=q.dtype)
    m = torch.zeros((), dtype=q.dtype)
    out = []
    for t in range(T):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        a, b = torch.exp(f_log[t] + m - m_new), torch.exp(i_log[t] - m_new)
        S = a * S + b * k[t][:, None] * v[t][None, :]
        n = a * n + b * k[t]
        m = m_new
        out.append(S.T @ q[t] / (torch.maximum((n @ q[t]).abs(), torch.exp(-m)) + 1e-6))
    return torch.stack(out)


def matrix_memory(h, w, pre, m, eps, rnd=same):
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = ((h @ w[pre + "q"].T) * dk ** -0.5).view(T, H, dk)
    k = (h @ w[pre + "k"].T).view(T, H, dk)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    i_log = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    f_log = log_sigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    heads = [rms_unit(matrix_memory_scan(q[:, a], k[:, a], v[:, a], i_log[:, a], f_log[:, a]), eps) for a in range(H)]
    o = torch.cat(heads, dim=-1) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return rnd(o) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps, rnd=same):
    left = chunked_attention(h, w, pre + "left.", m["left"], eps, rnd)
    right = matrix_memory(h, w, pre + "right.", m["right"], eps, rnd)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---------------------------------------------------------------------------------- state space
def causal_taps(u, taps, bias):
    """u [T, C]; taps [C, K], the last column for the current token; zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + pad[j:j + T] * taps[:, j]
    return out


def state_space_scan(x, B, C, dt, A, D):
    """One head.  S_t = e^(A dt_t) S_(t-1) + dt_t B_t x_t^T (S: N x vdim); y_t = S_t^T C_t + D x_t."""
    T, N = B.shape
    S = torch.zeros(N, x.shape[1], dtype=x.dtype)
    out = []
    for t in range(T):
        S = torch.exp(A * dt[t]) * S + dt[t] * B[t][:, None] * x[t][None, :]
        out.append(S.T @ C[t] + D * x[t])
    return torch.stack(out)


def mamba2_mixer(h, w, pre, m, eps, rnd=same):
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    p = h @ w[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = rnd(silu(causal_taps(xbc, w[pre + "conv"], w[pre + "conv.b"])))
    x = xbc[:, :inner].view(T, H, P)
    Bm = xbc[:, inner:inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[pre + "dt_bias"])
    A = -torch.exp(w[pre + "A_log"])
    ys = []
    for a in range(H):
        g = a // (H // G)
        ys.append(state_space_scan(x[:, a], Bm[:, g], Cm[:, g], dt[:, a], A[a], w[pre + "D"][a]))
    y = torch.cat(ys, dim=-1) * silu(z)
    parts = int(m["norm_groups"])
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return rnd(y) @ w[pre + "o"].T


# ---------------------------------------------------------------------------------- feed-forward
def gated_mlp(h, w, pre, rnd=same, weight=None):
    """``weight``: a factor on the gated activations (a router's weight): a narrow run may round them before the
    factor and again after it, so both roundings are taken."""
    act = rnd(silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T))
    if weight is not None:
        act = rnd(act * weight)
    return act @ w[pre + "down"].T


def route(h, w_router, r: dict):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.sigmoid(h @ w_router.T)
    T, E = s.shape
    top = int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    per = E // count
    by_group = s.view(T, count, per)
    group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
    best = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    allowed = allowed[:, :, None].expand(T, count, per).reshape(T, E)
    pick = s.masked_fill(~allowed, float("-inf")).topk(top, dim=-1).indices
    chosen = s.gather(1, pick)
    return pick, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def mixture(h, w, pre, mlp: dict, rnd=same, h_router=None, router_inputs=None):
    T = h.shape[0]
    if router_inputs is not None:
        router_inputs.append(h)
    pick, weight = route(h if h_router is None else h_router, w[pre + "router"], mlp["router"])
    out = torch.zeros(T, w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        for e, a in zip(pick[t].tolist(), weight[t]):
            out[t] += gated_mlp(h[t:t + 1], w, f"{pre}e{e}.", rnd, weight=a)[0]
    if mlp.get("shared"):
        out = out + gated_mlp(h, w, pre + "shared.", rnd, weight=torch.sigmoid(h @ w[pre + "shared.sg"].T))
    return out


# ---------------------------------------------------------------------------------- the model
def mixer(h, w, pre, c, eps, rnd=same):
    if c["type"] == "parallel":
        return parallel_mixer(h, w, pre, c["mixer"], eps, rnd)
    if c["type"] == "mamba2":
        return mamba2_mixer(h, w, pre, c["mixer"], eps, rnd)
    raise ValueError(c["type"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=F64, rnd=same, layers_out=None, router_inputs=None):
    """Logits [T, vocab] of one whole sequence.  ``router_inputs`` (a list) gets the input of every mixture layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    T = len(tokens)
    x = w["embed"][tok] * float(cfg["embedding"]["scale"]) + w["pos"][:T]
    for i, c in enumerate(cfg["layers"]):
        pre = f"l{i}."
        x = x + rms_norm(mixer(rnd(x), w, pre + "mix.", c, eps, rnd), w[pre + "norm1"], eps)
        if c.get("mlp"):
            h = rnd(x)
            y = gated_mlp(h, w, pre + "mlp.", rnd) if c["mlp"]["kind"] == "dense" else \
                mixture(h, w, pre + "mlp.", c["mlp"], rnd, router_inputs=router_inputs)
            x = x + rms_norm(y, w[pre + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return float(cap) * torch.tanh(logits / float(cap)) if cap else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=F64) -> List[int]:
    """The n_new most likely next tokens, one after another, each from a whole forward pass."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward(cfg, w, toks, dtype)[-1].argmax())
        toks.append(t)
        out.append(t)
    return out
