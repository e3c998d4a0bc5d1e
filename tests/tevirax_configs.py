"""Small Tevirax configurations for the tests, the weights they run with, and the rounding-noise estimate.

The configurations differ from one another in every size, in the order of the layers and in which options are
on: one or several key/value heads, key and value sizes that differ or agree, a rotation of a part of the head,
of the whole head or of nothing, with and without stretched frequencies, chunks smaller and larger than a page
and no chunking at all, state space layers with one or several groups and norm parts and 1 to 5 taps, experts in
one or several groups with and without a shared expert, layers without a feed-forward, no cap on the logits.
Weights are drawn by the library's random-weights writer with its "loud" distributions and then sharpened where
a fault would otherwise hide: slow and fast decays, step-size and gate biases of size one, loud skip factors."""
import json
import math
import os

import torch
from safetensors.torch import load_file, save_file

from votavik_configs import assert_rows, prompts, read_folder, rel_rms, LIMIT_F32, NOISE_FACTOR  # noqa: F401  (generic helpers)


def _mamba(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def _par(left, right, ls, rs, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def _left(heads, kv, dim, vdim, size, rot, scale):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = rot
    return m


def _right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, ff, top, count, keep, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _yarn(dims, base, factor, original, fast=32.0, slow=1.0):
    return {"dims": dims, "base": base, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}


# A: the parallel layer first; chunks of 10 (smaller than a page, no divisor of it); three query heads a key head;
#    a rotation of 8 of 16 elements with stretched frequencies; experts in 3 groups of which 2 are kept
TEV_A = {"architecture": "Tevirax", "vocab": 97, "width": 64, "max_positions": 512, "norm": {"eps": 1e-5},
         "embedding": {"scale": 4.0}, "logit_softcap": 20.0,
         "layers": [_par(_left(6, 2, 16, 8, 10, _yarn(8, 100.0, 4.0, 64), 0.25), _right(2, 16, 24, 8.0), 0.7, 1.3,
                         _moe(12, 24, 3, 3, 2, 16)),
                    _mamba(4, 16, 24, 2, 4, 2, _dense(96)),
                    _mamba(2, 32, 16, 1, 2, 1, None),
                    _par(_left(2, 2, 24, 24, 70, {"dims": 24, "base": 10000.0}, 0.2), _right(3, 8, 16, 15.0), 1.0, 0.5,
                         _dense(40))]}

# B: one head everywhere, sizes that are no multiples of 8, no rotation, no chunking (plain causal attention), one
#    expert group, no shared expert, top 1, a convolution of one tap (no kept inputs), no cap on the logits
TEV_B = {"architecture": "Tevirax", "vocab": 131, "width": 48, "max_positions": 400, "norm": {"eps": 1e-3},
         "embedding": {"scale": 1.0},
         "layers": [_mamba(1, 20, 12, 1, 1, 1, _moe(5, 20, 1, 1, 1, 0)),
                    _par(_left(1, 1, 20, 20, 0, None, 0.3), _right(1, 20, 20, 4.0), 1.0, 1.0, None),
                    _mamba(3, 8, 20, 3, 5, 3, _dense(56))]}

# C: wider heads (states and keys of 72 and 136: more than 64 and 128 channels a thread group), a chunk of one page
#    exactly, a chunk of more than two pages, values wider than keys, all experts of the kept group chosen
TEV_C = {"architecture": "Tevirax", "vocab": 200, "width": 128, "max_positions": 600, "norm": {"eps": 1e-6},
         "embedding": {"scale": 11.0}, "logit_softcap": 50.0,
         "layers": [_mamba(2, 40, 72, 1, 3, 2, _moe(8, 32, 2, 4, 1, 48)),
                    _par(_left(4, 1, 32, 64, 64, _yarn(16, 500.0, 2.0, 128, 8.0, 2.0), 0.17), _right(1, 136, 17, 9.0), 0.6, 1.4,
                         _moe(6, 16, 4, 2, 2, 8)),
                    _mamba(1, 24, 136, 1, 4, 1, None),
                    _par(_left(2, 1, 64, 32, 150, _yarn(64, 50000.0, 8.0, 256), 0.125), _right(2, 72, 40, 30.0), 1.2, 0.9,
                         _dense(136))]}

# D: no attention-free layer at all is not possible here (every layer has a mixer); this one has no parallel
#    layer: a cache without keys and values (states only)
TEV_D = {"architecture": "Tevirax", "vocab": 77, "width": 40, "max_positions": 300, "norm": {"eps": 1e-5},
         "embedding": {"scale": 2.0}, "logit_softcap": 8.0,
         "layers": [_mamba(2, 16, 8, 2, 3, 4, _moe(4, 16, 2, 2, 1, 8)),
                    _mamba(4, 8, 8, 1, 4, 1, _dense(48))]}

CONFIGS = {"A": (TEV_A, 21), "B": (TEV_B, 22), "C": (TEV_C, 23), "D": (TEV_D, 24)}


ROUTE_PUSH = 16.0


def route_direction(cfg, seed):
    """The unit vector of the stream that "two_way" routers read."""
    u = torch.randn(cfg["width"], generator=torch.Generator().manual_seed(1000 + seed))
    return u / u.norm()


def sharpen(weights, cfg, seed, router="random"):
    """Values of size one where the random-weights writer draws small ones.  ``router`` = "random" leaves the
    routers' rows as drawn.  "two_way": every router's rows are multiples of ONE direction u of the stream, so the
    order of the scores, and of the groups' sums of scores, depends on the sign of u . h only, and the position table carries ``ROUTE_PUSH`` u with a
    sign that changes every three positions: u . h stays far from zero, and a bfloat16 run (whose activations carry
    a relative noise of 2^-9) chooses the experts that the plain implementation chooses, while tokens still take
    one of two routes."""
    gen = torch.Generator().manual_seed(seed)
    out = dict(weights)
    u = route_direction(cfg, seed)
    if router == "two_way":
        pos = weights["pos"].float()
        sign = 1.0 - 2.0 * ((torch.arange(pos.shape[0]) // 3) % 2)
        out["pos"] = (pos + ROUTE_PUSH * sign[:, None] * u[None, :]).to(weights["pos"].dtype)

    def rand(shape):
        return torch.randn(shape, generator=gen)
    for name, w in weights.items():
        if name.endswith(".A_log"):           # decays from e^-0.02 dt to e^-dt
            out[name] = torch.log(0.02 + 0.98 * torch.rand(w.shape, generator=gen)).to(w.dtype)
        elif name.endswith(".dt_bias"):
            out[name] = (-1.0 + rand(w.shape)).to(w.dtype)
        elif name.endswith(".D"):
            out[name] = rand(w.shape).to(w.dtype)
        elif name.endswith(".f.b"):           # forget gates near one: a long memory
            out[name] = (3.0 + rand(w.shape)).to(w.dtype)
        elif name.endswith(".i.b"):
            out[name] = rand(w.shape).to(w.dtype)
        elif name.endswith((".mix.right.i", ".mix.right.f")):
            out[name] = (3.0 * w.float()).to(w.dtype)
        elif name.endswith(".router") and router == "two_way":
            E, W = w.shape
            # unevenly spaced factors, ascending, dealt to the groups in runs (every factor of one group above every
            # factor of the next, so the groups' sums of scores keep their order whatever |u . h| is), then the groups
            # and the experts inside a group shuffled
            count = int((cfg["layers"][int(name.split(".")[0][1:])]["mlp"]["router"].get("groups") or {"count": 1})["count"])
            factors = (4.0 * torch.linspace(0.0, 1.0, E) ** 1.5 - 1.5).view(count, E // count)
            factors = factors[torch.randperm(count, generator=gen)]
            factors = torch.stack([row[torch.randperm(E // count, generator=gen)] for row in factors]).flatten()
            out[name] = (factors[:, None] * (1.8 / ROUTE_PUSH) * u[None, :]).to(w.dtype)
    return out


def write_tevirax(tmpdir, cfg, seed, store="bfloat16", change=None, tag="", router="random"):
    """A model folder for ``cfg``: loud random weights, sharpened; ``change(weights) -> weights`` edits them."""
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"tevirax_s{seed}_{store}_{router}{tag}")
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


def noise(cfg, weights, tokens, want, dtype=torch.bfloat16):
    """What rounding alone does to each row of the logits in a run of ``dtype``, on ``rel_rms``'s scale, and never
    less than twice the median of that over the rows.  Two samples of every row's sensitivity are taken, the plain
    implementation in float32 throughout and with bfloat16 roundings between kernels (whose unit is 2^15 times
    larger), and the larger one counts."""
    import plain_tevirax as P
    in32 = rel_rms(P.forward(cfg, weights, list(tokens), dtype=torch.float32), want)
    in16 = rel_rms(P.forward(cfg, weights, list(tokens), rnd=P.round_to(torch.bfloat16)), want)
    if dtype == torch.float32:
        own, other = in32, in16 * 2.0 ** -15
    else:
        own, other = in16, (in32 * 2.0 ** 15).clamp(max=1.0)
    return torch.maximum(torch.maximum(own, other), 2.0 * own.median())

