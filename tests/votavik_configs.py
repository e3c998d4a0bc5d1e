"""Small Votavik configurations for the tests, the weights they run with, and the comparison rule.

The configurations differ from one another in every size, in the order of the layers and in which
options are on: key and value sizes that differ or agree, one or several key/value heads, a window with
and without kept first tokens, rotation of a part of the head, of the whole head or of nothing, a decay
rank that is no multiple of eight, layers with and without a feed-forward, a model without the per-layer
token input.  Weights are drawn by the library's random-weights writer with its "loud" distributions
(every part moves the residual stream by as much as it holds) and then sharpened where a fault would
otherwise hide: sinks, decay biases and gates get values of size one."""
import json
import os

import torch
from safetensors.torch import load_file, save_file


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, "mlp": None}


def _attn(heads, kv, dim, vdim, size, keep, dims, base, scale, cap, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": size, "keep_first": keep},
         "rot": {"dims": dims, "base": base}, "scale": scale, "softcap": cap}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _light(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def _mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# P: attention first, a window of 9 with 3 kept tokens, three query heads a key head, partial rotation
VOT_P = {"architecture": "Votavik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
         "layers": [_attn(6, 2, 16, 8, 9, 3, 8, 100.0, 0.25, 30.0, _mlp(96, 1.5)),
                    _gla(2, 16, 24, 4.0, 8),
                    _light(3, 8, 16, [0.5, 0.9, 0.99], _mlp(40, 3.0)),
                    _attn(2, 2, 24, 24, 70, 0, 24, 10000.0, 0.2, 0.0, None)]}

# Q: no token input, key size equal to value size, one head everywhere, keys of 20 (no multiple of 8),
# a decay rank of 5, values of 20 (no multiple of 16), a window larger than a page, eps far from P's
VOT_Q = {"architecture": "Votavik", "vocab": 131, "width": 48, "norm": {"eps": 1e-3}, "token_side": None,
         "layers": [_light(1, 20, 20, [0.8]),
                    _gla(1, 20, 20, 1.0, 5),
                    _attn(1, 1, 20, 20, 80, 70, 0, 1.0, 0.3, 5.0, _mlp(56, 0.5)),
                    _gla(3, 8, 4, 12.0, 16)]}

# R: wider heads (keys of 72 and 136: more than 64 and 128 key channels a thread group), a window of one page
# exactly with a kept first page, every layer with a feed-forward
VOT_R = {"architecture": "Votavik", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "token_side": {"dim": 5},
         "layers": [_gla(2, 72, 40, 8.0, 24),
                    _attn(4, 1, 32, 64, 64, 64, 16, 500.0, 0.17, 40.0, _mlp(136, 2.5)),
                    _light(1, 136, 17, [0.97], _mlp(64, 2.0))]}

# S: no attention layer at all (a cache without keys and values: states only), a feed-forward on a recurrent layer
VOT_S = {"architecture": "Votavik", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "token_side": {"dim": 16},
         "layers": [_light(2, 16, 8, [0.9, 0.5], _mlp(48, 4.0)),
                    _gla(4, 8, 8, 2.0, 8)]}

CONFIGS = {"P": (VOT_P, 11), "Q": (VOT_Q, 12), "R": (VOT_R, 13), "S": (VOT_S, 14)}


def sharpen(weights, cfg, seed):
    """Values of size one where the random-weights writer draws small ones."""
    gen = torch.Generator().manual_seed(seed)
    out = dict(weights)
    for name, w in weights.items():
        if name.endswith(".sink"):
            out[name] = (1.5 * torch.randn(w.shape, generator=gen)).to(w.dtype)
        elif name.endswith(".a2.b"):
            out[name] = (2.0 + 1.5 * torch.randn(w.shape, generator=gen)).to(w.dtype)
    return out


def write_votavik(tmpdir, cfg, seed, store="bfloat16", change=None, tag=""):
    """A model folder for ``cfg``: loud random weights, sharpened; ``change(weights) -> weights`` edits them."""
    from mivi_v4_b200 import write_random_model
    d = os.path.join(str(tmpdir), f"votavik_s{seed}_{store}{tag}")
    if os.path.isdir(d):
        return d
    write_random_model(d, cfg, seed, store, "loud")
    path = os.path.join(d, "model.safetensors")
    weights = sharpen(load_file(path), cfg, seed)
    if change is not None:
        weights = change(weights)
    save_file({k: v.contiguous() for k, v in weights.items()}, path)
    return d


def read_folder(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))


def prompts(vocab, lengths, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in lengths]


def rel_rms(got, want):
    """Per row: root mean square of the difference of the logits (each row's mean taken off), divided by
    the root mean square of the wanted logits over all rows."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.isfinite(got).all()
    a, b = got - got.mean(-1, keepdim=True), want - want.mean(-1, keepdim=True)
    return (a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean().sqrt()


# float32 runs differ from the float64 plain implementation by rounding and summation order.  A bfloat16 run
# rounds its activations (2^-9) a few times a layer; how far either moves the logits is measured, not assumed: the
# plain implementation is run once more with the same roundings (``noise``), and a row of the engine may be off by
# NOISE_FACTOR times the root mean square of that difference over the sequence's rows (the engine rounds at
# slightly other places, and single rows scatter around the mean).  The faults the tests are after (a key one
# off, a lost state, a sink left out, a slot used again without zeroing) are many times larger, which
# ``test_a_lost_sink_window_edge_or_state_would_show`` holds them to.
LIMIT_F32 = 3e-5
NOISE_FACTOR = 4.0


def noise(cfg, weights, tokens, want, dtype=torch.bfloat16):
    """What rounding alone does to each row of the logits in a run of ``dtype``, on ``rel_rms``'s scale, and
    never less than twice the median of that over the rows.  A row can be far noisier than the rest:
    where a head's output is divided by its own root mean square and the head has seen one or two tokens
    only, q . k may all but cancel, and rounding moves the result by thousands of times its usual share.
    Two samples of every row's sensitivity are taken, the plain implementation in float32 throughout and
    with bfloat16 roundings between kernels (whose unit is 2^15 times larger), and the larger one counts."""
    import plain_votavik as P
    in32 = rel_rms(P.forward(cfg, weights, list(tokens), dtype=torch.float32), want)
    in16 = rel_rms(P.forward(cfg, weights, list(tokens), rnd=P.round_to(torch.bfloat16)), want)
    if dtype == torch.float32:
        own, other = in32, in16 * 2.0 ** -15
    else:
        own, other = in16, (in32 * 2.0 ** 15).clamp(max=1.0)
    return torch.maximum(torch.maximum(own, other), 2.0 * own.median())


def assert_rows(got, want, dtype, what="", noise=None):
    """``noise``: a number or one number a row (``noise()``); float32 rows are allowed LIMIT_F32 at least."""
    err = rel_rms(got, want)
    limit = NOISE_FACTOR * torch.as_tensor(noise) * torch.ones_like(err)
    if dtype == torch.float32:
        limit = limit.clamp(min=LIMIT_F32)
    worst = int((err / limit).argmax())
    assert err[worst].item() <= limit[worst].item(), \
        f"{what}: row {worst} is off by {err[worst].item():.3g} (limit {limit[worst].item():.3g})"
