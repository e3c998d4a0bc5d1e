"""The plain Votavik implementation against closed forms, one mechanism at a time, and the configuration
reader and name table of the library (no GPU)."""
import math

import pytest
import torch

import plain_votavik as P
from votavik_configs import CONFIGS, VOT_P

F64 = torch.float64


def test_window_keeps_the_first_tokens():
    assert P.visible(10, 10, 4, 0) and P.visible(10, 7, 4, 0) and not P.visible(10, 6, 4, 0)
    assert not P.visible(10, 11, 4, 0)
    assert P.visible(10, 1, 4, 2) and not P.visible(10, 2, 4, 2) and P.visible(10, 0, 4, 2)


def test_decayed_scan_is_the_weighted_sum():
    torch.manual_seed(0)
    T, dk, dv = 7, 3, 2
    q, k, v = torch.randn(T, dk, dtype=F64), torch.randn(T, dk, dtype=F64), torch.randn(T, dv, dtype=F64)
    a = torch.rand(T, dk, dtype=F64)
    o, S = P.decayed_outer_scan(q, k, v, a)
    for t in range(T):
        want = torch.zeros(dv, dtype=F64)
        for s in range(t + 1):
            w = torch.ones(dk, dtype=F64)
            for r in range(s + 1, t + 1):
                w = w * a[r]
            want += (q[t] * w * k[s]).sum() * v[s]
        assert torch.allclose(o[t], want, atol=1e-12)
    assert S.shape == (dk, dv)


def test_partial_rotation_turns_pairs_and_leaves_the_rest():
    x = torch.randn(5, 2, 12, dtype=F64)
    pos = torch.tensor([0, 1, 2, 30, 31])
    y = P.rotate_partial(x, pos, 8, 100.0)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :8].pow(2).sum(-1), x[..., :8].pow(2).sum(-1))
    # pair (i, i + 4) at position p turns by p * base^(-2 i / 8)
    ang = 30 * 100.0 ** (-2 * 1 / 8)
    u, v = x[3, 0, 1], x[3, 0, 5]
    assert torch.allclose(y[3, 0, 1], u * math.cos(ang) - v * math.sin(ang))
    assert torch.allclose(y[3, 0, 5], v * math.cos(ang) + u * math.sin(ang))


def _attention_case(sink_value, T=6):
    torch.manual_seed(1)
    c = {"mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "mask": {"size": 100, "keep_first": 0},
                   "rot": {"dims": 0, "base": 1.0}, "scale": 0.5, "softcap": 0.0}}
    W = 8
    w = {"m.q": torch.randn(8, W, dtype=F64), "m.k": torch.randn(4, W, dtype=F64), "m.v": torch.randn(3, W, dtype=F64),
         "m.q.norm": torch.ones(8, dtype=F64), "m.k.norm": torch.ones(4, dtype=F64),
         "m.sink": torch.full((2,), sink_value, dtype=F64), "m.g": torch.zeros(2, W, dtype=F64),
         "m.o": torch.eye(6, dtype=F64)}
    return c, w, torch.randn(T, W, dtype=F64)


def test_sink_counts_once_and_has_no_value():
    c, w, h = _attention_case(-1e9)
    free = P.attention_mixer(h, w, "m.", c, 1e-5)
    c, w, h = _attention_case(0.7)
    with_sink = P.attention_mixer(h, w, "m.", c, 1e-5)
    # the first token sees itself only: weight e^s / (e^s + e^sink), gate sigmoid(0) = 1/2
    q = P.rms_unit(h[:1] @ w["m.q"].T, 1e-5)[0, :4]
    k = P.rms_unit(h[:1] @ w["m.k"].T, 1e-5)[0]
    s = (q @ k) * 0.5
    v = h[0] @ w["m.v"].T
    assert torch.allclose(with_sink[0, :3], 0.5 * v * torch.exp(s) / (torch.exp(s) + math.exp(0.7)))
    assert torch.allclose(free[0, :3], 0.5 * v)


def test_softcap_bounds_the_scores():
    c, w, h = _attention_case(0.0)
    c["mixer"]["softcap"] = 1e-3          # every score is squeezed to about 0: uniform weights over the keys and the sink
    w["m.sink"] = torch.zeros(2, dtype=F64)
    out = P.attention_mixer(h, w, "m.", c, 1e-5)
    v = h @ w["m.v"].T
    assert torch.allclose(out[2, :3], 0.5 * v[:3].sum(0) / 4, atol=1e-3)


def test_dense_feed_forward_clamps():
    c = {"mlp": {"limit": 1.0}}
    w = {"f.gate": torch.tensor([[10.0], [-10.0]], dtype=F64), "f.up": torch.tensor([[10.0], [-10.0]], dtype=F64),
         "f.down": torch.eye(2, dtype=F64)}
    y = P.dense_ff(torch.ones(1, 1, dtype=F64), w, "f.", c)
    # gate 10 -> 1 (capped above only), up 10 -> 1; gate -10 stays, up -10 -> -1 so (u + 1) = 0
    assert torch.allclose(y[0, 0], 2.0 * torch.sigmoid(torch.tensor(1.702, dtype=F64)))
    assert y[0, 1].abs() < 1e-12


def test_layer_norm_uses_the_mean_of_squared_deviations():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=F64)
    y = P.layer_norm(x, torch.ones(4, dtype=F64), 0.0)
    assert torch.allclose(y.mean(), torch.tensor(0.0, dtype=F64), atol=1e-12)
    assert torch.allclose(y.pow(2).mean(), torch.tensor(1.0, dtype=F64))


def test_name_table_and_config_errors():
    from mivi_v4_b200 import ConfigError
    from mivi_v4_b200.engine.model import describe_config, expected_tensors
    names = expected_tensors(VOT_P)
    assert names["embed"].shape == (97, 64) and names["side.embed"].shape == (97, 4 * 8)
    assert names["l0.mix.q.norm"].shape == (6 * 16,) and names["l0.mix.g"].shape == (6, 64)
    assert names["l1.mix.a1"].shape == (8, 64) and names["l1.mix.a2.b"].shape == (32,)
    assert "l1.norm2" not in names and "l0.norm2" in names and "l3.mlp.up" not in names
    assert names["l2.mix.norm"].shape == (48,) and names["l1.mix.norm"].shape == (24,)
    for cfg, _ in CONFIGS.values():
        describe_config(cfg)
    bad = dict(VOT_P, layers=[dict(VOT_P["layers"][0], type="conv")])
    with pytest.raises(ConfigError):
        describe_config(bad)
    bad = dict(VOT_P, layers=[{"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "decay": [0.5]}, "mlp": None}])
    with pytest.raises(ConfigError):
        describe_config(bad)
    with pytest.raises(ConfigError):
        describe_config({k: v for k, v in VOT_P.items() if k != "width"})


def test_window_cache_keeps_the_pages_of_the_first_tokens():
    from mivi_v4_b200.cache import KVNeed, SequenceCache, plan_cache
    need = KVNeed(2, 8, window=10, v_dim=4, keep_first=5)
    cache = SequenceCache(plan_cache([need], [None]), n_slots=2, n_pages=8, page_size=4, dtype=torch.float32, device="cpu")
    s = cache.assign()
    cache.reserve(s, 30)
    cache.advance(s, 30)
    # the next token (30) reads keys 21.. and 0..4: blocks 0 and 1 stay, blocks 2..4 go, block 5 (20..23) stays
    held = [p is not None for p in cache._get(s).pages[0]]
    assert held == [True, True, False, False, False, True, True, True]
    assert cache.storage[0].shape == (1, 8, 2 * 4 * (8 + 4))
    cache.check()
    cache.release(s)
    cache.check()
    assert cache.pages[0].free_count == 8


def test_command_line_random_then_info_and_a_checkpoint_that_gives_the_rank(tmp_path, capsys):
    import json
    from safetensors.torch import load_file
    from mivi_v4_b200 import WeightsError
    from mivi_v4_b200.cli import main
    from mivi_v4_b200.engine.model import expected_tensors
    from mivi_v4_b200.weights.loader import check_entries
    from mivi_v4_b200.weights.safetensors_io import read_model_headers
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(VOT_P))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "3", "--out", str(out)]) == 0
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Votavik" in text and "side.embed" in text and "l1.mix.a2.b" in text
    weights = load_file(str(out / "model.safetensors"))
    assert weights["l1.mix.a1"].shape == (8, 64) and weights["l0.mix.sink"].shape == (6,)
    # a configuration without the decay's rank takes it from the checkpoint: any rank fits the name table,
    # but the two projections must still have the declared outer sizes
    no_rank = json.loads(json.dumps(VOT_P))
    del no_rank["layers"][1]["mixer"]["rank"]
    check_entries("the folder", expected_tensors(no_rank), read_model_headers(str(out)))
    wrong = json.loads(json.dumps(no_rank))
    wrong["layers"][1]["mixer"]["dim"] = 24
    with pytest.raises(WeightsError):
        check_entries("the folder", expected_tensors(wrong), read_model_headers(str(out)))
    with pytest.raises(ValueError):
        main(["random", "--config", str(_write(tmp_path / "c2.json", no_rank)), "--out", str(tmp_path / "m2")])


def _write(path, cfg):
    import json
    path.write_text(json.dumps(cfg))
    return path
