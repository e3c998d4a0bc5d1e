"""The plain Tevirax implementation against closed forms (no GPU), and the parts of the package that need no GPU:
the configuration reader, the name table, the stretched rotation's frequencies, the cache's pages under a chunked
mask."""
import json
import math

import pytest
import torch

import plain_tevirax as P
from tevirax_configs import CONFIGS, TEV_A, TEV_B

F64 = torch.float64


def test_chunked_mask_sees_its_own_chunk_only():
    ok = P.visible(25, {"size": 10})
    for i in range(25):
        for j in range(25):
            assert bool(ok[i, j]) == (j <= i and i // 10 == j // 10)
    assert bool(P.visible(5, None).equal(torch.tril(torch.ones(5, 5, dtype=torch.bool))))
    # the first token of a chunk sees itself alone; the last one the whole chunk
    assert ok[10].sum() == 1 and ok[19].sum() == 10 and ok[20].sum() == 1


def test_rotation_pairs_frequencies_and_amplitude():
    rot = {"dims": 8, "base": 100.0}
    f, amp = P.rotary_frequencies(rot)
    assert amp == 1.0 and torch.allclose(f, torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=F64))
    x = torch.randn(3, 2, 12, dtype=F64)
    y = P.rotate(x, torch.tensor([0, 5, 9]), rot)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])          # position 0 and the unrotated rest
    a = 5 * f[1]
    assert torch.allclose(y[1, :, 1], x[1, :, 1] * math.cos(a) - x[1, :, 5] * math.sin(a))
    assert torch.allclose(y[1, :, 5], x[1, :, 5] * math.cos(a) + x[1, :, 1] * math.sin(a))
    # stretched: high frequencies stay, low ones are divided by the factor, lengths grow by 0.1 ln(factor) + 1
    rs = {"dims": 32, "base": 10000.0, "scaling": {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0}}
    fs, amp = P.rotary_frequencies(rs)
    f0, _ = P.rotary_frequencies({"dims": 32, "base": 10000.0})
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert fs[0] == f0[0] and fs[-1] == pytest.approx(float(f0[-1]) / 4.0)
    assert ((fs <= f0) & (fs >= f0 / 4.0)).all()
    z = P.rotate(x.new_ones(1, 1, 32), torch.tensor([3]), rs)
    assert torch.allclose(z[0, 0, :16] ** 2 + z[0, 0, 16:] ** 2, torch.full((16,), 2 * amp * amp, dtype=F64))


def test_package_rotation_has_the_plain_frequencies():
    from mivi_v4_b200.parts.position import YarnRope
    for rot in (TEV_A["layers"][0]["mixer"]["left"]["rot"], {"dims": 64, "base": 50000.0, "scaling": {"factor": 8.0, "original": 256, "fast": 32.0, "slow": 1.0}},
                {"dims": 16, "base": 500.0, "scaling": {"factor": 2.0, "original": 128, "fast": 8.0, "slow": 2.0}}):
        sc = rot["scaling"]
        part = YarnRope(rot["dims"], rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
        inv, half = part.rotary("cpu")
        f, amp = P.rotary_frequencies(rot)
        assert half and torch.equal(inv, f.to(torch.float32)) and part.amplitude() == pytest.approx(amp)


def test_state_space_scan_is_the_explicit_sum():
    T, N, Pd = 9, 5, 3
    x, B, C = torch.randn(T, Pd, dtype=F64), torch.randn(T, N, dtype=F64), torch.randn(T, N, dtype=F64)
    dt, A, D = torch.rand(T, dtype=F64) + 0.1, torch.tensor(-0.7, dtype=F64), torch.tensor(0.3, dtype=F64)
    y = P.state_space_scan(x, B, C, dt, A, D)
    for t in range(T):
        want = D * x[t]
        for s in range(t + 1):
            want = want + torch.exp(A * dt[s + 1:t + 1].sum()) * dt[s] * (B[s] @ C[t]) * x[s]
        assert torch.allclose(y[t], want)


def test_matrix_memory_scan_is_the_unstabilised_form():
    T, dk, dv = 12, 4, 3
    q, k, v = torch.randn(T, dk, dtype=F64), torch.randn(T, dk, dtype=F64), torch.randn(T, dv, dtype=F64)
    i_log, f_log = torch.randn(T, dtype=F64), -torch.rand(T, dtype=F64)
    o = P.matrix_memory_scan(q, k, v, i_log, f_log)
    S, n, m = torch.zeros(dk, dv, dtype=F64), torch.zeros(dk, dtype=F64), 0.0
    for t in range(T):                      # without the running maximum: C = sum of e^(gates) k v^T, rescaled at the end
        S = math.exp(f_log[t]) * S + math.exp(i_log[t]) * k[t][:, None] * v[t][None, :]
        n = math.exp(f_log[t]) * n + math.exp(i_log[t]) * k[t]
        m = max(float(f_log[t]) + m, float(i_log[t]))
        # the state above carries e^(sum f) from a start at m = 0; the stabilised one is it times e^(-m)
        want = (S.T @ q[t]) * math.exp(-m) / (max(abs(float(n @ q[t])) * math.exp(-m), math.exp(-m)) + 1e-6)
        assert torch.allclose(o[t], want)


def test_causal_taps_last_column_is_the_current_token():
    u = torch.randn(6, 2, dtype=F64)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=F64)
    out = P.causal_taps(u, taps, torch.zeros(2, dtype=F64))
    assert torch.equal(out[:, 0], u[:, 0])
    assert torch.equal(out[2:, 1], u[:-2, 1]) and torch.equal(out[:2, 1], torch.zeros(2, dtype=F64))


def test_router_groups_top_and_weights():
    w_router = torch.eye(6, dtype=F64)
    h = torch.tensor([[3.0, 2.9, -5.0, 2.0, 1.0, 0.5]], dtype=F64)
    # groups (0,1,2), (3,4,5): sums of the two largest sigmoids 1.90 and 1.61: only the first group may be chosen
    pick, wgt = P.route(h, w_router, {"experts": 6, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert pick.tolist() == [[0, 1]]
    s = torch.sigmoid(h[0])
    assert torch.allclose(wgt[0], s[:2] / s[:2].sum())
    pick, _ = P.route(h, w_router, {"experts": 6, "top": 3, "groups": {"count": 2, "keep": 2}})
    assert pick.tolist() == [[0, 1, 3]]
    pick, _ = P.route(h, w_router, {"experts": 6, "top": 3})
    assert pick.tolist() == [[0, 1, 3]]


def test_config_reader_and_name_table():
    from mivi_v4_b200.config import ConfigError, TeviraxConfig
    from mivi_v4_b200.engine.model import expected_tensors
    for cfg, _ in CONFIGS.values():
        c = TeviraxConfig.from_dict(cfg)
        assert len(c.layers) == len(cfg["layers"]) and c.embedding_scale == cfg["embedding"]["scale"]
    names = expected_tensors(TEV_A)
    assert names["embed"].shape == (97, 64) and names["pos"].shape == (512, 64)
    assert names["l0.mix.left.q.norm"].shape == (16,) and names["l0.mix.left.o"].shape == (64, 48)
    assert names["l0.mix.right.i.b"].shape == (2,) and names["l0.mlp.shared.sg"].shape == (1, 64)
    assert names["l0.mlp.e11.down"].shape == (64, 24) and "l0.mlp.e12.down" not in names
    assert names["l1.mix.in"].shape == (2 * 64 + 2 * 2 * 24 + 4, 64) and names["l1.mix.conv"].shape == (64 + 96, 4)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names and names["l3.mlp.gate"].shape == (40, 64)
    assert "l1.mlp.router" not in expected_tensors(TEV_B) and "l0.mlp.shared.sg" not in expected_tensors(TEV_B)
    without = {k: v for k, v in TEV_A.items() if k != "max_positions"}       # the table's length is then the checkpoint's to say
    assert expected_tensors(without)["pos"].shape == (None, 64)

    def broken(edit):
        c = json.loads(json.dumps(TEV_A))
        edit(c)
        with pytest.raises(ConfigError):
            TeviraxConfig.from_dict(c)
    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4))
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda c: c["layers"][1]["mixer"].update(groups=3))
    broken(lambda c: c["layers"][1]["mixer"].update(norm_groups=7))
    broken(lambda c: c.update(max_positions=0))
    broken(lambda c: c["layers"][0]["mixer"]["right"].update(gate_cap=0))


def test_pages_before_the_current_chunk_go_back():
    from mivi_v4_b200.cache import KVNeed, SequenceCache, plan_cache
    cache = SequenceCache(plan_cache([KVNeed(1, 8, chunk=20)], [None]), n_slots=2, n_pages=6, page_size=8, device="cpu")
    s = cache.assign()
    cache.reserve(s, 45)
    cache.advance(s, 45)                   # the next token, 45, reads from 40 on: blocks 0..4 (tokens 0..39) are free
    assert cache.pages[0].free_count == 5
    cache.reserve(s, 3)
    cache.advance(s, 3)                    # 48: still chunk 40..59, still inside the page of tokens 40..47
    assert cache.pages[0].free_count == 5
    cache.reserve(s, 12)
    cache.advance(s, 12)                   # 60: a new chunk starts; everything before it goes back
    assert cache.pages[0].free_count == 6 - 1
    cache.check()
    cache.release(s)
    assert cache.pages[0].free_count == 6


def test_two_way_routers_stay_far_from_a_close_call(tmp_path):
    """The weights of the bfloat16 engine tests: every mixture layer's input keeps |u . h| far from zero, where the
    order of its router's scores would turn over, and both routes are taken."""
    from tevirax_configs import prompts, read_folder, route_direction, write_tevirax
    for name, (cfg, seed) in CONFIGS.items():
        c, w = read_folder(write_tevirax(tmp_path, cfg, seed, router="two_way"))
        inputs = []
        P.forward(c, w, prompts(cfg["vocab"], [150], seed)[0], router_inputs=inputs)
        assert inputs, name
        u = route_direction(cfg, seed).double()
        for h in inputs:
            x = h @ u
            assert x.abs().min() > 4.0, (name, float(x.abs().min()))
            assert (x > 0).any() and (x < 0).any()


def test_command_line_writes_and_describes_a_model_folder(tmp_path, capsys):
    from mivi_v4_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TEV_A))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--seed", "1", "--out", str(out)]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "architecture: Tevirax" in text and "logit_softcap: 20.0" in text
    assert "l0.mix.left.q.norm" in text and "l0.mix.right.f.b" in text and "l0.mlp.e11.down" in text and "l1.mix.A_log" in text
