"""Every kernel that the Tevirax decoder added, alone, against the plain implementation's function of the same
mechanism (float64), at sizes of the tests' own: the scalar-decay recurrence as a state space layer and as a
matrix memory (any cut, slots used again, groups of heads, wide keys), the log gates and their running maximum,
the causal convolution (any cut, 1 to 7 taps), the step size, the router and the routed activation, the per-head
q/k norm with a stretched rotation, attention under a chunked mask (keys far away, just inside and just outside a
chunk, in long steps and token by token), the gate before the grouped norm, the post-norm sum, the scaled
embedding with positions, the capped logits."""
import math

import pytest
import torch

import plain_tevirax as P

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda:0"


def K():
    from mivi_v4_b200.ops import kernels
    return kernels


def dev(x, dtype=torch.float32):
    return x.to(dtype).to(DEV).contiguous()


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def close(got, want, tol=2e-5, what=""):
    got, want = got.detach().double().cpu(), want.double()
    assert torch.isfinite(got).all(), what
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err <= tol, f"{what}: off by {err:.3g} of the largest value (limit {tol})"


def cuts_of(T):
    return [[T], [1] * T, [2] * (T // 2) + ([T % 2] if T % 2 else []), [5, 1, T - 6] if T > 7 else [T], [T - 1, 1]]


# ------------------------------------------------------------------------------------------ recurrence
@pytest.mark.parametrize("H,G,N,Pd", [(4, 2, 24, 16), (1, 1, 8, 3), (3, 3, 72, 20), (2, 1, 136, 33)])
def test_scalar_scan_as_a_state_space_layer_under_every_cut(H, G, N, Pd):
    k = K()
    T = 37
    g = torch.Generator().manual_seed(H * 100 + N)
    x = torch.randn(T, H, Pd, generator=g, dtype=F64)
    B, C = torch.randn(T, G, N, generator=g, dtype=F64), torch.randn(T, G, N, generator=g, dtype=F64)
    dt = torch.rand(T, H, generator=g, dtype=F64) * 2 + 0.01
    A, D = -torch.rand(H, generator=g, dtype=F64) * 2 - 0.01, torch.randn(H, generator=g, dtype=F64)
    want = torch.cat([P.state_space_scan(x[:, a], B[:, a // (H // G)], C[:, a // (H // G)], dt[:, a], A[a], D[a]) for a in range(H)], -1)
    # q, k, v as column slices of one wide matrix, as the layer has them
    wide = dev(torch.cat([x.reshape(T, -1), B.reshape(T, -1), C.reshape(T, -1)], -1))
    inner, gn = H * Pd, G * N
    log_a, b = dev(A[None, :] * dt), dev(dt)
    first = None
    for cuts in cuts_of(T):
        state = torch.zeros(3, H, Pd, N, device=DEV)
        state[0].fill_(7.0)                      # another sequence's slot must stay as it is
        outs, at = [], 0
        for n in cuts:
            rows = slice(at, at + n)
            out = torch.full((n, inner), float("nan"), device=DEV)
            k.scalar_scan(wide[rows, inner + gn:], wide[rows, inner:inner + gn], wide[rows, :inner], log_a[rows], b[rows],
                          state, i32([2]), i32([0, n]), out, 1, H, N, Pd, heads_per_group=H // G, skip=dev(D))
            outs.append(out)
            at += n
        got = torch.cat(outs)
        close(got, want, 2e-5, f"cuts {cuts[:4]}")
        first = got if first is None else first
        assert torch.equal(got, first), "a cut changes the numbers of the token-by-token kernel"
        assert torch.equal(state[0], torch.full_like(state[0], 7.0)) and state[1].abs().max() == 0


def test_scalar_scan_batches_and_slots_used_again():
    k = K()
    H, N, Pd = 2, 16, 8
    g = torch.Generator().manual_seed(5)
    lens = [9, 1, 30]
    seqs = [(torch.randn(n, H, N, generator=g, dtype=F64), torch.randn(n, H, N, generator=g, dtype=F64),
             torch.randn(n, H, Pd, generator=g, dtype=F64), -torch.rand(n, H, generator=g, dtype=F64),
             torch.rand(n, H, generator=g, dtype=F64)) for n in lens]

    def plain(q, kk, v, la, b):
        S = torch.zeros(H, N, Pd, dtype=F64)
        out = []
        for t in range(q.shape[0]):
            S = torch.exp(la[t])[:, None, None] * S + b[t][:, None, None] * kk[t][:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hnp,hn->hp", S, q[t]).reshape(-1))
        return torch.stack(out)
    cat = [dev(torch.cat([s[i].reshape(s[i].shape[0], -1) for s in seqs])) for i in range(5)]
    state = torch.zeros(4, H, Pd, N, device=DEV)
    for _ in range(2):                            # the second time the slots hold the first run's states: zero them as the cache does
        state.zero_()
        out = torch.empty(sum(lens), H * Pd, device=DEV)
        k.scalar_scan(cat[0], cat[1], cat[2], cat[3], cat[4], state, i32([3, 0, 1]), i32([0, 9, 10, 40]), out, 3, H, N, Pd)
        close(out, torch.cat([plain(*s) for s in seqs]), 2e-5, "batch of three")


@pytest.mark.parametrize("H,dk,dv", [(3, 16, 24), (1, 136, 5), (2, 72, 40)])
def test_scalar_scan_as_a_matrix_memory_with_its_gates(H, dk, dv):
    k = K()
    T, cap = 41, 6.0
    g = torch.Generator().manual_seed(dk)
    q, kk = torch.randn(T, H, dk, generator=g, dtype=F64), torch.randn(T, H, dk, generator=g, dtype=F64)
    v = torch.randn(T, H, dv, generator=g, dtype=F64)
    zi, zf = 4 * torch.randn(T, H, generator=g, dtype=F64), 4 * torch.randn(T, H, generator=g, dtype=F64) + 2
    bi, bf = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    i_log = cap * torch.tanh((zi + bi) / cap)
    f_log = P.log_sigmoid(cap * torch.tanh((zf + bf) / cap))
    want = torch.cat([P.matrix_memory_scan(q[:, a] * dk ** -0.5, kk[:, a], v[:, a], i_log[:, a], f_log[:, a]) for a in range(H)], -1)
    qd, kd, vd = dev(q.reshape(T, -1)), dev(kk.reshape(T, -1)), dev(v.reshape(T, -1))
    gates = dev(torch.cat([zi, zf], -1))
    for cuts in cuts_of(T):
        memory, maxima = torch.zeros(2, H, dv + 1, dk, device=DEV), torch.zeros(2, H, device=DEV)
        outs, at = [], 0
        for n in cuts:
            rows = slice(at, at + n)
            log_a, b, m = (torch.empty(n, H, device=DEV) for _ in range(3))
            k.memory_gates(gates[rows, :H], gates[rows, H:], dev(bi), dev(bf), cap, maxima, i32([1]), i32([0, n]), log_a, b, m, 1, H)
            out = torch.full((n, H * dv), float("nan"), device=DEV)
            k.scalar_scan(qd[rows], kd[rows], vd[rows], log_a, b, memory, i32([1]), i32([0, n]), out, 1, H, dk, dv, m_tok=m,
                          q_scale=dk ** -0.5)
            outs.append(out)
            at += n
        close(torch.cat(outs), want, 5e-5, f"cuts {cuts[:4]}")
        assert memory[0].abs().max() == 0 and maxima[0].abs().max() == 0


def test_memory_gates_running_maximum_starts_at_zero_not_at_minus_infinity():
    k = K()
    H, T = 2, 6
    zi, zf = torch.full((T, H), -3.0, dtype=F64), torch.full((T, H), 5.0, dtype=F64)      # i far below 0: m stays near 0
    maxima = torch.zeros(1, H, device=DEV)
    log_a, b, m = (torch.empty(T, H, device=DEV) for _ in range(3))
    zero = torch.zeros(H, device=DEV)
    k.memory_gates(dev(zi), dev(zf), zero, zero, 50.0, maxima, i32([0]), i32([0, T]), log_a, b, m, 1, H)
    f = P.log_sigmoid(50.0 * torch.tanh(zf / 50.0))
    il = 50.0 * torch.tanh(zi / 50.0)
    want_m = torch.cumsum(f, 0)                                # max(f + m, i) = f + m while that is above -3
    close(m, want_m, 1e-5, "m")
    close(b, torch.exp(il - want_m), 1e-5, "b")
    assert (log_a.abs() < 1e-6).all()                          # f + m_(t-1) - m_t = 0 while the forget path wins


# ------------------------------------------------------------------------------------------ convolution, step size
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_convolution_under_every_cut(taps):
    k = K()
    T, C = 23, 37
    g = torch.Generator().manual_seed(taps)
    u, w, bias = torch.randn(T, C + 5, generator=g, dtype=F64), torch.randn(C, taps, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    want = P.silu(P.causal_taps(u[:, 2:2 + C], w, bias))
    ud = dev(u)
    for cuts in cuts_of(T):
        state = torch.zeros(3, max(taps - 1, 0), C, device=DEV)
        outs, at = [], 0
        for n in cuts:
            out = torch.full((n, C), float("nan"), device=DEV)
            seq_of = i32([0] * n)
            k.causal_conv_silu(ud[at:at + n, 2:2 + C], dev(w), dev(bias), state, seq_of, i32([0, n]), i32([1]), out, 1)
            outs.append(out)
            at += n
        close(torch.cat(outs), want, 1e-5, f"taps {taps} cuts {cuts[:4]}")
        if taps > 1:
            close(state[1], u[T - (taps - 1):, 2:2 + C] if T >= taps - 1 else None, 1e-6, "kept inputs")
            assert state[0].abs().max() == 0 and state[2].abs().max() == 0


def test_causal_convolution_of_a_batch():
    k = K()
    C, taps = 9, 4
    g = torch.Generator().manual_seed(1)
    lens = [1, 6, 2]
    us = [torch.randn(n, C, generator=g, dtype=F64) for n in lens]
    w, bias = torch.randn(C, taps, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    state = torch.zeros(3, taps - 1, C, device=DEV)
    out = torch.empty(sum(lens), C, device=DEV)
    k.causal_conv_silu(dev(torch.cat(us)), dev(w), dev(bias), state, i32([0, 1, 1, 1, 1, 1, 1, 2, 2]), i32([0, 1, 7, 9]), i32([2, 0, 1]), out, 3)
    close(out, torch.cat([P.silu(P.causal_taps(u, w, bias)) for u in us]), 1e-5, "batch")


def test_step_size():
    k = K()
    raw = torch.tensor([[-30.0, -1.0, 0.0], [2.0, 25.0, 60.0]], dtype=F64)
    bias, a_log = torch.tensor([0.5, -0.5, 0.0], dtype=F64), torch.tensor([0.0, -2.0, 1.0], dtype=F64)
    log_a, b = torch.empty(2, 3, device=DEV), torch.empty(2, 3, device=DEV)
    k.step_size(dev(raw), dev(bias), dev(a_log), log_a, b)
    dt = P.softplus(raw + bias)
    close(b, dt, 1e-6, "dt")
    close(log_a, -torch.exp(a_log) * dt, 1e-6, "log a")


# ------------------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("E,count,keep,top,shared", [(16, 4, 1, 3, True), (12, 3, 2, 3, True), (5, 1, 1, 1, False),
                                                      (8, 4, 1, 2, False), (64, 8, 3, 6, True), (6, 6, 2, 2, False)])
def test_router_and_routed_activation(E, count, keep, top, shared):
    k = K()
    N, ff, sff = 50, 8, (6 if shared else 0)
    g = torch.Generator().manual_seed(E)
    z = 2 * torch.randn(N, E + 1 + 3, generator=g, dtype=torch.float32)
    cols = E + (1 if shared else 0)
    pick_w, wgt_w = P.route(z[:, :E].double(), torch.eye(E, dtype=F64), {"experts": E, "top": top, "groups": {"count": count, "keep": keep}})
    dense, pick, pw = torch.empty(N, cols, device=DEV), torch.empty(N, top, dtype=torch.int32, device=DEV), torch.empty(N, top, device=DEV)
    k.route(dev(z)[:, :cols], dense, pick, pw, E, count, keep, top, shared)
    assert torch.equal(pick.cpu().long().sort(-1).values, pick_w.sort(-1).values)
    want = torch.zeros(N, cols, dtype=F64)
    want[:, :E].scatter_(1, pick_w, wgt_w)
    if shared:
        want[:, E] = torch.sigmoid(z[:, E].double())
    close(dense, want, 1e-6, "dense weights")
    assert ((dense[:, :E] != 0).sum(-1) == top).all()
    F = E * ff + sff
    gate, up = torch.randn(N, F, generator=g, dtype=torch.float32), torch.randn(N, F, generator=g, dtype=torch.float32)
    # every expert's gates and ups together: the gates, then the ups
    blocks = [torch.cat([gate[:, e * ff:(e + 1) * ff], up[:, e * ff:(e + 1) * ff]], 1) for e in range(E)]
    if shared:
        blocks.append(torch.cat([gate[:, E * ff:], up[:, E * ff:]], 1))
    gu = torch.cat(blocks, 1)
    col_w = torch.cat([want[:, :E].repeat_interleave(ff, 1)] + ([want[:, E:].expand(N, sff)] if shared else []), 1)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 4e-3)):
        hid = torch.full((N, F), float("nan"), dtype=dtype, device=DEV)
        k.routed_glu(dev(gu), dense, hid, E, ff, sff)
        close(hid, col_w * P.silu(gate.double()) * up.double(), tol, f"routed activation {dtype}")
    # the entries sorted by expert, and the experts' results gathered back
    H = 24
    x = torch.randn(N, H, generator=g)
    rank, place = (torch.empty(N * top, dtype=torch.int32, device=DEV) for _ in range(2))
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    xs = torch.full((N * top, H), float("nan"), device=DEV)
    k.expert_sort(pick, E, dev(x), rank, counts, place, xs)
    flat = pick.cpu().long().flatten()
    assert counts.cpu().tolist() == torch.bincount(flat, minlength=E).tolist()
    order = torch.argsort(flat, stable=True)
    assert torch.equal(place.cpu().long()[order], torch.arange(N * top))
    assert torch.equal(xs.cpu(), x[order // top])
    ys = torch.randn(N * top, H, generator=g)
    sh = torch.randn(N, H, generator=g) if shared else None
    start = torch.randn(N, H, generator=g)
    for accumulate in (False, True):
        out = dev(start)
        k.expert_combine(dev(ys), place, pw, None if sh is None else dev(sh), dense[:, E:E + 1] if shared else None, out, accumulate)
        wantc = (pw.cpu().double()[:, :, None] * ys.double()[place.cpu().long()].view(N, top, H)).sum(1)
        if shared:
            wantc = wantc + want[:, E:E + 1] * sh.double()
        close(out, wantc + (start.double() if accumulate else 0), 1e-5, "combine")


# ------------------------------------------------------------------------------------------ attention
def _attention_case(dtype, T, H, G, dk, dv, chunk, rot, page_size, loud=None, seed=0, scale=0.4):
    """q, k, v projections of T tokens through prepare + attention, whole and token by token, against the plain
    mixer without its projections."""
    g = torch.Generator().manual_seed(seed)
    proj = torch.randn(T, H * dk + G * (dk + dv) + 3, generator=g, dtype=F64)
    wq, wk = 1 + 0.3 * torch.randn(dk, generator=g, dtype=F64), 1 + 0.3 * torch.randn(dk, generator=g, dtype=F64)
    eps = 1e-5
    if loud is not None:                          # one key that a query far away must find (or must not)
        qi, kj = loud
        proj[kj, H * dk:H * dk + G * dk] *= 3.0
        proj[qi, :H * dk] = proj[kj, H * dk:H * dk + dk].repeat(H) * 3.0
    q = proj[:, :H * dk].view(T, H, dk)
    kk = proj[:, H * dk:H * dk + G * dk].view(T, G, dk)
    v = proj[:, H * dk + G * dk:H * dk + G * (dk + dv)].view(T, G, dv)
    rnd = P.round_to(dtype) if dtype != torch.float32 else P.same
    qn = rnd(P.rotate(P.rms_unit(q, eps) * wq, torch.arange(T), rot))
    kn = rnd(P.rotate(P.rms_unit(kk, eps) * wk, torch.arange(T), rot))
    ok = P.visible(T, {"size": chunk} if chunk else None)
    want = torch.cat([torch.softmax(((qn[:, a] @ kn[:, a // (H // G)].T) * scale).masked_fill(~ok, float("-inf")), -1)
                      @ rnd(v[:, a // (H // G)]) for a in range(H)], -1)
    return proj, wq, wk, eps, scale, want


def _run_attention(k, dtype, proj, wq, wk, eps, scale, T, H, G, dk, dv, chunk, rot, page_size, cuts, prefill):
    from mivi_v4_b200.parts.position import Rope, YarnRope
    n_pages = -(-T // page_size)
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(3))[:n_pages].tolist()     # pages in no order
    pool = torch.zeros(n_pages + 3, G * page_size * (dk + dv), dtype=dtype, device=DEV) if dk != dv else \
        torch.zeros(n_pages + 3, 2, G, page_size, dk, dtype=dtype, device=DEV)
    table = i32([perm + [0] * 2])
    inv, amp, dims = None, 1.0, 0
    if rot:
        sc, dims = rot.get("scaling"), rot["dims"]
        part = YarnRope(dims, rot["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else Rope(dims, rot["base"], "half_split")
        inv, amp = part.rotary(DEV)[0], part.amplitude()
    pd = dev(proj)
    outs, at = [], 0
    for n in cuts:
        rows = slice(at, at + n)
        pos, seq_of = i32(list(range(at, at + n))), i32([0] * n)
        q = torch.empty(n, H * dk, dtype=dtype, device=DEV)
        k.qkv_prepare_wide(pd[rows], dev(wq), dev(wk), eps, dims, inv, pos, seq_of, table, pool, page_size, q, H, G, dk, dv,
                           per_head=True, amplitude=amp)
        o = torch.full((n, H * dv), float("nan"), dtype=dtype, device=DEV)
        if prefill and n > 1:
            k.attention_sink_prefill(q, pool, page_size, table, i32([0, n]), i32([at]), o, 1, H, G, dk, dv, scale, chunk=chunk)
        else:
            k.attention_sink(q, pool, page_size, table, pos, seq_of, o, H, G, dk, dv, scale, chunk=chunk)
        outs.append(o)
        at += n
    return torch.cat(outs)


YARN = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 32.0, "slow": 1.0}}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,chunk,rot,page", [(6, 2, 16, 8, 10, YARN, 8), (2, 2, 24, 24, 70, {"dims": 24, "base": 1e4}, 16),
                                                      (1, 1, 20, 20, 0, None, 8), (4, 1, 32, 64, 64, YARN, 64), (3, 1, 12, 40, 33, None, 16)])
def test_attention_per_head_norm_stretched_rotation_chunked_mask(dtype, H, G, dk, dv, chunk, rot, page):
    k = K()
    T = 150
    proj, wq, wk, eps, scale, want = _attention_case(dtype, T, H, G, dk, dv, chunk, rot, page, seed=dk)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for cuts in ([T], [1] * T, [100] + [1] * 50, [7] * 21 + [3]):
        got = _run_attention(k, dtype, proj, wq, wk, eps, scale, T, H, G, dk, dv, chunk, rot, page, cuts, prefill=False)
        close(got, want, tol, f"single-token kernel, cuts {cuts[:3]}")
    if dtype == torch.bfloat16 and k.attention_sink_prefill_supported(dtype, dk, dv):
        for cuts in ([T], [64, 86], [100] + [1] * 50, [7] * 21 + [3], [63, 65, 22]):
            got = _run_attention(k, dtype, proj, wq, wk, eps, scale, T, H, G, dk, dv, chunk, rot, page, cuts, prefill=True)
            close(got, want, tol, f"long-step kernel, cuts {cuts[:3]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("prefill", [False, True])
def test_a_loud_key_just_inside_and_just_outside_a_chunk(dtype, prefill):
    """Query 139 of chunk [100, 150) and a key made to stand out: at 100 (the chunk's first: seen), at 99 (the
    last of the chunk before: not seen), at 0 (far away, unseen); with chunks of 200 the far key at 0 is seen."""
    k = K()
    if prefill and dtype != torch.bfloat16:
        pytest.skip("the long-step kernel is bfloat16")
    H, G, dk, dv, T = 2, 1, 16, 16, 140
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for chunk, key, seen in ((50, 100, True), (50, 99, False), (50, 0, False), (200, 0, True), (70, 70, True), (70, 69, False)):
        proj, wq, wk, eps, scale, want = _attention_case(dtype, T, H, G, dk, dv, chunk, None, 16, loud=(139, key), seed=key, scale=1.5)
        for cuts in ([T], [120] + [1] * 20):
            got = _run_attention(k, dtype, proj, wq, wk, eps, scale, T, H, G, dk, dv, chunk, None, 16, cuts, prefill)
            close(got, want, tol, f"chunk {chunk} loud key {key}")
        # the loud key decides the row where it is seen: the test would notice a mask that is one off
        v_key = proj[key, H * dk + G * dk:H * dk + G * dk + dv]
        near = (want[139, :dv] - v_key).abs().max() < 0.05 * v_key.abs().max()
        assert bool(near) == seen, (chunk, key)


# ------------------------------------------------------------------------------------------ norms, embedding, cap
def test_gate_before_the_grouped_norm_and_the_post_norm_sum():
    k = K()
    g = torch.Generator().manual_seed(2)
    N, C = 7, 48
    y, z, w = torch.randn(N, C, generator=g, dtype=F64), torch.randn(N, C + 4, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    for parts in (1, 3, 4):
        want = P.rms_unit((y * P.silu(z[:, 2:2 + C])).view(N, parts, C // parts), 1e-5).reshape(N, C) * w
        out = torch.empty(N, C, device=DEV)
        k.gated_rmsnorm(dev(y), dev(z)[:, 2:2 + C], dev(w), C // parts, 1e-5, k.GATE_SILU_FIRST, out)
        close(out, want, 1e-5, f"{parts} parts")
    y2, resid = torch.randn(N, C, generator=g, dtype=F64), torch.randn(N, C, generator=g, dtype=F64)
    for second in (None, y2):
        r = dev(resid)
        rounded = torch.empty(N, C, dtype=torch.bfloat16, device=DEV)
        k.rmsnorm_add_sum(dev(y), dev(w), 1e-5, r, s1=0.7, y2=None if second is None else dev(second), s2=1.3, rounded=rounded)
        total = 0.7 * y + (1.3 * second if second is not None else 0)
        close(r, resid + P.rms_norm(total, w, 1e-5), 1e-5, "post-norm sum")
        assert torch.equal(rounded, r.to(torch.bfloat16))


def test_scaled_embedding_with_positions_and_capped_logits():
    k = K()
    g = torch.Generator().manual_seed(3)
    table, pos = torch.randn(11, 24, generator=g), torch.randn(9, 24, generator=g)
    toks, places = [3, 10, 0, 3], [0, 8, 2, 1]
    for dtype in (torch.float32, torch.bfloat16):
        t, p = table.to(dtype), pos.to(dtype)
        out = torch.empty(4, 24, device=DEV)
        rounded = torch.empty(4, 24, dtype=torch.bfloat16, device=DEV)
        k.embed_scaled_pos(t.to(DEV), i32(toks), 5.0, p.to(DEV), i32(places), out, rounded)
        close(out, t.double()[toks] * 5.0 + p.double()[places], 1e-6, "embedding")
        assert torch.equal(rounded, out.to(torch.bfloat16))
    x = torch.tensor([[-100.0, -1.0, 0.0, 0.5, 40.0]])
    got = k.softcap_(x.to(DEV), 30.0)
    close(got, 30.0 * torch.tanh(x.double() / 30.0), 1e-6, "cap")


# ------------------------------------------------------------------------------------------ recurrence in chunks
def _workspace():
    from mivi_v4_b200.engine.step import Workspace
    return Workspace(DEV)


@pytest.mark.parametrize("H,G,N,Pd", [(4, 2, 24, 16), (1, 1, 8, 3), (3, 3, 72, 20), (2, 1, 136, 33), (8, 1, 128, 64)])
def test_chunked_scan_as_a_state_space_layer(H, G, N, Pd):
    """Chunks full, one token short and one over; a decay that underflows within a chunk; steps that continue a
    state; several sequences of unequal lengths in one step."""
    k = K()
    ws = _workspace()
    g = torch.Generator().manual_seed(H * 7 + N)
    for T, cuts in ((31, [31]), (32, [32]), (33, [33]), (97, [97]), (97, [40, 57]), (97, [16, 17, 64]), (80, [3, 77])):
        x = torch.randn(T, H, Pd, generator=g, dtype=F64)
        B, C = torch.randn(T, G, N, generator=g, dtype=F64), torch.randn(T, G, N, generator=g, dtype=F64)
        dt = torch.rand(T, H, generator=g, dtype=F64) * 2 + 0.01
        A, D = -torch.rand(H, generator=g, dtype=F64) * 2 - 0.01, torch.randn(H, generator=g, dtype=F64)
        A[0] = -40.0                                     # e^(-40 dt): gone within a few tokens, e^(-1000) over a chunk
        want = torch.cat([P.state_space_scan(x[:, a], B[:, a // (H // G)], C[:, a // (H // G)], dt[:, a], A[a], D[a]) for a in range(H)], -1)
        wide = dev(torch.cat([x.reshape(T, -1), B.reshape(T, -1), C.reshape(T, -1)], -1))
        inner, gn = H * Pd, G * N
        log_a, b = dev(A[None, :] * dt), dev(dt)
        state = torch.zeros(2, H, Pd, N, device=DEV)
        outs, at = [], 0
        for n in cuts:
            rows = slice(at, at + n)
            out = torch.full((n, inner), float("nan"), device=DEV)
            k.scalar_scan(wide[rows, inner + gn:], wide[rows, inner:inner + gn], wide[rows, :inner], log_a[rows], b[rows],
                          state, i32([1]), i32([0, n]), out, 1, H, N, Pd, heads_per_group=H // G, skip=dev(D), max_len=n, ws=ws)
            outs.append(out)
            at += n
        close(torch.cat(outs), want, 3e-5, f"T {T} cuts {cuts}")
        # the state the chunks leave is the state the token-by-token kernel leaves
        ref = torch.zeros(2, H, Pd, N, device=DEV)
        k.scalar_scan(wide[:, inner + gn:], wide[:, inner:inner + gn], wide[:, :inner], log_a, b, ref, i32([1]), i32([0, T]),
                      torch.empty(T, inner, device=DEV), 1, H, N, Pd, heads_per_group=H // G, skip=dev(D))
        close(state, ref.double().cpu(), 3e-5, "state")


def test_chunked_scan_of_unequal_sequences_and_a_matrix_memory():
    k = K()
    ws = _workspace()
    H, dk, dv, cap = 3, 40, 24, 9.0
    g = torch.Generator().manual_seed(9)
    lens = [70, 1, 33, 16]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q, kk = torch.randn(T, H, dk, generator=g, dtype=F64), torch.randn(T, H, dk, generator=g, dtype=F64)
    v = torch.randn(T, H, dv, generator=g, dtype=F64)
    zi, zf = 4 * torch.randn(T, H, generator=g, dtype=F64), 4 * torch.randn(T, H, generator=g, dtype=F64) + 2
    zero = torch.zeros(H, dtype=F64)
    i_log = cap * torch.tanh(zi / cap)
    f_log = P.log_sigmoid(cap * torch.tanh(zf / cap))
    want = torch.cat([torch.cat([P.matrix_memory_scan(q[a:b, h] * dk ** -0.5, kk[a:b, h], v[a:b, h], i_log[a:b, h], f_log[a:b, h])
                                 for h in range(H)], -1) for a, b in zip(cu[:-1], cu[1:])])
    memory, maxima = torch.zeros(5, H, dv + 1, dk, device=DEV), torch.zeros(5, H, device=DEV)
    slots, cud = i32([4, 0, 2, 1]), i32(cu)
    log_a, b, m = (torch.empty(T, H, device=DEV) for _ in range(3))
    k.memory_gates(dev(zi), dev(zf), dev(zero), dev(zero), cap, maxima, slots, cud, log_a, b, m, len(lens), H)
    out = torch.full((T, H * dv), float("nan"), device=DEV)
    k.scalar_scan(dev(q.reshape(T, -1)), dev(kk.reshape(T, -1)), dev(v.reshape(T, -1)), log_a, b, memory, slots, cud, out,
                  len(lens), H, dk, dv, m_tok=m, q_scale=dk ** -0.5, max_len=max(lens), ws=ws)
    # the division by |n . q| amplifies float32 rounding where n . q nearly cancels, and the chunks sum in another order
    close(out, want, 3e-4, "matrix memory in chunks")
    assert memory[3].abs().max() == 0


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_one_token_a_sequence_convolution_and_step_size_in_one_kernel(taps):
    k = K()
    C, H, T, B = 21, 3, 9, 3
    g = torch.Generator().manual_seed(taps + 40)
    u = torch.randn(B, T, 2 + C + H, generator=g, dtype=F64)                 # [.. | channels | step sizes] a token
    w, bias = torch.randn(C, taps, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    dt_bias, a_log = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    want = torch.stack([P.silu(P.causal_taps(u[b, :, 2:2 + C], w, bias)) for b in range(B)])
    state = torch.zeros(4, max(taps - 1, 0), C, device=DEV)
    slots = i32([2, 0, 3])
    for t in range(T):
        rows = dev(u[:, t])
        out = torch.full((B, C), float("nan"), device=DEV)
        log_a, b = torch.empty(B, H, device=DEV), torch.empty(B, H, device=DEV)
        k.ssm_decode_prepare(rows[:, 2:2 + C], dev(w), dev(bias), state, slots, out, rows[:, 2 + C:], dev(dt_bias), dev(a_log), log_a, b)
        close(out, want[:, t], 1e-5, f"taps {taps} token {t}")
        dt = P.softplus(u[:, t, 2 + C:] + dt_bias)
        close(b, dt, 1e-6, "dt")
        close(log_a, -torch.exp(a_log) * dt, 1e-6, "log a")
    if taps > 1:
        assert state[1].abs().max() == 0
        close(state[0], u[1, T - (taps - 1):, 2:2 + C], 1e-6, "kept inputs")


@pytest.mark.parametrize("E,top,ff,H,N", [(4, 2, 32, 64, 300), (16, 4, 64, 128, 700), (6, 1, 16, 40, 130), (3, 2, 48, 72, 5)])
def test_grouped_products_over_rows_sorted_by_expert(E, top, ff, H, N):
    """Every expert's run of rows starts on a tile; one product takes each tile's rows through ITS expert's gate and
    up rows (with the activation), one through its down columns; experts that nobody chose, and runs of one row."""
    k = K()
    g = torch.Generator().manual_seed(E * 10 + top)
    x = torch.randn(N, H, generator=g).bfloat16()
    choice = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(N)]).int()     # the last expert: never
    if N > 100:
        choice[7, 0] = E - 1                                                                      # but once
        choice[7, 1:] = torch.arange(top - 1)
    w_gate, w_up = (torch.randn(E, ff, H, generator=g) / H ** 0.5).bfloat16(), (torch.randn(E, ff, H, generator=g) / H ** 0.5).bfloat16()
    w_down = (torch.randn(E, H, ff, generator=g) / ff ** 0.5).bfloat16()
    w_gu = torch.stack([w_gate.view(E, ff // 16, 16, H), w_up.view(E, ff // 16, 16, H)], dim=2).reshape(E * 2 * ff, H).contiguous()
    w_dn = torch.cat(list(w_down), dim=1).contiguous()                                            # [H, E * ff]
    tiles = k.grouped_tiles(N * top, E)
    rows = tiles * k.GROUPED_TILE_ROWS
    pick = choice.to(DEV)
    rank, place = (torch.empty(N * top, dtype=torch.int32, device=DEV) for _ in range(2))
    counts, offsets = (torch.empty(E, dtype=torch.int32, device=DEV) for _ in range(2))
    tile_group = torch.empty(tiles, dtype=torch.int32, device=DEV)
    xs = torch.full((rows, H), float("nan"), dtype=torch.bfloat16, device=DEV)                   # the padding stays as it is
    k.expert_sort(pick, E, x.to(DEV), rank, counts, place, xs, offsets, tile_group)
    cnt = torch.bincount(choice.flatten().long(), minlength=E)
    assert counts.cpu().tolist() == cnt.tolist()
    tiles_of = (cnt + 127) // 128
    want_off = torch.cat([torch.zeros(1, dtype=torch.long), tiles_of.cumsum(0)[:-1]]) * 128
    assert offsets.cpu().tolist() == want_off.tolist()
    want_groups = sum(([e] * int(t) for e, t in enumerate(tiles_of)), [])
    assert tile_group.cpu().tolist() == want_groups + [-1] * (tiles - len(want_groups))
    pl = place.cpu().long()
    assert torch.equal(xs.cpu()[pl].float(), x[torch.arange(N * top) // top].float())
    hs = torch.full((rows, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    k.gemm_tc_grouped(xs, w_gu.to(DEV), hs, tile_group, 2 * ff, H, row_step=2 * ff, swiglu=True)
    ys = torch.full((rows, H), float("nan"), device=DEV)
    k.gemm_tc_grouped(hs, w_dn.to(DEV), ys, tile_group, H, ff, k_step=ff)
    e_of = choice.flatten().long()
    xe = x[torch.arange(N * top) // top].double()
    gate = torch.einsum("nh,nfh->nf", xe, w_gate.double()[e_of])
    up = torch.einsum("nh,nfh->nf", xe, w_up.double()[e_of])
    hid = (P.silu(gate) * up).bfloat16().double()
    close(hs.cpu()[pl], hid, 1e-2, "gated activations")
    close(ys.cpu()[pl], torch.einsum("nf,nhf->nh", hid, w_down.double()[e_of]), 1e-2, "down")


@pytest.mark.parametrize("taps", [1, 3, 4])
def test_causal_convolution_of_long_steps_four_channels_a_thread(taps):
    k = K()
    C = 40
    g = torch.Generator().manual_seed(taps + 70)
    lens = [130, 1, 67]
    us = [torch.randn(n, 4 + C, generator=g, dtype=F64) for n in lens]
    w, bias = torch.randn(C, taps, generator=g, dtype=F64), torch.randn(C, generator=g, dtype=F64)
    want = torch.cat([P.silu(P.causal_taps(u[:, 4:], w, bias)) for u in us])
    for cuts in ([1.0], [0.5, 0.5]):                      # whole, and each sequence in two steps of about half
        state = torch.zeros(3, max(taps - 1, 0), C, device=DEV)
        done = [0] * len(lens)
        outs = [[] for _ in lens]
        for frac in cuts:
            part = [(d, n if frac == 1.0 or d else max(1, n // 2)) for d, n in zip(done, lens)]
            part = [(d, (n - d) if d else m) for (d, m), n in zip(part, lens)]
            rows = torch.cat([u[d:d + m] for u, (d, m) in zip(us, part)])
            cu, seq_of = [0], []
            for i, (_, m) in enumerate(part):
                cu.append(cu[-1] + m)
                seq_of += [i] * m
            out = torch.full((rows.shape[0], C), float("nan"), device=DEV)
            k.causal_conv_silu(dev(rows)[:, 4:], dev(w), dev(bias), state, i32(seq_of), i32(cu), i32([2, 0, 1]), out, len(lens))
            for i, (d, m) in enumerate(part):
                outs[i].append(out[cu[i]:cu[i + 1]])
                done[i] = d + m
            if all(d == n for d, n in zip(done, lens)):
                break
        close(torch.cat([torch.cat(o) for o in outs]), want, 1e-5, f"taps {taps} cuts {cuts}")
