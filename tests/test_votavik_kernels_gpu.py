"""Each kernel of the Votavik mechanisms alone against a plain float64 expression, at sizes of the tests'
own, in float32 and bfloat16 where the kernel has both."""
import math

import pytest
import torch

import plain_votavik as P
from mivi_v4_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    err = (got - want).abs().max().item()
    assert torch.isfinite(got).all() and err <= tol * max(1.0, want.abs().max().item()), (what, err)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 200, 1030])
def test_layernorm(H, out_dtype):
    torch.manual_seed(H)
    x = (torch.randn(9, H) * 3 + 5).to(DEV)                 # a mean far from zero: a one-pass variance would lose digits
    w = torch.randn(H).to(DEV)
    out = torch.full((9, H), float("nan"), dtype=out_dtype, device=DEV)
    K.layernorm(x, w, 1e-5, out)
    close(out, P.layer_norm(x.double().cpu(), w.double().cpu(), 1e-5), out_dtype)
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    out = torch.empty((3, H), dtype=out_dtype, device=DEV)
    K.layernorm(x, w, 1e-5, out, rows)
    close(out, P.layer_norm(x.double().cpu()[[7, 0, 7]], w.double().cpu(), 1e-5), out_dtype)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gated_rmsnorm_per_head_and_over_all_heads(out_dtype):
    torch.manual_seed(3)
    N, heads, dv = 5, 3, 20
    wide = torch.randn(N, 2 * heads * dv + 7).to(DEV)        # the gate is a column slice of a wider matrix
    x = torch.randn(N, heads * dv).to(DEV)
    gate = wide[:, heads * dv + 3: 2 * heads * dv + 3]
    xd, gd = x.double().cpu(), gate.double().cpu()
    w = torch.randn(dv).to(DEV)
    out = torch.empty((N, heads * dv), dtype=out_dtype, device=DEV)
    K.gated_rmsnorm(x, gate, w, dv, 1e-4, K.GATE_SILU, out)
    want = (P.rms_unit(xd.view(N, heads, dv), 1e-4) * w.double().cpu()).reshape(N, -1) * P.silu(gd)
    close(out, want, out_dtype, "per head")
    w2 = torch.randn(heads * dv).to(DEV)
    K.gated_rmsnorm(x, gate, w2, heads * dv, 1e-4, K.GATE_SIGMOID, out)
    close(out, P.rms_unit(xd, 1e-4) * w2.double().cpu() * torch.sigmoid(gd), out_dtype, "all heads")


def test_rmsnorm_add_glu_table_gate_round():
    torch.manual_seed(4)
    N, H, D, V = 6, 72, 5, 31
    y, w, resid = torch.randn(N, H).to(DEV), torch.randn(H).to(DEV), torch.randn(N, H).to(DEV)
    want = resid.double().cpu() + P.rms_unit(y.double().cpu(), 1e-5) * w.double().cpu()
    K.rmsnorm_add(y, w, 1e-5, resid)
    close(resid, want, torch.float32)
    for dt in (torch.float32, torch.bfloat16):                # the same with the next layer norm in the same kernel
        resid2 = torch.randn(N, H).to(DEV) * 2 + 3
        ln_w = torch.randn(H).to(DEV)
        new = resid2.double().cpu() + P.rms_unit(y.double().cpu(), 1e-5) * w.double().cpu()
        out = torch.full((N, H), float("nan"), dtype=dt, device=DEV)
        K.rmsnorm_add_layernorm(y, w, 1e-5, resid2, ln_w, 1e-4, out)
        close(resid2, new, torch.float32)
        close(out, P.layer_norm(new, ln_w.double().cpu(), 1e-4), dt)
    gu = (torch.randn(N, 2 * 33) * 3).to(DEV)
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty((N, 33), dtype=dt, device=DEV)
        K.glu_clamped(gu, out, 1.25, 1.702)
        g = gu.double().cpu()[:, :33].clamp(max=1.25)
        u = gu.double().cpu()[:, 33:].clamp(-1.25, 1.25)
        close(out, g * torch.sigmoid(1.702 * g) * (u + 1), dt)
        table = torch.randn(V, 4 * D).to(dt).to(DEV)
        p = torch.randn(N, D).to(DEV)
        toks = torch.tensor([0, 30, 5, 5, 17, 1], dtype=torch.int32, device=DEV)
        out = torch.empty((N, D), dtype=dt, device=DEV)
        K.table_gate(p, table, 2 * D, toks, out)
        close(out, P.gelu_tanh(p.double().cpu()) * table.double().cpu()[toks.long().cpu(), 2 * D:3 * D], dt)
    r = torch.empty((N, H), dtype=torch.bfloat16, device=DEV)
    K.round_rows(y, r)
    assert torch.equal(r, y.to(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D", [(72, 5), (256, 64), (1001, 24)])
def test_table_gate_proj_in_one_kernel(H, D, dtype):
    torch.manual_seed(H + D)
    N, V, col0 = 7, 50, 2 * D
    resid = torch.randn(N, H).to(DEV)
    gate = (torch.randn(D, H) / H ** 0.5).to(dtype).to(DEV)
    table = torch.randn(V, 4 * D).to(dtype).to(DEV)
    toks = torch.tensor([0, 49, 7, 7, 13, 1, 30], dtype=torch.int32, device=DEV)
    x = resid.cpu().to(dtype).double()
    want = P.gelu_tanh(x @ gate.double().cpu().T) * table.double().cpu()[toks.long().cpu(), col0:col0 + D]
    out = torch.full((N, D), float("nan"), dtype=dtype, device=DEV)
    assert K.table_gate_proj_ok(N, gate, table, dtype)
    K.table_gate_proj(resid, gate, table, col0, toks, out)
    close(out, want, dtype)


def _scan_case(N, heads, dk, dv, seed):
    torch.manual_seed(seed)
    wide = torch.randn(N, heads * (2 * dk + dv) + 3).to(DEV)
    q, k = wide[:, :heads * dk], wide[:, heads * dk:2 * heads * dk]
    v = wide[:, 2 * heads * dk:2 * heads * dk + heads * dv]
    z = (torch.randn(N, heads * dk) * 2 + 1).to(DEV)
    return q, k, v, z


def _plain_scan(q, k, v, decay, lens, heads, dk, dv, act):
    """Sequences packed one after another; returns o [N, heads * dv] and the last state of each sequence
    [seq][heads, dv, dk] (the kernel's transposed layout)."""
    f = P.silu if act else (lambda t: t)
    q, k, v = f(q.double().cpu()), f(k.double().cpu()), f(v.double().cpu())
    outs, states, at = [], [], 0
    for n in lens:
        o = torch.zeros(n, heads * dv, dtype=F64)
        st = torch.zeros(heads, dv, dk, dtype=F64)
        for h in range(heads):
            oh, S = P.decayed_outer_scan(q[at:at + n, h * dk:(h + 1) * dk], k[at:at + n, h * dk:(h + 1) * dk],
                                         v[at:at + n, h * dv:(h + 1) * dv], decay[at:at + n, h * dk:(h + 1) * dk])
            o[:, h * dv:(h + 1) * dv] = oh
            st[h] = S.T
        outs.append(o)
        states.append(st)
        at += n
    return torch.cat(outs), states


@pytest.mark.parametrize("heads,dk,dv", [(2, 16, 24), (1, 20, 5), (3, 72, 17), (1, 136, 40), (2, 256, 16)])
def test_decay_scan_with_a_decay_per_channel(heads, dk, dv):
    lens = [13, 1, 30]
    N = sum(lens)
    q, k, v, z = _scan_case(N, heads, dk, dv, dk)
    tau = 3.0
    decay = torch.sigmoid(z.double().cpu()) ** (1.0 / tau)
    want_o, want_s = _plain_scan(q * dk ** -0.5, k, v, decay, lens, heads, dk, dv, act=False)
    state = torch.full((5, heads, dv, dk), float("nan"), device=DEV)
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device=DEV)
    state[slots.long()] = 0
    cu = torch.tensor([0, 13, 14, 44], dtype=torch.int32, device=DEV)
    out = torch.full((N, heads * dv), float("nan"), device=DEV)
    K.decay_scan(q, k, v, state, slots, cu, out, 3, heads, dk, dv, decay_logits=z, inv_tau=1 / tau, q_scale=dk ** -0.5)
    close(out, want_o, torch.float32, "outputs")
    for b, s in enumerate([3, 0, 4]):
        close(state[s], want_s[b], torch.float32, f"state of sequence {b}")
    assert torch.isnan(state[1]).all() and torch.isnan(state[2]).all()          # other slots untouched


class _Scratch:
    """What the chunked kernels ask of a workspace."""
    def __init__(self):
        self.bufs = {}

    def get(self, name, shape, dtype):
        self.bufs[name] = torch.full(tuple(shape), float("nan"), dtype=dtype, device=DEV)
        return self.bufs[name]


@pytest.mark.parametrize("heads,dk,dv,per_channel", [(2, 16, 24, True), (1, 20, 5, False), (3, 72, 40, True),
                                                      (1, 136, 33, False), (2, 256, 64, True)])
def test_decay_scan_in_chunks(heads, dk, dv, per_channel):
    """Sequences of 1, 31, 32, 33 and 150 tokens in one step (chunks that are full, one short, one over), on top
    of states that earlier steps left; decays small enough that a product over a chunk underflows."""
    lens = [33, 1, 150, 32, 31]
    N, B = sum(lens), len(lens)
    q, k, v, z = _scan_case(N, heads, dk, dv, dk + 1)
    z = z * 4 - 2                                          # sigmoid(z)^(1/tau) down to 1e-3 a token with tau 1
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    slots = torch.tensor([4, 2, 0, 5, 1], dtype=torch.int32, device=DEV)
    hd = (torch.rand(heads) * 0.5 + 0.5).to(DEV)
    if per_channel:
        decay = torch.sigmoid(z.double().cpu())
        kw = dict(decay_logits=z, inv_tau=1.0, q_scale=0.7)
        qs = q * 0.7
    else:
        decay = hd.double().cpu().repeat_interleave(dk)[None, :].expand(N, -1)
        kw = dict(head_decay=hd, act=K.SCAN_ACT_SILU)
        qs = q
    # the state every sequence starts from: what a first step of 5 tokens left (token by token kernel)
    q0, k0, v0, z0 = _scan_case(5 * B, heads, dk, dv, 99)
    state = torch.zeros((6, heads, dv, dk), device=DEV)
    o0 = torch.empty((5 * B, heads * dv), device=DEV)
    cu0 = torch.arange(0, 5 * B + 1, 5, dtype=torch.int32, device=DEV)
    kw0 = dict(kw, decay_logits=z0) if per_channel else kw
    K.decay_scan(q0, k0, v0, state, slots, cu0, o0, B, heads, dk, dv, **kw0)
    seq = state.clone()
    out_seq = torch.empty((N, heads * dv), device=DEV)
    K.decay_scan(q, k, v, seq, slots, cu, out_seq, B, heads, dk, dv, **kw)                 # token by token
    out = torch.full((N, heads * dv), float("nan"), device=DEV)
    K.decay_scan(q, k, v, state, slots, cu, out, B, heads, dk, dv, max_len=max(lens), ws=_Scratch(), **kw)
    scale = out_seq.abs().max().item()
    assert torch.isfinite(out).all()
    assert (out - out_seq).abs().max().item() <= 2e-5 * scale
    assert (state - seq).abs().max().item() <= 2e-5 * seq.abs().max().item()
    assert torch.equal(state[3], torch.zeros_like(state[3]))                               # a slot of no sequence
    # and against the plain scan from a zero state (the first sequence's first step left out: fresh slots)
    fresh = torch.zeros((6, heads, dv, dk), device=DEV)
    K.decay_scan(q, k, v, fresh, slots, cu, out, B, heads, dk, dv, max_len=max(lens), ws=_Scratch(), **kw)
    want_o, want_s = _plain_scan(qs, k, v, decay, lens, heads, dk, dv, act=not per_channel)
    close(out, want_o, torch.float32, "outputs")
    for b, s in enumerate(slots.tolist()):
        close(fresh[s], want_s[b], torch.float32, f"state of sequence {b}")


def test_decay_scan_any_cut_gives_the_same_numbers_and_slots_are_reused():
    heads, dk, dv = 2, 24, 20
    lens = [37]
    q, k, v, _ = _scan_case(37, heads, dk, dv, 5)
    hd = torch.tensor([0.5, 0.999], device=DEV)
    decay = hd.double().cpu().repeat_interleave(dk)[None, :].expand(37, -1)
    want_o, want_s = _plain_scan(q, k, v, decay, lens, heads, dk, dv, act=True)
    whole = torch.empty((37, heads * dv), device=DEV)
    state = torch.zeros((2, heads, dv, dk), device=DEV)
    one = torch.tensor([1], dtype=torch.int32, device=DEV)
    K.decay_scan(q, k, v, state, one, torch.tensor([0, 37], dtype=torch.int32, device=DEV), whole, 1, heads, dk, dv,
                 head_decay=hd, act=K.SCAN_ACT_SILU)
    close(whole, want_o, torch.float32)
    close(state[1], want_s[0], torch.float32)
    for cuts in ([1] * 37, [2] * 18 + [1], [8, 9, 7, 13], [36, 1]):
        state[1] = 0                                   # the slot is used again by a new sequence
        got, at = [], 0
        for n in cuts:
            o = torch.empty((n, heads * dv), device=DEV)
            K.decay_scan(q[at:at + n], k[at:at + n], v[at:at + n], state, one,
                         torch.tensor([0, n], dtype=torch.int32, device=DEV), o, 1, heads, dk, dv, head_decay=hd,
                         act=K.SCAN_ACT_SILU)
            got.append(o)
            at += n
        assert torch.equal(torch.cat(got), whole), cuts       # bit for bit: the order of the sums does not depend on the cut
        close(state[1], want_s[0], torch.float32)


def _fill_cache(k, v, page_size, nkv, dk, dv, dtype, pages_order):
    """Keys [T, nkv, dk] and values [T, nkv, dv] of one sequence into a flat pool, its pages in the given order."""
    T = k.shape[0]
    n_blocks = -(-T // page_size)
    pool = torch.full((max(pages_order) + 1, nkv * page_size * (dk + dv)), float("nan"), dtype=dtype, device=DEV)
    for blk in range(n_blocks):
        page = pages_order[blk]
        lo, hi = blk * page_size, min(T, (blk + 1) * page_size)
        kp = torch.zeros(nkv, page_size, dk, dtype=dtype, device=DEV)
        vp = torch.zeros(nkv, page_size, dv, dtype=dtype, device=DEV)
        kp[:, :hi - lo] = k[lo:hi].permute(1, 0, 2).to(dtype)
        vp[:, :hi - lo] = v[lo:hi].permute(1, 0, 2).to(dtype)
        pool[page] = torch.cat([kp.reshape(-1), vp.reshape(-1)])
    table = torch.tensor([pages_order[:n_blocks]], dtype=torch.int32, device=DEV)
    return pool, table


def _plain_attention(q, k, v, nh, nkv, scale, cap, window, keep, sinks, gate, positions):
    """q [N, nh, dk] of the query positions over all keys k [T, nkv, dk], v [T, nkv, dv]."""
    out = []
    for n, pos in enumerate(positions):
        row = []
        for h in range(nh):
            g = h // (nh // nkv)
            js = [j for j in range(k.shape[0]) if P.visible(pos, j, window if window else 10 ** 9, keep)]
            s = (k[js, g] @ q[n, h]) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            top = s.max() if sinks is None else torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(sinks[h] - top) if sinks is not None else 0.0)
            o = (e[:, None] * v[js, g]).sum(0) / den
            row.append(o * (torch.sigmoid(gate[n, h]) if gate is not None else 1.0))
        out.append(torch.cat(row))
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,window,keep,cap", [
    (4, 2, 16, 8, 9, 3, 20.0), (3, 1, 20, 20, 0, 0, 0.0), (2, 2, 40, 72, 64, 64, 5.0), (6, 3, 8, 136, 130, 1, 0.0)])
def test_attention_sink_window_edges_far_keys_and_the_sink(nh, nkv, dk, dv, window, keep, cap, dtype):
    torch.manual_seed(nh * dk)
    T, ps = 300, 64
    k, v = torch.randn(T, nkv, dk), torch.randn(T, nkv, dv)
    positions = [0, 1, keep, keep + 1, window, window + keep, 63, 64, 65, 128, 200, T - 1]
    q = torch.randn(len(positions), nh, dk)
    # one key stands out for each query: the one just inside the window's edge, the one just outside it, the
    # last kept token, the first one not kept, and a key far back; whether it is read decides the result
    targets = [0, 0, max(keep - 1, 0), keep, 1, keep, 0, 64 - window + 1 if window else 3, 65 - window if window else 0,
               128 - window if window else 5, 200 - window + 1 if window else 7, 2]
    for n, (pos, j) in enumerate(zip(positions, targets)):
        j = min(max(j, 0), pos)
        k[j] = k[j] * 0.2 + 3.0 * q[n, 0, :][None, :] / q[n, 0].norm()
    sinks = torch.randn(nh) * 2
    gate = torch.randn(len(positions), nh)
    scale = 1.3 / math.sqrt(dk)
    kq, vq, qq = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
    want = _plain_attention(qq, kq, vq, nh, nkv, scale, cap, window, keep, sinks.double(), gate.double(), positions)
    order = [4, 0, 3, 1, 2]                                   # pages of the sequence in no particular order
    pool, table = _fill_cache(k, v, ps, nkv, dk, dv, dtype, order)
    N = len(positions)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(N, dtype=torch.int32, device=DEV)
    out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
    gate_wide = torch.randn(N, nh + 5).to(DEV)
    gate_wide[:, 2:2 + nh] = gate.to(DEV)
    K.attention_sink(q.reshape(N, -1).to(dtype).to(DEV), pool, ps, table, pos_t, seq_of, out, nh, nkv, dk, dv, scale,
                     softcap=cap, window=window, keep_first=keep, sinks=sinks.to(DEV), gate=gate_wide[:, 2:2 + nh])
    close(out, want, dtype, "with sink and gate")
    for tile in (1, 2, 4):                                    # query heads of a kv head sharing a block's loads
        out.fill_(float("nan"))
        K.attention_sink(q.reshape(N, -1).to(dtype).to(DEV), pool, ps, table, pos_t, seq_of, out, nh, nkv, dk, dv, scale,
                         softcap=cap, window=window, keep_first=keep, sinks=sinks.to(DEV), gate=gate_wide[:, 2:2 + nh],
                         head_tile=tile)
        close(out, want, dtype, f"head tile {tile}")
    # without sink and gate the same keys are read and the weights sum to one
    K.attention_sink(q.reshape(N, -1).to(dtype).to(DEV), pool, ps, table, pos_t, seq_of, out, nh, nkv, dk, dv, scale,
                     softcap=cap, window=window, keep_first=keep)
    close(out, _plain_attention(qq, kq, vq, nh, nkv, scale, cap, window, keep, None, None, positions), dtype, "plain")


@pytest.mark.parametrize("nh,nkv,dk,dv,window,keep,cap", [
    (4, 2, 16, 32, 9, 3, 20.0), (3, 1, 96, 32, 0, 0, 0.0), (2, 2, 48, 80, 64, 64, 5.0), (2, 1, 128, 128, 130, 70, 0.0),
    (2, 1, 64, 112, 70, 129, 30.0)])
def test_attention_sink_prefill_on_tensor_cores(nh, nkv, dk, dv, window, keep, cap):
    """Two sequences in one step, the second one a later portion of its prompt (its first keys already cached);
    every query against the plain expression; keys that stand out just inside and just outside the window of
    some queries and among the kept first tokens."""
    torch.manual_seed(dk + dv)
    dtype, ps = torch.bfloat16, 64
    T1, T2, start2 = 150, 333, 120
    scale = 1.1 / math.sqrt(dk)
    sinks, outs, wants = torch.randn(nh) * 2, [], []
    pools, tables, qs, gates = [], [], [], []
    for T, start in ((T1, 0), (T2, start2)):
        k, v = torch.randn(T, nkv, dk), torch.randn(T, nkv, dv)
        q = torch.randn(T - start, nh, dk)
        for n in range(0, T - start, 7):                   # a loud key at the window's edges and among the kept ones
            pos = start + n
            for j in (pos - window + 1, pos - window, keep - 1, keep):
                if window and 0 <= j <= pos:
                    k[j] = k[j] * 0.3 + 2.0 * q[n, n % nh][None, :] / q[n, n % nh].norm()
        gate = torch.randn(T - start, nh)
        kq, vq, qq = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
        wants.append(_plain_attention(qq, kq, vq, nh, nkv, scale, cap, window, keep, sinks.double(), gate.double(),
                                      list(range(start, T))))
        pools.append((k, v))
        qs.append(q.reshape(T - start, -1))
        gates.append(gate)
    # both sequences in one pool: the first takes pages 7, 1, 4; the second 0, 2, 8, 3, 6, 5
    orders = ([7, 1, 4], [0, 2, 8, 3, 6, 5])
    pool = torch.zeros((9, nkv * ps * (dk + dv)), dtype=dtype, device=DEV)
    for (k, v), order in zip(pools, orders):
        part, _ = _fill_cache(k, v, ps, nkv, dk, dv, dtype, order)
        for p in order:
            pool[p] = part[p]
    table = torch.zeros((2, 6), dtype=torch.int32, device=DEV)
    table[0, :3] = torch.tensor(orders[0], dtype=torch.int32)
    table[1] = torch.tensor(orders[1], dtype=torch.int32)
    N = T1 + T2 - start2
    q_all = torch.cat(qs).to(dtype).to(DEV)
    gate_all = torch.cat(gates).to(DEV)
    cu = torch.tensor([0, T1, N], dtype=torch.int32, device=DEV)
    starts = torch.tensor([0, start2], dtype=torch.int32, device=DEV)
    out = torch.full((N, nh * dv), float("nan"), dtype=dtype, device=DEV)
    K.attention_sink_prefill(q_all, pool, ps, table, cu, starts, out, 2, nh, nkv, dk, dv, scale, softcap=cap, window=window,
                             keep_first=keep, sinks=sinks.to(DEV), gate=gate_all)
    close(out, torch.cat(wants), dtype, "tensor-core prefill")
    # and the kernel of single query tokens gives the same, token by token
    positions = torch.cat([torch.arange(0, T1), torch.arange(start2, T2)]).to(torch.int32).to(DEV)
    seq_of = torch.cat([torch.zeros(T1), torch.ones(T2 - start2)]).to(torch.int32).to(DEV)
    out2 = torch.empty_like(out)
    K.attention_sink(q_all, pool, ps, table, positions, seq_of, out2, nh, nkv, dk, dv, scale, softcap=cap, window=window,
                     keep_first=keep, sinks=sinks.to(DEV), gate=gate_all)
    close(out2, torch.cat(wants), dtype, "token by token")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,dims", [(4, 2, 16, 8, 8), (1, 1, 20, 20, 0), (3, 3, 24, 40, 24)])
def test_qkv_prepare_norms_the_whole_projection_and_turns_a_part(nh, nkv, dk, dv, dims, dtype):
    torch.manual_seed(dims + nh)
    N, ps, eps = 7, 4, 1e-3
    width = nh * dk + nkv * (dk + dv)
    proj = torch.randn(N, width + 6).to(DEV)
    wq, wk = torch.randn(nh * dk).to(DEV), torch.randn(nkv * dk).to(DEV)
    positions = [0, 1, 2, 3, 4, 9, 10]                       # one sequence at 0..4, another at 9..10
    seq = [0, 0, 0, 0, 0, 1, 1]
    table = torch.tensor([[2, 5, 0], [1, 4, 3]], dtype=torch.int32, device=DEV)
    pool = torch.zeros((6, nkv * ps * (dk + dv)), dtype=dtype, device=DEV)
    inv = None
    if dims:
        inv = (1.0 / (torch.tensor(50.0, dtype=F64) ** (2.0 * torch.arange(dims // 2, dtype=F64) / dims))).float().to(DEV)
    q_out = torch.empty((N, nh * dk), dtype=dtype, device=DEV)
    K.qkv_prepare_wide(proj, wq, wk, eps, dims, inv, torch.tensor(positions, dtype=torch.int32, device=DEV),
                       torch.tensor(seq, dtype=torch.int32, device=DEV), table, pool, ps, q_out, nh, nkv, dk, dv)
    pd = proj.double().cpu()
    pos_t = torch.tensor(positions)
    q = P.rotate_partial((P.rms_unit(pd[:, :nh * dk], eps) * wq.double().cpu()).view(N, nh, dk), pos_t, dims, 50.0)
    k = P.rotate_partial((P.rms_unit(pd[:, nh * dk:nh * dk + nkv * dk], eps) * wk.double().cpu()).view(N, nkv, dk), pos_t, dims, 50.0)
    v = pd[:, nh * dk + nkv * dk:width].view(N, nkv, dv)
    close(q_out, q.reshape(N, -1), dtype, "q")
    for n in range(N):
        page = int(table[seq[n], positions[n] // ps])
        row = positions[n] % ps
        kp = pool[page, :nkv * ps * dk].view(nkv, ps, dk)[:, row]
        vp = pool[page, nkv * ps * dk:].view(nkv, ps, dv)[:, row]
        close(kp, k[n], dtype, f"k of token {n}")
        close(vp, v[n], dtype, f"v of token {n}")
