"""Each mechanism of the Boketar parts alone against its plain function (GPU): the kernels are
called as the parts call them, on inputs made so that a fault shows."""
import math

import pytest
import torch

from plain import boketar_plain as P

from poor_mans_mamba_b200.kernels import ops as K

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).float()


def close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    got, want = got.double().cpu(), want.double()
    tol = (f32 if dtype == torch.float32 else bf16) * max(1.0, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= tol, f"{what}: {err:.3e} > {tol:.3e}"


def batch_index(lens, slots):
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    seq_of = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(DEV)
    return cu, seq_of, torch.tensor(slots, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- residual lanes
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,D", [(1, 48), (2, 256), (3, 100), (8, 64), (2, 77), (5, 50)])
def test_lanes_mix_and_norm(dtype, n, D):
    T = 7
    x = rnd(n, T, D, seed=1)
    y = rnd(T, D, seed=2)
    mix, ow, iw, nw = rnd(n, n, seed=3), rnd(n, seed=4), rnd(n, seed=5), rnd(D, seed=6) + 1.0
    new = torch.einsum("st,sij->tij", mix.double(), x.double()) + ow.double().view(n, 1, 1) * y.double()
    want = P.norm_plain(torch.einsum("s,sij->ij", iw.double(), new), nw.double(), 1e-5)
    lanes = x.to(DEV).clone()
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    K.hc_mix_norm(lanes, lanes, y.to(DEV, dtype), mix.reshape(-1).to(DEV), ow.to(DEV), iw.to(DEV), nw.to(DEV), 1e-5, out)
    close(lanes, new, torch.float32, "lanes")
    close(out, want, dtype, "normed")
    # all lanes start from one stream; listed rows only, lanes untouched
    h = rnd(T, D, seed=7).to(DEV)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, D, dtype=dtype, device=DEV)
    K.hc_mix_norm(h.unsqueeze(0).expand(n, T, D), None, y.to(DEV, dtype), mix.reshape(-1).to(DEV), ow.to(DEV),
                  torch.ones(n, device=DEV), nw.to(DEV), 1e-5, out2, rows)
    new2 = mix.double().sum(0).view(n, 1, 1) * h.cpu().double() + ow.double().view(n, 1, 1) * y.double()
    close(out2, P.norm_plain(new2.sum(0), nw.double(), 1e-5)[[5, 0, 5]], dtype, "rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_sum_of_branches(dtype):
    T, D = 5, 72
    a, b, wa, wb = rnd(T, D, seed=1, scale=3.0), rnd(T, D, seed=2, scale=0.1), rnd(D, seed=3), rnd(D, seed=4)
    wide = torch.zeros(T, 2 * D + 8, dtype=dtype, device=DEV)  # branches as column slices
    wide[:, :D], wide[:, D + 8:] = a.to(DEV, dtype), b.to(DEV, dtype)
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    K.normed_sum([(wide[:, :D], wa.to(DEV)), (wide[:, D + 8:], wb.to(DEV))], 1e-6, 0.5, out)
    want = 0.5 * (P.norm_plain(a.double(), wa.double(), 1e-6) + P.norm_plain(b.double(), wb.double(), 1e-6))
    close(out, want, dtype, "normed sum")
    bias = rnd(D, seed=5)  # a branch's bias joins it before its norm
    K.normed_sum([(wide[:, :D], wa.to(DEV)), (wide[:, D + 8:], wb.to(DEV))], 1e-6, 0.5, out, biases=[None, bias.to(DEV)])
    want = 0.5 * (P.norm_plain(a.double(), wa.double(), 1e-6) + P.norm_plain(b.double() + bias.double(), wb.double(), 1e-6))
    close(out, want, dtype, "normed sum with a bias")


# ----------------------------------------------------------------------------- matrix-state recurrences
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 16), (2, 2, 64, 40), (3, 1, 128, 96), (1, 1, 8, 8), (2, 1, 200, 33)])
def test_gated_delta_rule_in_portions(dtype, H, G, d, dv):
    """Three sequences of unequal length, in two steps that cut them at odd places, in slots that
    are not in order; the state of a slot that is used again starts from zero."""
    lens = [37, 1, 22]
    T = sum(lens)
    q, k, v = rnd(T, G * d, seed=1), rnd(T, G * d, seed=2), rnd(T, H * dv, seed=3)
    beta, a = rnd(T, H, seed=4), rnd(T, H * d, seed=5)
    dt_bias, a_log = rnd(H * d, seed=6) - 1.0, rnd(H, seed=7) * 0.5
    g = torch.exp(-torch.exp(a_log.double())[None, :, None] * P.softplus(a.double() + dt_bias.double()).view(T, H, d))
    qd, kd = q.double().view(T, G, d), k.double().view(T, G, d)
    qn = (qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * d ** -0.5).repeat_interleave(H // G, dim=1)
    kn = (kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, dim=1)
    want, t0 = [], 0
    for n in lens:
        s = slice(t0, t0 + n)
        want.append(P.gated_delta_rule(qn[s], kn[s], v.double().view(T, H, dv)[s], torch.sigmoid(beta.double())[s], g[s]))
        t0 += n
    want = torch.cat(want).reshape(T, H * dv)
    state = torch.full((5, H, d, dv), 7.0, device=DEV)  # stale values of earlier owners
    slots = [3, 0, 4]
    for s in slots:
        state[s].zero_()
    out = torch.empty(T, H * dv, device=DEV)
    dev = lambda t: t.to(DEV, dtype)
    first = [20, 1, 2]  # tokens of each sequence in the first step (the second sequence ends there)
    starts = [0, 37, 38]
    for part in (0, 1):
        rows, ls, sl = [], [], []
        for i, n in enumerate(lens):
            lo, hi = (0, first[i]) if part == 0 else (first[i], n)
            if hi > lo:
                rows += list(range(starts[i] + lo, starts[i] + hi))
                ls.append(hi - lo)
                sl.append(slots[i])
        idx = torch.tensor(rows)
        cu, _, sl_t = batch_index(ls, sl)
        o = torch.empty(len(rows), H * dv, device=DEV)
        K.delta_scan(dev(q[idx]), dev(k[idx]), dev(v[idx]), dev(beta[idx]), dev(a[idx]), dt_bias.to(DEV), a_log.to(DEV),
                     state, cu, sl_t, len(ls), o, H, G, d, dv, 1e-6, d ** -0.5)
        out[idx.to(DEV)] = o
    close(out, want, torch.float32, "delta rule", f32=1e-4)  # inputs are exact in both types; the state is float
    assert float(state[1].min()) == 7.0 and float(state[2].max()) == 7.0  # other slots untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv", [(2, 16, 24), (4, 32, 32), (1, 100, 7), (3, 4, 130)])
def test_decayed_linear_attention_far_back(dtype, H, d, dv):
    """600 tokens in portions of changing size with a decay of one on the first head: the first
    token weighs as much as the last."""
    T = 600
    q, k, v = rnd(T, H * d, seed=1), rnd(T, H * d, seed=2), rnd(T, H * dv, seed=3)
    decay = [1.0] + [0.97] * (H - 1)
    want = P.decayed_linear_attention(P.silu(q.double()).view(T, H, d), P.silu(k.double()).view(T, H, d),
                                      P.silu(v.double()).view(T, H, dv), decay).reshape(T, H * dv)
    state = torch.zeros(2, H, d, dv, device=DEV)
    out = torch.empty(T, H * dv, device=DEV)
    t0 = 0
    for n in [1, 2, 16, 17, 64, 100, 1, 1, 398]:
        cu, _, sl = batch_index([n], [1])
        K.decay_scan(q[t0:t0 + n].to(DEV, dtype), k[t0:t0 + n].to(DEV, dtype), v[t0:t0 + n].to(DEV, dtype),
                     torch.tensor(decay, device=DEV), state, cu, sl, 1, out[t0:t0 + n], H, d, dv)
        t0 += n
    close(out, want, torch.float32, "decayed linear attention", f32=1e-4)
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 24, 16), (2, 2, 64, 40), (3, 1, 128, 96), (1, 1, 8, 8), (2, 1, 192, 33)])
def test_gated_delta_rule_in_chunks(dtype, H, G, d, dv):
    """Sequences of 1, 63, 64, 65 and 200 tokens (chunk edges), the longest cut into two steps at an odd
    place, strong and weak decays side by side: the chunked kernels against the plain recurrence and
    against the token-serial kernel, state included."""
    lens = [200, 1, 63, 64, 65]
    T = sum(lens)
    q, k, v = rnd(T, G * d, seed=1), rnd(T, G * d, seed=2), rnd(T, H * dv, seed=3)
    beta, a = rnd(T, H, seed=4), rnd(T, H * d, seed=5, scale=3.0)
    dt_bias, a_log = rnd(H * d, seed=6) - 1.0, rnd(H, seed=7) * 0.5 + 1.0   # decays from 1 down to e^-12 a token
    g = torch.exp(-torch.exp(a_log.double())[None, :, None] * P.softplus(a.double() + dt_bias.double()).view(T, H, d))
    assert float(g.min()) < 1e-3 and float(g.max()) > 0.99
    qd, kd = q.double().view(T, G, d), k.double().view(T, G, d)
    qn = (qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * d ** -0.5).repeat_interleave(H // G, dim=1)
    kn = (kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, dim=1)
    want, t0 = [], 0
    for n in lens:
        sl = slice(t0, t0 + n)
        want.append(P.gated_delta_rule(qn[sl], kn[sl], v.double().view(T, H, dv)[sl], torch.sigmoid(beta.double())[sl], g[sl]))
        t0 += n
    want = torch.cat(want).reshape(T, H * dv)
    dev = lambda t: t.to(DEV, dtype)
    slots = [4, 0, 2, 1, 3]
    results = {}
    for kind in ("chunked", "serial"):
        state = torch.zeros(6, H, d, dv, device=DEV)
        out = torch.empty(T, H * dv, device=DEV)
        first = [77, 1, 63, 64, 65]
        starts = [0, 200, 201, 264, 328]
        for part in (0, 1):
            rows, ls, sl = [], [], []
            for i, n in enumerate(lens):
                lo, hi = (0, first[i]) if part == 0 else (first[i], n)
                if hi > lo:
                    rows += list(range(starts[i] + lo, starts[i] + hi))
                    ls.append(hi - lo)
                    sl.append(slots[i])
            idx = torch.tensor(rows)
            cu, _, sl_t = batch_index(ls, sl)
            o = torch.empty(len(rows), H * dv, device=DEV)
            if kind == "chunked":
                scratch = torch.empty(K.recurrent_chunked_scratch_floats(ls, H, d, dv, True), device=DEV)
                K.recurrent_chunked(dev(q[idx]), dev(k[idx]), dev(v[idx]), state, cu, sl_t, ls, o, scratch, H, G, d, dv,
                                    beta=dev(beta[idx]), a=dev(a[idx]), dt_bias=dt_bias.to(DEV), a_log=a_log.to(DEV),
                                    unit_eps=1e-6, q_scale=d ** -0.5)
            else:
                K.delta_scan(dev(q[idx]), dev(k[idx]), dev(v[idx]), dev(beta[idx]), dev(a[idx]), dt_bias.to(DEV),
                             a_log.to(DEV), state, cu, sl_t, len(ls), o, H, G, d, dv, 1e-6, d ** -0.5)
            out[idx.to(DEV)] = o
        close(out, want, torch.float32, f"delta rule, {kind}", f32=1e-4)
        results[kind] = state
    close(results["chunked"], results["serial"].cpu(), torch.float32, "states", f32=1e-4)
    assert float(results["chunked"][5].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv", [(2, 16, 24), (4, 32, 32), (1, 100, 7), (3, 4, 130)])
def test_decayed_linear_attention_in_chunks(dtype, H, d, dv):
    T = 600
    q, k, v = rnd(T, H * d, seed=1), rnd(T, H * d, seed=2), rnd(T, H * dv, seed=3)
    decay = [1.0] + [0.97, 0.5, 0.0][:H - 1]
    want = P.decayed_linear_attention(P.silu(q.double()).view(T, H, d), P.silu(k.double()).view(T, H, d),
                                      P.silu(v.double()).view(T, H, dv), decay).reshape(T, H * dv)
    state = torch.zeros(2, H, d, dv, device=DEV)
    out = torch.empty(T, H * dv, device=DEV)
    t0 = 0
    for n in [1, 65, 64, 270, 200]:
        cu, _, sl = batch_index([n], [1])
        scratch = torch.empty(K.recurrent_chunked_scratch_floats([n], H, d, dv, False), device=DEV)
        K.recurrent_chunked(q[t0:t0 + n].to(DEV, dtype), k[t0:t0 + n].to(DEV, dtype), v[t0:t0 + n].to(DEV, dtype), state,
                            cu, sl, [n], out[t0:t0 + n], scratch, H, H, d, dv, decay=torch.tensor(decay, device=DEV))
        t0 += n
    close(out, want, torch.float32, "decayed linear attention in chunks", f32=1e-4)
    assert float(state[0].abs().max()) == 0.0


# ----------------------------------------------------------------------------- window attention pieces
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,rot", [(4, 2, 16, 32, 8), (2, 2, 48, 48, 48), (3, 1, 64, 16, 0), (8, 4, 64, 48, 64)])
def test_pair_rotation_and_padded_pages(dtype, H, G, d, dv, rot):
    T, page = 9, 4
    Dp = (max(d, dv) + 15) // 16 * 16
    q, k, v = rnd(T, H * d, seed=1), rnd(T, G * d, seed=2), rnd(T, G * dv, seed=3)
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 1000, 1001, 70000], dtype=torch.int32)
    pool = torch.full((8, 2, page, G * Dp), 9.0, dtype=dtype, device=DEV)
    table = torch.zeros(1, 20000, dtype=torch.int32, device=DEV)
    table[0, :2] = torch.tensor([5, 2]); table[0, 250] = 7; table[0, 17500] = 1
    inv = None
    if rot:
        inv = torch.pow(torch.tensor(777.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
        inv = inv.float().to(DEV)
    q_out = torch.empty(T, H * Dp, dtype=dtype, device=DEV)
    K.rope_pairs_store(q.to(DEV, dtype), k.to(DEV, dtype), v.to(DEV, dtype), inv, rot, positions.to(DEV),
                       torch.zeros(T, dtype=torch.int32, device=DEV), table, pool, q_out, H, G, d, dv, Dp)
    qr = P.rotate_pairs(q.double().view(T, H, d), positions, rot, 777.0) if rot else q.double().view(T, H, d)
    kr = P.rotate_pairs(k.double().view(T, G, d), positions, rot, 777.0) if rot else k.double().view(T, G, d)
    # angles are float: at position 70,000 the angle's rounding alone is 4e-3 radians
    tol = dict(f32=2e-5, bf16=1e-2)
    close(q_out.view(T, H, Dp)[:6, :, :d], qr[:6], dtype, "q", **tol)
    close(q_out.view(T, H, Dp)[6:8, :, :d], qr[6:8], dtype, "q at 1000", f32=2e-4)
    close(q_out.view(T, H, Dp)[8:, :, :d], qr[8:], dtype, "q at 70000", f32=2e-2, bf16=3e-2)
    assert float(q_out.view(T, H, Dp)[:, :, d:].abs().max() if Dp > d else 0.0) == 0.0
    where = {0: (5, 0), 3: (5, 3), 4: (2, 0), 6: (7, 0), 7: (7, 1), 8: (1, 0)}
    for t, (pg, r) in where.items():
        krow, vrow = pool[pg, 0, r].view(G, Dp), pool[pg, 1, r].view(G, Dp)
        close(krow[:, :d], kr[t], dtype, f"key {t}", f32=2e-2 if t == 8 else 2e-4, bf16=3e-2)
        close(vrow[:, :dv], v.double().view(T, G, dv)[t], dtype, f"value {t}", f32=0.0, bf16=1e-2)
        assert float(vrow[:, dv:].abs().max() if Dp > dv else 0.0) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 16, 17, 40, 0])
def test_window_edge_and_sink_stand_out(dtype, window):
    """One key just inside the window and one just outside it carry scores far above the rest, and the
    sink is large: a window that is one token off, or a sink left out, changes the result by order one.
    Prompt rows and rows decoded one by one, across page borders, with key ranges."""
    H, G, Dh, page, T = 4, 2, 32, 16, 150
    q, k, v = rnd(T, H * Dh, seed=1, scale=0.3), rnd(T, G * Dh, seed=2, scale=0.3), rnd(T, G * Dh, seed=3)
    qh, kh = q.view(T, H, Dh), k.view(T, G, Dh)
    w = window if window > 0 else T
    for i in range(T):  # the keys at distance w - 1 (seen) and w (not seen) match the query's direction
        for j in (i - w + 1, i - w):
            if j >= 0 and j != i:
                kh[j] += 0.05 * qh[i, ::2] / (qh[i, ::2].norm(dim=-1, keepdim=True) ** 2) * 40.0
    k = kh.reshape(T, G * Dh).to(torch.bfloat16).float()
    sink = torch.tensor([3.0, -2.0, 0.5, 6.0])
    scale = 0.7
    want = P.windowed_sink_attention(q.double().view(T, H, Dh), k.double().view(T, G, Dh), v.double().view(T, G, Dh),
                                     scale, w, sink.double()).reshape(T, H * Dh)
    other = P.windowed_sink_attention(q.double().view(T, H, Dh), k.double().view(T, G, Dh), v.double().view(T, G, Dh),
                                      scale, w + 1, sink.double()).reshape(T, H * Dh)
    if window > 0:
        assert float((want - other).abs().max()) > 0.3  # the test can tell the two apart
    n_pages = (T + page - 1) // page
    pool = torch.zeros(n_pages + 2, 2, page, G * Dh, dtype=dtype, device=DEV)
    table = torch.tensor([list(range(n_pages, 0, -1))], dtype=torch.int32, device=DEV)  # pages out of order
    qd = torch.empty(T, H * Dh, dtype=dtype, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq0 = torch.zeros(T, dtype=torch.int32, device=DEV)
    K.rope_pairs_store(q.to(DEV, dtype), k.to(DEV, dtype), v.to(DEV, dtype), None, 0, pos, seq0, table, pool, qd,
                       H, G, Dh, Dh, Dh)
    for n_splits, split_len in ((1, 0), (3, 64)):
        out = torch.empty(T, H * Dh, dtype=dtype, device=DEV)
        scratch = torch.empty(K.attention_scratch_floats(T, H, Dh, n_splits), device=DEV) if n_splits > 1 else None
        K.paged_attention(qd, pool, table, pos, seq0, out, H, G, Dh, scale, window=window, n_splits=n_splits,
                          split_len=split_len, scratch=scratch, sink=sink.to(DEV))
        close(out, want, dtype, f"prompt rows, {n_splits} key ranges", f32=2e-5, bf16=3e-2)
        one = torch.empty(1, H * Dh, dtype=dtype, device=DEV)
        for t in (0, 1, w - 1, w, w + 1, 15, 16, 17, T - 1):
            if 0 <= t < T:
                K.paged_attention(qd[t:t + 1], pool, table, pos[t:t + 1], seq0[:1], one, H, G, Dh, scale, window=window,
                                  n_splits=n_splits, split_len=split_len, scratch=scratch, sink=sink.to(DEV))
                close(one, want[t:t + 1], dtype, f"row {t} alone", f32=2e-5, bf16=3e-2)


@pytest.mark.parametrize("window", [40, 64, 65, 200, 0])
@pytest.mark.parametrize("H,G,Dh", [(4, 2, 64), (8, 1, 64), (2, 2, 128)])
def test_tensor_core_attention_with_sink_and_window(window, H, G, Dh, monkeypatch):
    """The same standing-out keys and sinks through every bfloat16 attention kernel: tcgen05 and
    mma.sync prompt tiles, decode tiles with TMA and with cp.async gathers, one and several key ranges."""
    dtype, page, T = torch.bfloat16, 64, 330
    q, k, v = rnd(T, H * Dh, seed=1, scale=0.3), rnd(T, G * Dh, seed=2, scale=0.3), rnd(T, G * Dh, seed=3)
    qh, kh = q.view(T, H, Dh), k.view(T, G, Dh)
    w = window if window > 0 else T
    rep = H // G
    for i in range(T):
        for j in (i - w + 1, i - w):
            if j >= 0 and j != i:
                kh[j] += qh[i, ::rep] / (qh[i, ::rep].norm(dim=-1, keepdim=True) ** 2) * 2.0
    k = kh.reshape(T, G * Dh).to(torch.bfloat16).float()
    sink = torch.linspace(-2.0, 5.0, H)
    scale = 0.9
    args = (q.double().view(T, H, Dh), k.double().view(T, G, Dh), v.double().view(T, G, Dh), scale)
    want = P.windowed_sink_attention(*args, w, sink.double()).reshape(T, H * Dh)
    if window > 0:
        assert float((want - P.windowed_sink_attention(*args, w + 1, sink.double()).reshape(T, H * Dh)).abs().max()) > 0.15
    assert float((want - P.windowed_sink_attention(*args, w, sink.double() - 50.0).reshape(T, H * Dh)).abs().max()) > 0.3
    n_pages = (T + page - 1) // page
    pool = torch.zeros(n_pages + 2, 2, page, G * Dh, dtype=dtype, device=DEV)
    table = torch.tensor([list(range(n_pages, 0, -1))], dtype=torch.int32, device=DEV)
    qd = torch.empty(T, H * Dh, dtype=dtype, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seq0 = torch.zeros(T, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    K.rope_pairs_store(q.to(DEV, dtype), k.to(DEV, dtype), v.to(DEV, dtype), None, 0, pos, seq0, table, pool, qd,
                       H, G, Dh, Dh, Dh)
    counter = torch.zeros(4096, dtype=torch.int32, device=DEV)
    sk = sink.to(DEV)
    for n_splits, split_len in ((1, 0), (3, 128)):
        scratch = torch.empty(K.attention_scratch_floats(T, H, Dh, n_splits), device=DEV) if n_splits > 1 else None
        out = torch.zeros(T, H * Dh, dtype=dtype, device=DEV)
        K.attention_tc(qd, pool, table, pos, cu, [T], out, H, G, Dh, scale, window=window, n_splits=n_splits,
                       split_len=split_len, scratch=scratch, split_counter=counter, sink=sk)
        close(out, want, dtype, f"tcgen05 prompt rows, {n_splits} key ranges", bf16=3e-2)
        out.zero_()
        K.paged_attention(qd, pool, table, pos, seq0, out, H, G, Dh, scale, window=window, n_splits=n_splits,
                          split_len=split_len, scratch=scratch, cu_seqlens=cu, new_lens=[T], split_counter=counter, sink=sk)
        close(out, want, dtype, f"mma.sync prompt rows, {n_splits} key ranges", bf16=3e-2)
        for tma in (True, False):
            monkeypatch.setattr(K, "_TMA_DECODE", tma)
            for t in (0, 1, w - 1, w, w + 1, 63, 64, 65, 127, 128, T - 1):
                if 0 <= t < T:
                    one = torch.zeros(1, H * Dh, dtype=dtype, device=DEV)
                    K.flash_decode_attention(qd[t:t + 1], None, None, 1.0, 1.0, 1.0, None, pool, table, pos[t:t + 1], one,
                                             H, G, Dh, scale, window=window, n_splits=n_splits, split_len=split_len,
                                             scratch=scratch, split_counter=counter, sink=sk)
                    close(one, want[t:t + 1], dtype, f"decode row {t}, tma {tma}, {n_splits} key ranges", bf16=3e-2)
    assert int(counter.abs().sum()) == 0
    K.check_status(DEV, wait=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_convolution_without_activation_carries_its_window(dtype, taps):
    C, lens = 24, [11, 1, 6]
    T = sum(lens)
    x, w, b = rnd(T, C, seed=1), rnd(C, taps, seed=2), rnd(C, seed=3)
    want, t0 = [], 0
    for n in lens:
        want.append(P.causal_conv(x[t0:t0 + n].double() + b.double(), w.double()))
        t0 += n
    want = torch.cat(want)
    window = torch.full((4, taps - 1, C), 5.0, device=DEV)
    slots = [2, 0, 3]
    for s in slots:
        window[s].zero_()
    ones = torch.ones(C, device=DEV)
    out = torch.empty(T, C, dtype=dtype, device=DEV)
    xd = x.to(DEV, dtype)
    # first step: 4, 1 and 2 tokens; then the rest of the first and third one token at a time
    first = [4, 1, 2]
    starts = [0, 11, 12]
    rows = [r for i in range(3) for r in range(starts[i], starts[i] + first[i])]
    cu, seq_of, sl = batch_index(first, slots)
    o = torch.empty(len(rows), C, dtype=dtype, device=DEV)
    xin = xd[torch.tensor(rows, device=DEV)].contiguous()
    K.conv1d_fwd(xin, ones, b.to(DEV), w.to(DEV), None, window, seq_of, cu, sl, o, weight_t=w.t().contiguous().to(DEV),
                 activation=False)
    K.conv1d_window_update(xin, ones, b.to(DEV), window, cu, sl, 3, taps)
    out[torch.tensor(rows, device=DEV)] = o
    for step in range(7):
        rows = [starts[0] + 4 + step] + ([starts[2] + 2 + step] if step < 4 else [])
        sl = torch.tensor([2, 3][:len(rows)], dtype=torch.int32, device=DEV)
        o = torch.empty(len(rows), C, dtype=dtype, device=DEV)
        K.conv1d_decode(xd[torch.tensor(rows, device=DEV)].contiguous(), ones, b.to(DEV), w.to(DEV), None, window, sl, o,
                        activation=False)
        out[torch.tensor(rows, device=DEV)] = o
    close(out, want, dtype, "convolution", f32=1e-5, bf16=2e-2)
    if taps > 1:
        assert float(window[1].min()) == 5.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_norm_with_sigmoid_gate_on_float_rows(dtype):
    T, H, dv = 6, 3, 40
    o, z, w = rnd(T, H * dv, seed=1, scale=5.0), rnd(T, H * dv, seed=2), rnd(dv, seed=3) + 1.0
    want = (P.rms_unit(o.double().view(T, H, dv), 1e-5) * w.double() * torch.sigmoid(z.double()).view(T, H, dv))
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    K.gated_norm(o.to(DEV), z.to(DEV, dtype), 1.0, None, w.repeat(H).to(DEV), 1e-5, H, True, out, gate="sigmoid")
    close(out, want.reshape(T, H * dv), dtype, "per-head norm with sigmoid gate")
    want1 = P.norm_plain(o.double(), w.repeat(H).double(), 1e-5) * torch.sigmoid(z.double())
    K.gated_norm(o.to(DEV), z.to(DEV, dtype), 1.0, None, w.repeat(H).to(DEV), 1e-5, 1, True, out, gate="sigmoid")
    close(out, want1, dtype, "norm over all heads with sigmoid gate")
