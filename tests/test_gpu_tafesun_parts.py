"""Each mechanism of the Tafesun parts alone against its plain function (GPU): the kernels and parts
are called as the model calls them, on inputs made so that a fault shows."""
import types

import pytest
import torch

from plain import tafesun_plain as P

from poor_mans_mamba_b200.engine.workspace import Workspace
from poor_mans_mamba_b200.kernels import ops as K
from poor_mans_mamba_b200.parts.base import PartSpec, build_part
import poor_mans_mamba_b200.parts  # noqa: F401  (registration)

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


# ----------------------------------------------------------------------------- the tanh norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [72, 100, 1031, 2048])
def test_tanh_norm_with_the_residual_fold(dtype, D):
    T = 6
    h = rnd(T, D, seed=1, scale=2.0)
    a, b = rnd(T, D, seed=2), rnd(T, D, seed=3, scale=3.0)
    trio = lambda s: (torch.tensor([0.3 + 0.1 * s]), rnd(D, seed=10 + s) + 1.0, rnd(D, seed=20 + s))
    pre, post = trio(1), trio(2)
    dev = lambda t3: tuple(t.to(DEV) for t in t3)
    ad, bd = a.to(DEV, dtype), b.to(DEV, dtype)
    # the norm alone
    hd = h.to(DEV).clone()
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    K.add_tanh_norm(hd, [], None, dev(pre), out)
    close(out, P.tanh_norm(h.double(), *[t.double() for t in pre]), dtype, "norm")
    assert torch.equal(hd.cpu(), h)
    # two scaled branches, normed once more before they join, then the norm of the new stream
    s = 0.8 * ad.float().cpu().double() + 1.3 * bd.float().cpu().double()
    new = h.double() + P.tanh_norm(s, *[t.double() for t in post])
    K.add_tanh_norm(hd, [(ad, 0.8), (bd, 1.3)], dev(post), dev(pre), out)
    close(hd, new, torch.float32, "stream after the fold")
    close(out, P.tanh_norm(new, *[t.double() for t in pre]), dtype, "norm after the fold")
    # listed rows only: the stream stays as it is
    hd = h.to(DEV).clone()
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, D, dtype=dtype, device=DEV)
    K.add_tanh_norm(hd, [(ad, 0.8), (bd, 1.3)], dev(post), dev(pre), out3, rows)
    close(out3, P.tanh_norm(new, *[t.double() for t in pre])[[4, 0, 4]], dtype, "rows")
    assert torch.equal(hd.cpu(), h)
    # fold without a norm following, and a sublayer's result normed by itself
    K.add_tanh_norm(hd, [(ad, 0.8), (bd, 1.3)], dev(post), None, None)
    close(hd, new, torch.float32, "fold alone")
    K.add_tanh_norm(None, [(ad, 0.8), (bd, 1.3)], None, dev(post), out)
    close(out, P.tanh_norm(s, *[t.double() for t in post]), dtype, "applied alone")


# ----------------------------------------------------------------------------- rotation, biases, padded heads
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,rot,factor", [(4, 2, 16, 24, 8, 2.0), (2, 1, 32, 16, 32, 8.0), (1, 1, 8, 40, 0, 1.0),
                                                 (8, 2, 64, 96, 48, 3.0), (3, 3, 24, 8, 24, 1.0)])
def test_half_layout_rotation_into_the_pages(dtype, H, G, d, dv, rot, factor):
    """Positions up to 1,000 in two sequences whose pages are not in order; the rotated queries and what the
    pages hold afterwards against the plain rotation (values unrotated, heads padded with zeros)."""
    page, Dp = 16, (max(d, dv) + 15) // 16 * 16
    positions = [0, 1, 15, 16, 17, 999, 1000, 5, 31, 32]
    seq = [0, 0, 0, 0, 0, 0, 0, 1, 1, 1]
    T = len(positions)
    q, k, v = rnd(T, H * d, seed=1), rnd(T, G * d, seed=2), rnd(T, G * dv, seed=3)
    qb, kb, vb = rnd(H * d, seed=4), rnd(G * d, seed=5), rnd(G * dv, seed=6)
    n_blocks = 1000 // page + 1
    perm = torch.randperm(2 * n_blocks, generator=torch.Generator().manual_seed(7)).to(torch.int32)
    table = perm.view(2, n_blocks).to(DEV)
    pool = torch.zeros(2 * n_blocks, 2, page, G * Dp, dtype=dtype, device=DEV)
    inv = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        inv = (torch.pow(torch.tensor(1000.0, dtype=torch.float64), -2.0 * i / rot) / factor).float().to(DEV)
    q_out = torch.empty(T, H * Dp, dtype=dtype, device=DEV)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    K.rope_pairs_store(q.to(DEV, dtype), k.to(DEV, dtype), v.to(DEV, dtype), inv, rot, pos_t,
                       torch.tensor(seq, dtype=torch.int32, device=DEV), table, pool, q_out, H, G, d, dv, Dp,
                       half_layout=True, biases=(qb.to(DEV), kb.to(DEV), vb.to(DEV)))
    pos64 = torch.tensor(positions)
    want_q = P.rotate_halves((q + qb).double().view(T, H, d), pos64, rot, 1000.0, factor)
    want_k = P.rotate_halves((k + kb).double().view(T, G, d), pos64, rot, 1000.0, factor)
    got_q = q_out.view(T, H, Dp)
    close(got_q[:, :, :d], want_q, dtype, "rotated queries", f32=3e-5)
    assert float(got_q[:, :, d:].abs().max()) == 0.0 if Dp > d else True
    for t in range(T):
        pg = int(table[seq[t], positions[t] // page])
        row_k = pool[pg, 0, positions[t] % page].view(G, Dp)
        row_v = pool[pg, 1, positions[t] % page].view(G, Dp)
        close(row_k[:, :d], want_k[t], dtype, "rotated keys in their page", f32=3e-5)
        close(row_v[:, :dv], (v + vb).double().view(T, G, dv)[t], dtype, "values in their page")
        if Dp > dv:
            assert float(row_v[:, dv:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_output_gate_on_padded_heads_and_the_clamped_activation(dtype):
    T, H, Dp, dv = 5, 3, 48, 40
    a, g = rnd(T, H * Dp, seed=1), rnd(T, H * dv, seed=2, scale=2.0)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    K.sigmoid_gate(a.to(DEV, dtype), g.to(DEV, dtype), 1.0, out, H, Dp, dv)
    want = a.double().view(T, H, Dp)[:, :, :dv] * torch.sigmoid(g.double()).view(T, H, dv)
    close(out, want.reshape(T, H * dv), dtype, "gate")
    F = 37
    gu = rnd(T, 2 * F, seed=3, scale=3.0)
    act = torch.empty(T, F, dtype=dtype, device=DEV)
    K.clamped_glu(gu.to(DEV, dtype), 1.25, 1.702, 1.0, act)
    gg = torch.clamp(gu[:, :F].double(), max=1.25)
    uu = torch.clamp(gu[:, F:].double(), min=-1.25, max=1.25)
    close(act, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), dtype, "clamped activation")
    assert float(gu[:, :F].max()) > 1.25 and float(gu[:, F:].min()) < -1.25  # the clamps were met


# ----------------------------------------------------------------------------- the gated norm in parts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I,parts", [(48, 3), (64, 1), (96, 4), (24, 2)])
def test_gated_norm_in_equal_parts(dtype, I, parts):
    T = 9
    y, z, w = rnd(T, I, seed=1), rnd(T, I, seed=2), rnd(I, seed=3) + 1.0
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    K.gated_norm(y.to(DEV, dtype), z.to(DEV, dtype), 1.0, None, w.to(DEV), 1e-5, parts, False, out)
    want = P.rms_parts(y.double() * P.silu(z.double()), parts, 1e-5) * w.double()
    close(out, want, dtype, "gated norm")


# ----------------------------------------------------------------------------- the routed feed-forward
def _routed_case(D, E, top, F, Fs, seed, T, starve=None):
    names = {"router": (E, D), "router.b": (E,)}
    for e in range(E):
        names.update({f"e{e}.gate": (F, D), f"e{e}.up": (F, D), f"e{e}.down": (D, F)})
    if Fs:
        names.update({"shared.gate": (Fs, D), "shared.up": (Fs, D), "shared.down": (D, Fs)})
    w = {}
    for i, (n, shape) in enumerate(names.items()):
        gain = 3.0 if n == "router" else 1.5
        w[n] = rnd(*shape, seed=seed * 1000 + i, scale=gain / (shape[-1] ** 0.5 if len(shape) > 1 else 1.0))
    if starve is not None:
        w["router.b"][starve] = -50.0  # an expert that no token chooses
    x = rnd(T, D, seed=seed + 7)
    cfg = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": 0.8}}
    if Fs:
        cfg["shared"] = {"ff": Fs, "limit": 1.7}
    return w, x, cfg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,E,top,F,Fs,T,starve", [
    (72, 5, 2, 40, 56, 33, None),      # rows of whole 16-byte groups: the tensor-core products in bfloat16
    (100, 3, 3, 20, 0, 7, None),       # every expert for every token, no shared expert, float products
    (44, 9, 1, 12, 8, 300, 4),         # one expert a token, many tiles an expert, an expert without tokens
    (64, 12, 5, 48, 80, 1, None),      # a single token
    (128, 8, 2, 96, 32, 517, 0),       # several row tiles, a ragged last one
    (256, 6, 3, 192, 64, 700, 2),      # rows of whole 128-byte pieces and many pairs: the tcgen05 products in bfloat16
    (128, 4, 1, 64, 0, 1500, None),    # the same with one expert a token
])
def test_routed_experts_against_the_plain_sum(dtype, D, E, top, F, Fs, T, starve):
    w, x, cfg = _routed_case(D, E, top, F, Fs, seed=3, T=T, starve=starve)
    part = build_part("feed_forward", PartSpec("routed_glu", "mlp", {
        "experts": E, "top": top, "expert_ff": F, "expert_limit": 0.8, "shared_ff": Fs, "shared_limit": 1.7}),
        hidden_size=D)
    params = {}
    for ps in part.param_specs():
        t = w[ps.name].to(DEV)
        params[ps.name] = t if ps.kind == "vector" else t.to(dtype)
    part.bind(params)
    part.finalize(dtype, torch.device(DEV))
    ctx = types.SimpleNamespace(workspace=Workspace(torch.device(DEV)), dtype=dtype)
    xd = x.to(DEV, dtype)
    out = torch.full((T, D), float("nan"), dtype=dtype, device=DEV)
    part.forward(xd, ctx, out)
    want = P.routed_experts(x.double(), {"mlp." + k: v.double() for k, v in w.items()}, "mlp.", cfg)
    close(out, want, dtype, "routed feed-forward", f32=3e-5, bf16=3e-2)
    # the router's choice itself, where the logits are not close
    z = x.double() @ w["router"].double().t() + w["router.b"].double()
    val, idx = torch.topk(z, top, dim=-1)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    pw = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K.moe_route(xd, params["router"], params["router.b"], top, ids, pw)
    gap = (val[:, :-1] - val[:, 1:]).min(dim=-1).values if top > 1 else torch.full((T,), 1.0, dtype=torch.float64)
    rest = torch.where(torch.zeros_like(z, dtype=torch.bool).scatter(1, idx, True), torch.full_like(z, -1e9), z)
    gap = torch.minimum(gap, val[:, -1] - rest.max(dim=-1).values) if top < E else gap
    sure = gap > 1e-3
    assert torch.equal(ids.cpu().long()[sure], idx[sure])
    if bool(sure.any()):
        close(pw[sure.to(DEV)], torch.softmax(val, dim=-1)[sure], torch.float32, "router weights", f32=1e-5)
    assert T < 8 or int(sure.sum()) >= T // 2  # (most tokens are far from a close call)
    if starve is not None:
        assert not bool((ids == starve).any())
    # the plan: every pair once, grouped by expert
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    tiles = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    perm = torch.empty(T * top, dtype=torch.int32, device=DEV)
    for tc in ("float", "mma", "mma_few", "tcgen05"):
        K.moe_plan(ids, E, tc, offsets, tiles, perm)
        assert sorted(perm.cpu().tolist()) == list(range(T * top))
        flat, off, rows = ids.view(-1).cpu(), offsets.cpu().tolist(), K.moe_tile_rows(tc)
        assert off[0] == 0 and off[-1] == T * top
        for e in range(E):
            mine = perm.cpu()[off[e]:off[e + 1]].long()
            assert bool((flat[mine] == e).all()) and mine.tolist() == sorted(mine.tolist())
        assert tiles.cpu().tolist() == [sum(-(-(off[j + 1] - off[j]) // rows) for j in range(e)) for e in range(E + 1)]
