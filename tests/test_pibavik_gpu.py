"""The Pibavik decoder in the engine against the plain statement (tests/plain_pibavik.py): each mechanism's kernels
alone, then whole models through the step function, the cache manager and the scheduler."""
import numpy as np
import pytest
import torch

import plain_pibavik as PP
import replay_util as R
from engine_fixtures import make_runner
from pibavik_fixtures import CONFIGS, TOL, make_requests, model_dir, plain_logits, plain_model
from test_banelix_gpu import _Alone, _i32, _rel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rebind(a):
    a.part.bind({k: v.to(DEV) for k, v in a.w.items()})


def _feed(a, h, first, sizes, rid="r"):
    """The rows of h through the mixer: a portion of ``first`` rows, portions of ``sizes``, then single tokens."""
    outs, at = [a.step([(rid, h[:first])])[rid]], first
    for size in sizes:
        if at >= h.shape[0]:
            break
        outs.append(a.step([(rid, h[at:at + size])])[rid])
        at += size
    while at < h.shape[0]:
        outs.append(a.step([(rid, h[at:at + 1])])[rid])
        at += 1
    return torch.cat(outs)


# ---- small kernels ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,rot", [(4, 2, 16, 16, 8), (3, 3, 10, 6, 4), (8, 2, 64, 64, 16), (1, 1, 8, 8, 0), (4, 4, 128, 128, 128)])
def test_heads_normed_with_a_shared_weight_then_turned(dtype, H, G, D, V, rot):
    from infero_b200.kernels import layer_ops as L
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(H * 100 + D)
    T, page = 6, 4
    width = 3 + H * D + G * D + G * V
    proj = torch.randn(T, width, generator=g) * 1.5
    pos = [0, 1, 7, 1000, 50001, 131071]
    base = 300.0
    freqs = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
    qw, kw = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.3 * torch.randn(D, generator=g)
    n_pages = max(pos) // page + 1
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    used = sorted({p // page for p in pos})
    table[0, used] = torch.tensor(list(reversed(range(len(used)))), dtype=torch.int32)
    kc = torch.full((len(used), G, page, D), 99.0, dtype=td, device=DEV)
    vc = torch.full((len(used), G, page, V), 99.0, dtype=td, device=DEV)
    q_out = torch.empty(T, H * D, dtype=td, device=DEV)
    L.qk_prepare(proj.to(DEV), 3, 3 + H * D, 3 + H * D + G * D, 3, qw.to(DEV), kw.to(DEV), 1e-5, freqs.to(DEV) if rot else None,
                 1.0, _i32(pos), _i32([0] * T), table.to(DEV), page, q_out, kc, vc, H, G, D, V)
    p64 = proj.double()
    q = PP.rms_norm(p64[:, 3:3 + H * D].view(T, H, D), qw.double(), 1e-5)
    k = PP.rms_norm(p64[:, 3 + H * D:3 + H * D + G * D].view(T, G, D), kw.double(), 1e-5)
    v = p64[:, 3 + H * D + G * D:].view(T, G, V)

    def turn(x):                                   # x [T, n, D] at the positions above
        half = rot // 2
        ang = torch.tensor(pos, dtype=torch.float64).view(T, 1, 1) * freqs.view(1, 1, half)
        c, s_ = torch.cos(ang), torch.sin(ang)
        u, v_ = x[..., :half], x[..., half:rot]
        return torch.cat([u * c - v_ * s_, v_ * c + u * s_, x[..., rot:]], dim=-1)
    q, k = turn(q), turn(k)
    tol = 4e-6 if dtype == "float32" else 6e-3
    assert _rel(q_out, q.reshape(T, H * D)) < tol
    for t, p in enumerate(pos):
        pg = int(table[0, p // page])
        assert _rel(kc[pg, :, p % page], k[t]) < tol and _rel(vc[pg, :, p % page], v[t]) < tol


@pytest.mark.parametrize("n,parts,gated", [(128, 2, True), (30, 3, True), (48, 1, False), (1024, 4, True), (7, 7, True)])
def test_the_gated_norm_in_equal_parts(n, parts, gated):
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(n)
    T = 9
    wide = torch.randn(T, 2 * n + 5, generator=g) * 2
    w = 1 + 0.3 * torch.randn(n, generator=g)
    y, z = wide[:, 2:2 + n], wide[:, 5 + n:5 + 2 * n]
    v = y.double() * PP.silu(z.double()) if gated else y.double()
    want = PP.grouped_rms_norm(v, w.double(), parts, 1e-5) * 0.8
    wd = wide.to(DEV)
    for td, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
        out = torch.zeros(T, n + 3, dtype=td, device=DEV)
        L.gated_group_norm(wd[:, 2:2 + n], wd[:, 5 + n:5 + 2 * n] if gated else None, w.to(DEV), 1e-5, parts, out[:, 3:], 0.8)
        assert _rel(out[:, 3:], want) < tol and float(out[:, :3].abs().max()) == 0.0


def test_experts_are_chosen_by_their_scores():
    """Sigmoid scores, the largest chosen, the lowest index on a tie, weights as they are or over their sum."""
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(3)
    for E, top in ((12, 1), (5, 5), (7, 3), (64, 8), (1, 1)):
        z = torch.randn(33, E + 2, generator=g) * 3
        z[0, :E] = 0.5                                # all equal: the first `top` experts
        z[1, :E] = -30.0                              # scores that vanish
        z[2, :E] = 40.0                               # scores that are 1 in 32-bit: a tie among all
        if E > 2:
            z[3, 1] = z[3, 2] = 9.0                   # a tie between neighbours
        s = torch.sigmoid(z[:, :E].float()).double()
        for renorm in (False, True):
            idx, w = L.moe_select_scored(z.to(DEV), E, top, renorm=renorm)
            idx, w = idx.cpu(), w.cpu().double()
            for t in range(z.shape[0]):
                order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
                assert idx[t].tolist() == order, (E, top, t)
                want = s[t, order] / (s[t, order].sum() + 1e-20) if renorm else s[t, order]
                assert float((w[t] - want).abs().max()) < 1e-6


def _moe_case(E, top, ff, d, T, shared, seed):
    g = torch.Generator().manual_seed(seed)
    w = {"mlp.router": torch.randn(E, d, generator=g) * 1.2 / d ** 0.5}
    for e in range(E):
        w[f"mlp.e{e}.up"] = torch.randn(ff, d, generator=g) * 0.2
        w[f"mlp.e{e}.down"] = torch.randn(d, ff, generator=g) * 0.2
    if shared:
        w["mlp.shared.up"] = torch.randn(shared, d, generator=g) * 0.2
        w["mlp.shared.down"] = torch.randn(d, shared, generator=g) * 0.2
    return w, torch.randn(T, d, generator=g)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,ff,d,T,shared", [(6, 2, 64, 128, 3, 32), (6, 2, 64, 128, 40, 32), (5, 5, 20, 36, 11, 0),
                                                 (10, 1, 80, 160, 700, 48), (1, 1, 16, 40, 5, 0), (8, 3, 128, 256, 300, 0)])
def test_routed_experts_that_read_their_weighted_input(dtype, E, top, ff, d, T, shared):
    """Few tokens (every pair streams its expert), many tokens (grouped tensor-core products in bf16), odd sizes."""
    from infero_b200 import parts                                                # noqa: F401
    from infero_b200.config.spec import FeedForwardSpec
    from infero_b200.registry import part_class
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    w, h = _moe_case(E, top, ff, d, T, shared, seed=E * 10 + T)
    w = {k: v.to(td).float() for k, v in w.items()}
    h = h.to(td).float()
    spec = FeedForwardSpec(kind="moe_scored", hidden=d, intermediate=ff, experts=E, top=top, shared_intermediate=shared,
                           activation="relu2", route_score="sigmoid", route_renorm=False, weight_input=True, weight_suffix="")
    part = part_class("feed_forward", "moe_scored")(spec, "l0")
    part.bind({"l0." + k: v.to(td).to(DEV) for k, v in w.items()})
    ctx = type("Ctx", (), {"act_dtype": td})()
    got = part.forward(ctx, h.to(td).to(DEV))
    if hasattr(got, "materialize"):
        got = got.materialize(torch.float32)
    ml = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = PP.routed_experts(h.double(), {k: v.double() for k, v in w.items()}, "mlp", ml)
    if dtype == "bfloat16":
        # a token whose choice hangs on a near tie may go either way in 16 bits: compare where the choice is clear
        s = (h.double() @ w["mlp.router"].double().T).sort(dim=1, descending=True).values
        clear = torch.ones(T, dtype=torch.bool) if top == E else (s[:, top - 1] - s[:, top]) > 0.01
        assert int(clear.sum()) >= T // 2
        assert _rel(got.float().cpu()[clear], want[clear]) < 3e-2
    else:
        assert _rel(got, want) < 1e-5


# ---- the mixers alone ---------------------------------------------------------------------------------------------
def _biased_spec(H, G, D, V, window, d, scale=0.3, borrows=False, keep=None):
    from infero_b200.config.spec import MixerSpec
    return MixerSpec(kind="normed_attention", hidden=d, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=V, scale=scale,
                     window=window, keep_window=keep or window, distance_slope_exp=8.0, borrows_cache=borrows, norm_eps=1e-5,
                     weight_suffix="")


def _biased_dict(H, G, D, V, window, scale=0.3):
    return {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale, "mask": {"size": window}}


def _plain_biased(a, h, m, owner=None):
    w = a.weights()
    kv = PP.biased_keys_values(h.double(), (owner or a).weights(), "mix", m)
    return PP.biased_attention(h.double(), w, "mix", m, kv)[:, :m["heads"] * m["vdim"]]


BIASED_SHAPES = [(2, 1, 8, 8, 5), (6, 2, 6, 10, 7), (4, 2, 64, 64, 24), (3, 3, 16, 24, 33), (4, 1, 128, 128, 100), (1, 1, 12, 5, 1),
                 (8, 2, 64, 32, 70), (16, 2, 64, 64, 300)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,window", BIASED_SHAPES)
def test_attention_with_a_distance_bias_in_portions_and_single_tokens(dtype, H, G, D, V, window):
    d = max(64, H * V)
    scale = 48.0 / (d * D ** 0.5)                  # scores of a few units whatever the sizes
    m = _biased_dict(H, G, D, V, window, scale)
    a = _Alone(_biased_spec(H, G, D, V, window, d, scale), dtype, pages=128)
    g = torch.Generator().manual_seed(7)
    n = min(3 * window + 40, 700)
    h1, h2 = torch.randn(n, d, generator=g), torch.randn(50, d, generator=g)
    if dtype == "bfloat16":
        h1, h2 = h1.bfloat16().float(), h2.bfloat16().float()
    got1 = [a.step([("a", h1[:window + 3]), ("b", h2[:2])])]
    got1.append(a.step([("b", h2[2:50]), ("a", h1[window + 3:window + 4])]))
    at = window + 4
    outs = [got1[0]["a"], got1[1]["a"]]
    for size in (2, 1, 1, window - 1 or 1, window, 1, window + 1, 17):
        outs.append(a.step([("a", h1[at:at + size])])["a"])
        at += size
    while at < n:
        outs.append(a.step([("a", h1[at:at + 1])])["a"])
        at += 1
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert _rel(torch.cat(outs)[:, :H * V], _plain_biased(a, h1, m)) < tol
    assert _rel(torch.cat([got1[0]["b"], got1[1]["b"]])[:, :H * V], _plain_biased(a, h2, m)) < tol
    a.close("b")                                   # a request that starts on pages and in a slot another gave back
    assert _rel(a.step([("c", h2[:20])])["c"][:, :H * V], _plain_biased(a, h2[:20], m)) < tol


def test_the_distance_bias_moves_the_weight_towards_near_keys():
    """Equal keys everywhere: without the bias every visible key would weigh the same; with it head h's weights fall off
    by exp(-slope_h) per token, so the result leans to the latest values, the first head most."""
    H, G, D, V, window, d = 4, 1, 16, 16, 30, 64
    m = _biased_dict(H, G, D, V, window, scale=1.0)
    a = _Alone(_biased_spec(H, G, D, V, window, d, scale=1.0), "float32")
    a.w["l0.mix.k"] = torch.zeros_like(a.w["l0.mix.k"])
    _rebind(a)
    h = torch.randn(40, d, generator=torch.Generator().manual_seed(2))
    got = a.step([("r", h)])["r"][:, :H * V].double()
    assert _rel(got, _plain_biased(a, h, m)) < 1e-5
    v = h.double() @ a.weights()["mix.v"].T
    slopes = PP.distance_slopes(H)
    for head in range(H):
        wts = torch.exp(-slopes[head] * torch.arange(window, dtype=torch.float64))          # distance 0 .. window - 1
        want = (wts.unsqueeze(1) * v[39 - torch.arange(window)]).sum(0) / wts.sum()
        assert float((got[39, head * V:(head + 1) * V] - want).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("back", [0, 1, 15, 16, 17, 38, 39, 40, 41, 47, 48, 49])
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_stands_out_inside_the_window_and_vanishes_outside_it(dtype, back, decode):
    """One key carries almost all the weight for the last query; it sits `back` tokens before it.  Inside a window of 40
    (back <= 39) the result is that key's value; one further back and it is gone.  In a portion and token by token."""
    H, G, D, V, window, d = 2, 1, 64, 64, 40, 128
    m = _biased_dict(H, G, D, V, window, scale=0.02)
    a = _Alone(_biased_spec(H, G, D, V, window, d, scale=0.02), dtype, seed=back)
    # every query head is projected as the key head is, but from the input with its second half negated: the query of
    # a token whose input is an earlier token's with that half negated is that token's key, its own key points elsewhere
    a.w["l0.mix.q"] = torch.cat([a.w["l0.mix.k"]] * H)
    a.w["l0.mix.q"][:, d // 2:] *= -1
    _rebind(a)
    g = torch.Generator().manual_seed(back)
    n = 70
    h = torch.randn(n, d, generator=g)
    h[n - 1] = h[n - 1 - back]
    h[n - 1, d // 2:] *= -1
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    want = _plain_biased(a, h, m)
    if decode:
        got = torch.cat([a.step([("r", h[:n - 50])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 50, n)])
    else:
        got = torch.cat([a.step([("r", h[:11])])["r"], a.step([("r", h[11:])])["r"]])
    assert _rel(got[:, :H * V], want) < (3e-5 if dtype == "float32" else 4e-2)
    h2 = h.clone()
    h2[n - 1 - back] = 0.0
    moved = _rel(_plain_biased(a, h2, m)[-1:], want[-1:])
    assert (moved > 0.3) if back < window else (moved < 1e-9)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_that_borrows_keys_and_values_looks_further_back_than_their_owner(dtype):
    H, G, D, V, d = 4, 2, 16, 24, 96
    owner = _Alone(_biased_spec(H, G, D, V, 9, d, keep=21), dtype, seed=1)
    reader = _Alone(_biased_spec(2 * H, G, D, V, 21, 2 * H * V, borrows=True, keep=21), dtype, seed=2, cache=owner.kv)
    assert not any(k.endswith((".k", ".v")) for k in reader.w)
    reader.free, reader.table = owner.free, owner.table                # the two layers share pages and block tables
    g = torch.Generator().manual_seed(5)
    h = torch.randn(60, d, generator=g)
    x = torch.randn(60, 2 * H * V, generator=g)
    if dtype == "bfloat16":
        h, x = h.bfloat16().float(), x.bfloat16().float()
    outs = []
    for lo, hi in ((0, 13), (13, 14), (14, 40), (40, 41), (41, 42), (42, 60)):
        owner.step([("r", h[lo:hi])])
        reader.length["r"] = lo
        outs.append(reader.step([("r", x[lo:hi])], write_cache=False)["r"])
    m = _biased_dict(2 * H, G, D, V, 21)
    w = reader.weights()
    kv = PP.biased_keys_values(h.double(), owner.weights(), "mix", _biased_dict(H, G, D, V, 9))
    want = PP.biased_attention(x.double(), w, "mix", m, kv)
    assert _rel(torch.cat(outs)[:, :2 * H * V], want[:, :2 * H * V]) < (2e-5 if dtype == "float32" else 3e-2)


def _left_spec(H, G, D, V, window, d, dims, scale=0.3, names=()):
    from infero_b200.config.spec import MixerSpec, PositionSpec
    pos = PositionSpec("rope_neox", 700.0, dims) if dims else None
    return MixerSpec(kind="normed_attention", hidden=d, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=V, scale=scale,
                     window=window, position=pos, qk_norm_kind="head", out_gate=True, norm_eps=1e-5, names=names, weight_suffix="")


def _left_dict(H, G, D, V, window, dims, scale=0.3):
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if dims:
        m["rot"] = {"base": 700.0, "dims": dims}
    return m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,window,dims", [(4, 2, 64, 64, 24, 16), (3, 3, 10, 6, 7, 4), (4, 1, 128, 128, 60, 128), (2, 1, 16, 16, None, 0),
                                                (4, 4, 64, 32, 40, 64)])
def test_the_gated_normed_turned_window_attention(dtype, H, G, D, V, window, dims):
    d = max(64, H * V)
    a = _Alone(_left_spec(H, G, D, V, window, d, dims), dtype, pages=64)
    a.w["l0.mix.q"] = a.w["l0.mix.q"] * 2.0
    _rebind(a)
    m = _left_dict(H, G, D, V, window, dims)
    g = torch.Generator().manual_seed(11)
    n = 150
    h = torch.randn(n, d, generator=g)
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    got = _feed(a, h, 70, (2, 1, 3, 17, 31))
    want = PP.left_attention(h.double(), a.weights(), "mix", m, 1e-5)[:, :H * V]
    assert _rel(got[:, :H * V], want) < (2e-5 if dtype == "float32" else 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("back", [0, 1, 16, 38, 39, 40, 41, 48])
@pytest.mark.parametrize("decode", [False, True])
def test_the_gated_mixers_window_keeps_a_key_that_stands_out_and_drops_it_one_token_later(dtype, back, decode):
    """The left mixer's own window of 40, with normed heads: the query of the last token is an earlier token's key."""
    H, G, D, V, window, d = 2, 1, 64, 64, 40, 128
    m = _left_dict(H, G, D, V, window, 0, scale=0.25)
    a = _Alone(_left_spec(H, G, D, V, window, d, 0, scale=0.25), dtype, seed=back)
    a.w["l0.mix.q"] = torch.cat([a.w["l0.mix.k"]] * H)
    a.w["l0.mix.q"][:, d // 2:] *= -1
    a.w["l0.mix.q.norm"] = a.w["l0.mix.k.norm"].clone()
    _rebind(a)
    g = torch.Generator().manual_seed(back)
    n = 70
    h = torch.randn(n, d, generator=g)
    h[n - 1] = h[n - 1 - back]
    h[n - 1, d // 2:] *= -1
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    want = PP.left_attention(h.double(), a.weights(), "mix", m, 1e-5)[:, :H * V]
    if decode:
        got = torch.cat([a.step([("r", h[:n - 50])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 50, n)])
    else:
        got = torch.cat([a.step([("r", h[:11])])["r"], a.step([("r", h[11:])])["r"]])
    assert _rel(got[:, :H * V], want) < (3e-5 if dtype == "float32" else 4e-2)
    h2 = h.clone()
    h2[n - 1 - back] = 0.0
    moved = _rel(PP.left_attention(h2.double(), a.weights(), "mix", m, 1e-5)[-1:, :H * V], want[-1:])
    assert (moved > 0.3) if back < window else (moved < 1e-9)


def _ssd_spec(Hn, P, N, G, taps, parts, d, names=()):
    from infero_b200.config.spec import MixerSpec
    return MixerSpec(kind="ssd", hidden=d, num_heads=Hn, value_dim=P, state_dim=N, rec_groups=G, norm_groups=parts,
                     conv_taps=taps, norm_eps=1e-5, names=names, weight_suffix="")


def _ssd_dict(Hn, P, N, G, taps, parts):
    return {"heads": Hn, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": parts}


def _slow_decay(a, prefix="l0.mix"):
    """Step sizes of a few hundredths: a state that lasts for hundreds of tokens."""
    a.w[prefix + ".dt_bias"] = a.w[prefix + ".dt_bias"] - 3.5
    a.w[prefix + ".in"] = a.w[prefix + ".in"] * 0.6
    _rebind(a)


SSD_SHAPES = [(4, 32, 32, 2, 4, 2), (3, 10, 5, 1, 2, 3), (2, 12, 8, 2, 1, 1), (4, 64, 128, 2, 4, 2), (1, 24, 17, 1, 3, 1), (8, 16, 48, 4, 3, 4)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hn,P,N,G,taps,parts", SSD_SHAPES)
def test_the_state_space_recurrence_in_portions_and_single_tokens(dtype, Hn, P, N, G, taps, parts):
    """Portions that cut the convolution's reach, single tokens, a second request beside the first, a slot used again."""
    d = max(64, Hn * P)
    a = _Alone(_ssd_spec(Hn, P, N, G, taps, parts, d), dtype)
    _slow_decay(a)
    m = _ssd_dict(Hn, P, N, G, taps, parts)
    g = torch.Generator().manual_seed(13)
    h1, h2 = torch.randn(120, d, generator=g), torch.randn(40, d, generator=g)
    if dtype == "bfloat16":
        h1, h2 = h1.bfloat16().float(), h2.bfloat16().float()
    first = a.step([("a", h1[:33]), ("b", h2[:1])])
    second = a.step([("b", h2[1:40]), ("a", h1[33:34])])
    outs = [first["a"], second["a"]]
    at = 34
    for size in (1, 2, 1, 3, 17, 2, 31):
        outs.append(a.step([("a", h1[at:at + size])])["a"])
        at += size
    while at < 120:
        outs.append(a.step([("a", h1[at:at + 1])])["a"])
        at += 1
    w = a.weights()
    tol = 3e-5 if dtype == "float32" else 3e-2
    assert _rel(torch.cat(outs)[:, :Hn * P], PP.right_state_space(h1.double(), w, "mix", m, 1e-5)[:, :Hn * P]) < tol
    assert _rel(torch.cat([first["b"], second["b"]])[:, :Hn * P], PP.right_state_space(h2.double(), w, "mix", m, 1e-5)[:, :Hn * P]) < tol
    a.close("b")
    assert _rel(a.step([("c", h2[:9])])["c"][:, :Hn * P], PP.right_state_space(h2[:9].double(), w, "mix", m, 1e-5)[:, :Hn * P]) < tol


def test_a_state_lasts_for_hundreds_of_tokens_and_long_portions_run_by_chunks():
    """One token writes a large state; with step sizes near zero afterwards it is still read six hundred tokens later.
    A portion of 700 tokens runs by chunks side by side, beside a short one that does not; the same tokens one portion
    of 255 at a time and token by token give the same numbers to rounding."""
    Hn, P, N, G, taps, parts, d = 2, 16, 16, 1, 2, 1, 64
    m = _ssd_dict(Hn, P, N, G, taps, parts)
    g = torch.Generator().manual_seed(21)
    n = 700
    h = torch.randn(n, d, generator=g) * 0.5
    h[5] *= 10.0
    w = None
    got = {}
    for how in ("whole", "portions", "tokens"):
        a = _Alone(_ssd_spec(Hn, P, N, G, taps, parts, d), "float32", seed=4)
        a.w["l0.mix.dt_bias"] = a.w["l0.mix.dt_bias"] - 6.0
        _rebind(a)
        w = a.weights()
        if how == "whole":
            got[how] = a.step([("x", h[:20]), ("r", h)])["r"]
        elif how == "portions":
            got[how] = torch.cat([a.step([("r", h[p:p + 255])])["r"] for p in range(0, n, 255)])
        else:
            got[how] = torch.cat([a.step([("r", h[:n - 80])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 80, n)])
    want = PP.right_state_space(h.double(), w, "mix", m, 1e-5)[:, :Hn * P]
    for how in got:
        assert _rel(got[how][:, :Hn * P], want) < 3e-5, how
    h2 = h.clone()
    h2[5] = 0.0
    moved = _rel(PP.right_state_space(h2.double(), w, "mix", m, 1e-5)[-1:, :Hn * P], want[-1:])
    assert moved > 0.005                            # the last token still reads what token 5 wrote


def _parallel_spec(left, right, d, ls=0.7, rs=1.3):
    from infero_b200.config.spec import MixerSpec, NORMED_ATTENTION_NAMES, SSD_NAMES
    import dataclasses
    rename = lambda table, side: tuple((r, leaf.replace("mix.", f"mix.{side}.", 1)) for r, leaf in table)   # noqa: E731
    return MixerSpec(kind="parallel", hidden=d, weight_suffix="", branch_scales=(ls, rs),
                     branches=(dataclasses.replace(left, names=rename(NORMED_ATTENTION_NAMES, "left")),
                               dataclasses.replace(right, names=rename(SSD_NAMES, "right"))))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [((4, 2, 64, 64, 24, 16), (4, 32, 32, 2, 4, 2)), ((3, 3, 10, 6, 7, 4), (3, 10, 5, 1, 2, 3))])
def test_the_two_mixers_side_by_side(dtype, shape):
    (H, G, D, V, window, dims), (Hn, P, N, Gs, taps, parts) = shape
    d = H * V + Hn * P
    a = _Alone(_parallel_spec(_left_spec(H, G, D, V, window, d, dims), _ssd_spec(Hn, P, N, Gs, taps, parts, d), d), dtype)
    _slow_decay(a, "l0.mix.right")
    m = {"left": _left_dict(H, G, D, V, window, dims), "right": _ssd_dict(Hn, P, N, Gs, taps, parts), "left_scale": 0.7, "right_scale": 1.3}
    g = torch.Generator().manual_seed(17)
    h = torch.randn(90, d, generator=g)
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    got = _feed(a, h, 40, (2, 1, 13))
    w = a.weights()
    want = torch.cat([0.7 * PP.left_attention(h.double(), w, "mix.left", m["left"], 1e-5)[:, :H * V],
                      1.3 * PP.right_state_space(h.double(), w, "mix.right", m["right"], 1e-5)[:, H * V:d]], dim=1)
    assert _rel(got[:, :d], want) < (3e-5 if dtype == "float32" else 3e-2)


def _latent_spec(H, D, V, C, Q, d, scale=0.3):
    from infero_b200.config.spec import MixerSpec
    return MixerSpec(kind="latent_attention", hidden=d, num_heads=H, head_dim=D, value_dim=V, latent_dim=C, q_latent_dim=Q,
                     rot_dim=0, scale=scale, norm_eps=1e-5, weight_suffix="")


def _latent_dict(H, D, V, C, Q, scale=0.3):
    return {"heads": H, "dim": D, "vdim": V, "kv_rank": C, "q_rank": Q, "scale": scale}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,C,Q", [(4, 32, 32, 64, 48), (2, 6, 10, 12, 7), (1, 8, 8, 8, 8), (4, 64, 64, 128, 96), (16, 64, 64, 64, 128)])
def test_latent_attention_with_a_query_latent_and_no_rotated_part(dtype, H, D, V, C, Q):
    d = max(64, H * V)
    scale = 48.0 / (D * Q * C) ** 0.5              # scores of a few units whatever the sizes
    a = _Alone(_latent_spec(H, D, V, C, Q, d, scale), dtype, pages=64)
    m = _latent_dict(H, D, V, C, Q, scale)
    g = torch.Generator().manual_seed(19)
    h1, h2 = torch.randn(140, d, generator=g), torch.randn(30, d, generator=g)
    if dtype == "bfloat16":
        h1, h2 = h1.bfloat16().float(), h2.bfloat16().float()
    first = a.step([("b", h2[:1]), ("a", h1[:65])])
    second = a.step([("a", h1[65:66]), ("b", h2[1:30])])
    outs = [first["a"], second["a"]]
    at = 66
    for size in (2, 1, 31, 3):
        outs.append(a.step([("a", h1[at:at + size])])["a"])
        at += size
    while at < 140:
        outs.append(a.step([("a", h1[at:at + 1])])["a"])
        at += 1
    w = a.weights()
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert _rel(torch.cat(outs)[:, :H * V], PP.latent_attention(h1.double(), w, "mix", m, 1e-5)[:, :H * V]) < tol
    assert _rel(torch.cat([first["b"], second["b"]])[:, :H * V], PP.latent_attention(h2.double(), w, "mix", m, 1e-5)[:, :H * V]) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("back", [1, 255, 256, 257, 300])
def test_a_far_key_is_found_through_the_latent(dtype, back):
    """The key that carries the weight is hundreds of tokens back, at page borders; in a portion and in single tokens."""
    H, D, V, C, Q, d = 2, 32, 32, 64, 64, 64
    a = _Alone(_latent_spec(H, D, V, C, Q, d, scale=0.25), dtype, seed=back, pages=40)
    # the queries' latent is made as the keys' is, but from the input with its second half negated, and goes up through
    # the keys' matrix: the query of a token whose input is an earlier token's with that half negated is that token's
    # key, while its own key points elsewhere
    a.w["l0.mix.dq"], a.w["l0.mix.dq.norm"], a.w["l0.mix.uq"] = a.w["l0.mix.dkv"].clone(), a.w["l0.mix.dkv.norm"].clone(), a.w["l0.mix.uk"].clone()
    a.w["l0.mix.dq"][:, d // 2:] *= -1
    _rebind(a)
    m = _latent_dict(H, D, V, C, Q, scale=0.25)
    g = torch.Generator().manual_seed(back)
    n = 330
    h = torch.randn(n, d, generator=g)
    h[n - 1] = h[n - 1 - back]
    h[n - 1, d // 2:] *= -1
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    want = PP.latent_attention(h.double(), a.weights(), "mix", m, 1e-5)[:, :H * V]
    got = torch.cat([a.step([("r", h[:n - 3])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 3, n)])
    assert _rel(got[:, :H * V], want) < (3e-5 if dtype == "float32" else 4e-2)
    h2 = h.clone()
    h2[n - 1 - back] = 0.0
    assert _rel(PP.latent_attention(h2.double(), a.weights(), "mix", m, 1e-5)[-1:, :H * V], want[-1:]) > 0.1


# ---- whole models through the step function ---------------------------------------------------------------------
def _replay(name, dtype, steps_of, lengths, seed=0, page_size=16, max_seqs=3, tol=None):
    mdir = model_dir(name)
    reqs = make_requests(name, lengths, seed=seed)
    plain = plain_logits(mdir, reqs)
    steps = steps_of(reqs)
    runner = make_runner(mdir, dtype, R.max_live_tokens(steps, reqs), page_size=page_size, max_seqs=max_seqs)
    got = R.replay_inprocess(runner, steps)
    assert len(got) > 0
    worst, where = R.compare(got, plain)
    assert worst <= (tol or TOL[dtype]), f"{name} {dtype}: {worst:.3e} at {where}"
    assert not runner.manager.requests
    return runner


ALL = [("A", "float32"), ("A_all", "bfloat16"), ("B", "float32"), ("C", "float32"), ("D", "bfloat16"), ("D", "float32")]


@pytest.mark.parametrize("name,dtype", ALL + [("B_all", "bfloat16")])
def test_whole_prompts(name, dtype):
    _replay(name, dtype, R.steps_whole, [1, 2, 15, 16, 17, 33, 131])


def test_the_residual_after_every_layer():
    from infero_b200 import kernels as K
    from infero_b200.engine import StepEntry
    from infero_b200.parts.block import PreNormBlock
    mdir = model_dir("A")
    toks = make_requests("A", [47], seed=3)["r0"]
    cfg, w = plain_model(mdir)
    trail = []
    PP.forward(cfg, w, toks, trail)
    runner = make_runner(mdir, "float32", 64)
    seen = []
    orig = PreNormBlock.forward

    def spy(self, ctx, x, delta, slot):
        pending = orig(self, ctx, x, delta, slot)
        val = pending.materialize(torch.float32) if isinstance(pending, K.Partials) else pending
        seen.append((x + val.float()).cpu())
        return pending
    PreNormBlock.forward = spy
    try:
        runner.open("a")
        runner.step([StepEntry("a", toks, [len(toks) - 1])])
    finally:
        PreNormBlock.forward = orig
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert _rel(got, trail[i]) < 1e-5, (i, _rel(got, trail[i]))


@pytest.mark.parametrize("name,dtype", ALL)
def test_prompt_then_token_by_token(name, dtype):
    _replay(name, dtype, lambda r: R.steps_tail_decode(r, tail=60), [130, 61, 5])


@pytest.mark.parametrize("name,dtype", ALL)
def test_portions_down_to_two_tokens(name, dtype):
    _replay(name, dtype, lambda r: R.steps_chunked(r, seed=2), [150, 64, 31])
    _replay(name, dtype, lambda r: R.steps_chunked(r, seed=5, sizes=(1, 2, 1, 3, 2, 16, 1, 15, 17)), [70])


@pytest.mark.parametrize("name,dtype", ALL)
def test_mixed_batches_with_slots_and_pages_used_again(name, dtype):
    """Three live requests in exactly three request slots: every later request starts in a slot and on pages that an
    ended one gave back."""
    runner = _replay(name, dtype, lambda r: R.steps_mixed(r, seed=4, max_live=3), [120, 33, 80, 17, 64, 95, 2], max_seqs=3)
    assert runner.manager.pages_reused > 0


def test_a_batch_equals_each_request_alone_bitwise_in_32_bit():
    mdir = model_dir("A")
    reqs = make_requests("A", [50, 21, 37], seed=9)
    together = R.replay_inprocess(make_runner(mdir, "float32", 256, max_seqs=3), [
        {"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}])
    alone = R.replay_inprocess(make_runner(mdir, "float32", 256, max_seqs=3), R.steps_whole(reqs))
    assert together.keys() == alone.keys()
    for k in alone:
        assert np.array_equal(together[k], alone[k]), k


def test_three_hundred_single_tokens():
    _replay("B", "float32", lambda r: R.steps_tail_decode(r, tail=300), [310], tol=6e-5)
    _replay("D", "bfloat16", lambda r: R.steps_tail_decode(r, tail=300), [305])


def test_long_prompts_in_large_portions():
    """Portions longer than the tiles of the product and attention kernels and than the recurrence's chunks, cut beside
    their edges."""
    def steps(reqs):
        (a, ta), (b, tb) = list(reqs.items())[:2]
        return [{"step": 0, "entries": [{"id": a, "tokens": ta[:257], "want": [0, 127, 128, 129, 255, 256]},
                                        {"id": b, "tokens": tb[:40], "want": [39]}], "end": []},
                {"step": 1, "entries": [{"id": b, "tokens": tb[40:425], "want": [0, 87, 88, 384]},
                                        {"id": a, "tokens": ta[257:258], "want": [0]}], "end": []},
                {"step": 2, "entries": [{"id": a, "tokens": ta[258:], "want": list(range(len(ta) - 258))},
                                        {"id": b, "tokens": tb[425:], "want": list(range(len(tb) - 425))}], "end": [a, b]}]
    _replay("D", "bfloat16", steps, [300, 450], max_seqs=2)
    _replay("A", "float32", steps, [300, 450], max_seqs=2, tol=1e-4)


def test_page_size_64():
    _replay("D", "bfloat16", lambda r: R.steps_mixed(r, seed=1, max_live=2), [130, 70, 64], page_size=64)
    _replay("B", "float32", lambda r: R.steps_mixed(r, seed=1, max_live=2), [130, 70, 64], page_size=64)


# ---- the engine's own entry point --------------------------------------------------------------------------------
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(PP.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name):
    """Several prompts queued at once, more than there are request slots, prompts cut into portions by the
    scheduler's budget, decode steps replayed from captured graphs."""
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir(name)
    cfg, w = plain_model(mdir)
    prompts = list(make_requests(name, [19, 40, 3, 27], seed=21).values())
    eng = Engine(mdir, dtype="float32", ctx=128, max_seqs=2, kv_slots=2 * 128, max_batch_tokens=32, cuda_graphs=True)
    params = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    got = eng.generate(prompts, params, max_new_tokens=10, ignore_eos=True)
    for p, g in zip(prompts, got):
        assert g == _plain_greedy(cfg, w, p, 10)
    assert eng.runner.graph_replays > 0


def test_generation_in_bf16_from_captured_graphs_equals_uncaptured_steps():
    from infero_b200.engine import Engine
    from infero_b200.sampling import SamplingParams
    mdir = model_dir("D")
    prompts = list(make_requests("D", [19, 40, 3], seed=22).values())
    params = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    outs = []
    for graphs in (True, False):
        eng = Engine(mdir, dtype="bfloat16", ctx=128, max_seqs=4, kv_slots=4 * 128, max_batch_tokens=64, cuda_graphs=graphs)
        outs.append(eng.generate(prompts, params, max_new_tokens=12, ignore_eos=True))
        if graphs:
            assert eng.runner.graph_replays > 0
    assert outs[0] == outs[1]


def test_the_trace_runner_replays_a_pibavik_folder(tmp_path):
    mdir = model_dir("A")
    reqs = make_requests("A", [70, 30], seed=2)
    steps = R.steps_mixed(reqs, seed=3, max_live=2)
    got = R.replay_subprocess(mdir, "float32", steps, R.max_live_tokens(steps, reqs), str(tmp_path), CONFIGS["A"]["vocab"])
    worst, where = R.compare(got, plain_logits(mdir, reqs))
    assert worst <= TOL["float32"], (worst, where)


def test_the_generate_command_line_on_a_pibavik_folder():
    import os
    import subprocess
    import sys
    mdir = model_dir("B")
    cfg, w = plain_model(mdir)
    prompt = make_requests("B", [21], seed=8)["r0"]
    exe = os.path.join(R.ROOT, "bin", "generate")
    proc = subprocess.run([sys.executable, exe, mdir] + [str(t) for t in prompt] +
                          ["--greedy", "--repetition-penalty", "1.0", "-n", "7", "--dtype", "float32", "--ignore-eos",
                           "--max-seq-len", "128"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    lines = proc.stdout.splitlines()
    at = next(i for i, l in enumerate(lines) if l.startswith("kv cache"))
    toks = [int(t) for t in next(l for l in lines[at + 1:] if l.strip()).split()]
    assert toks == _plain_greedy(cfg, w, prompt, 7)
