"""The Banelix decoder in the engine against the plain statement (tests/plain_banelix.py): each mechanism's kernels
alone, then whole models through the step function, the cache manager and the scheduler."""
import types

import numpy as np
import pytest
import torch

import plain_banelix as PB
import replay_util as R
from banelix_fixtures import CONFIGS, TOL, make_requests, model_dir, plain_logits, plain_model
from engine_fixtures import make_runner

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rel(got, ref):
    ref = ref.double()
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


def _i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


# ---- mechanisms alone --------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,d", [(5, 36), (7, 128), (300, 256)])
def test_the_norm_adds_a_sublayers_result_times_a_constant(T, d):
    from infero_b200 import kernels as K
    g = torch.Generator().manual_seed(d)
    x, delta, w = torch.randn(T, d, generator=g) * 2, torch.randn(T, d, generator=g), 1 + 0.2 * torch.randn(d, generator=g)
    want_x = x.double() + 0.35 * delta.double()
    want_h = PB.rms_norm(want_x, w.double(), 1e-5)
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 6e-3)):
        xd = x.to(DEV)
        out = torch.empty(T, d, dtype=dtype, device=DEV)
        K.add_rmsnorm(xd, K.Scaled(delta.to(DEV), 0.35), w.to(DEV), 1e-5, out)
        assert _rel(xd, want_x) < 1e-6 and _rel(out, want_h) < tol
    parts = torch.randn(3, T, d, generator=g)
    bias = torch.randn(d, generator=g)
    xd = x.to(DEV)
    out = torch.empty(T, d, device=DEV)
    K.add_rmsnorm(xd, K.Partials(parts.to(DEV), bias.to(DEV)), w.to(DEV), 1e-5, out, delta_scale=-1.5)
    assert _rel(xd, x.double() - 1.5 * (parts.double().sum(0) + bias.double())) < 1e-6
    rows = _i32([T - 1, 0])
    xd, out = x.to(DEV), torch.empty(2, d, device=DEV)
    K.add_rmsnorm(xd, K.Scaled(delta.to(DEV), 0.35), w.to(DEV), 1e-5, out, rows)
    assert torch.equal(xd.cpu(), x) and _rel(out, want_h[[T - 1, 0]]) < 2e-6
    xd = x.to(DEV)                                             # a factor of one adds as if there were none
    K.add_rmsnorm(xd, K.Scaled(delta.to(DEV), 1.0), w.to(DEV), 1e-5, torch.empty(T, d, device=DEV))
    assert torch.equal(xd.cpu(), x + delta)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,rot,mode", [(4, 2, 16, 16, 8, 2), (3, 3, 10, 10, 4, 2), (6, 2, 6, 10, 6, 1), (8, 2, 64, 64, 64, 1),
                                              (1, 1, 8, 8, 0, 0), (2, 1, 12, 5, 6, 1), (4, 4, 128, 128, 32, 2)])
def test_queries_and_keys_normed_and_turned_and_the_cache_written(dtype, H, G, D, V, rot, mode):
    """Both norms around the rotation, positions far out, values of their own or taken from the keys as projected."""
    from infero_b200.kernels import layer_ops as L
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(H * 100 + D)
    T, page = 6, 4
    own_v = mode != 2
    width = 3 + H * D + G * D + (G * V if own_v else 0)
    proj = torch.randn(T, width, generator=g) * 1.5
    pos = [0, 1, 7, 1000, 50001, 131071]
    freqs = torch.tensor(PB.base_frequencies(rot, 300.0), dtype=torch.float64) if rot else torch.zeros(0, dtype=torch.float64)
    amp = 1.3 if mode == 1 else 1.0
    qw, kw = 1 + 0.3 * torch.randn(H * D, generator=g), 1 + 0.3 * torch.randn(G * D, generator=g)
    n_pages = max(pos) // page + 1
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    used = sorted({p // page for p in pos})
    table[0, used] = torch.tensor(list(reversed(range(len(used)))), dtype=torch.int32)
    kc = torch.full((len(used), G, page, D), 99.0, dtype=td, device=DEV)
    vc = torch.full((len(used), G, page, V), 99.0, dtype=td, device=DEV)
    q_out = torch.empty(T, H * D, dtype=td, device=DEV)
    L.qk_prepare(proj.to(DEV), 3, 3 + H * D, 3 + H * D + G * D if own_v else -1, mode, qw.to(DEV) if mode == 1 else None,
                 kw.to(DEV) if mode == 1 else None, 1e-5, freqs.to(DEV) if rot else None, amp, _i32(pos), _i32([0] * T),
                 table.to(DEV), page, q_out, kc, vc, H, G, D, V)
    p64 = proj.double()
    q, k = p64[:, 3:3 + H * D], p64[:, 3 + H * D:3 + H * D + G * D]
    positions = torch.tensor(pos)
    if mode == 1:
        q, k = PB.rms_norm(q, qw.double(), 1e-5), PB.rms_norm(k, kw.double(), 1e-5)
    q, k = PB.rotate_half(q.view(T, H, D), positions, freqs, amp), PB.rotate_half(k.view(T, G, D), positions, freqs, amp)
    if mode == 2:
        q, k = PB.rms_norm(q, None, 1e-5), PB.rms_norm(k, None, 1e-5)
    v = p64[:, 3 + H * D + G * D:].view(T, G, V) if own_v else p64[:, 3 + H * D:3 + H * D + G * D].view(T, G, D)
    tol = 4e-6 if dtype == "float32" else 6e-3
    assert _rel(q_out, q.reshape(T, H * D)) < tol
    for t, p in enumerate(pos):
        pg = int(table[0, p // page])
        assert _rel(kc[pg, :, p % page], k[t]) < tol and _rel(vc[pg, :, p % page], v[t]) < tol
    written = {(int(table[0, p // page]), p % page) for p in pos}
    for pg in range(len(used)):
        for s in range(page):
            if (pg, s) not in written:
                assert float(kc[pg, :, s].float().min()) == 99.0 and float(vc[pg, :, s].float().min()) == 99.0


class _Alone:
    """One mixer over a hand-made paged cache and state slots: requests get shuffled pages, portions are fed in steps of
    several requests, and the part runs as the model runs it (a stand-in for the step's context).  The output weights
    are identities, so the result is what the output product is handed."""

    def __init__(self, spec, dtype, page=16, pages=96, slots=3, seed=0, cache=None):
        from infero_b200 import parts                                            # noqa: F401
        from infero_b200.registry import part_class
        self.td = torch.float32 if dtype == "float32" else torch.bfloat16
        self.spec, self.page = spec, page
        self.part = part_class("mixer", spec.kind)(spec, "l0")
        g = torch.Generator().manual_seed(seed)
        self.w = {}
        for decl in self.part.declare():
            t = torch.randn(decl.shape, generator=g) * 0.25
            if decl.role == "norm":
                t = 1 + 0.4 * t
            if decl.name.endswith(".o"):
                t = torch.zeros(decl.shape)
            if decl.name.endswith(".lam"):
                t = t - 3.5
            self.w[decl.name] = t.to(self.td)
        col = 0
        for name in [n for n in self.w if n.endswith(".o")]:                    # every branch's activations pass through
            k = self.w[name].shape[1]
            self.w[name][col:col + k] = torch.eye(k).to(self.td)
            col += k
        assert col <= spec.hidden
        self.part.bind({k: v.to(DEV) for k, v in self.w.items()})
        cs, ss = self.part.cache_spec(), self.part.state_spec()
        self.kv = cache
        if cs is not None and cache is None:
            # rows that were never written hold large numbers: a key read from one shows at once
            from infero_b200.cache.storage import LayerKv
            self.kv = LayerKv(k=torch.full((pages, cs.num_kv_heads, page, cs.head_dim), 3.0e4, dtype=self.td, device=DEV),
                              v=torch.full((pages, cs.num_kv_heads, page, cs.value_dim), 3.0e4, dtype=self.td, device=DEV),
                              group=0, page_size=page)
        self.state = torch.full((slots,) + tuple(ss.shape), 7.0, dtype=torch.float32, device=DEV) if ss is not None else None
        self.free = [int(p) for p in torch.randperm(pages, generator=g)]
        self.free_slots = list(range(slots))
        self.table, self.length, self.slot = {}, {}, {}

    def weights(self, strip="l0."):
        return {k[len(strip):]: v.double() for k, v in self.w.items()}

    def close(self, rid):
        self.free = self.table.pop(rid) + self.free                     # the pages given back are handed out next
        self.free_slots.insert(0, self.slot.pop(rid))
        self.length.pop(rid)

    def step(self, entries, write_cache=True):
        """entries: (request, rows of the mixer's input); returns request -> result rows."""
        E = len(entries)
        tok_entry, positions, q_start, q_len, pos0, slots = [], [], [], [], [], []
        for e, (rid, rows) in enumerate(entries):
            n0, n = self.length.get(rid, 0), rows.shape[0]
            if rid not in self.slot:
                self.slot[rid] = self.free_slots.pop(0)
                if self.state is not None:
                    self.state[self.slot[rid]].zero_()
            pages = self.table.setdefault(rid, [])
            while len(pages) * self.page < n0 + n:
                pages.append(self.free.pop(0))
            q_start.append(len(tok_entry)), q_len.append(n), pos0.append(n0), slots.append(self.slot[rid])
            tok_entry += [e] * n
            positions += list(range(n0, n0 + n))
            self.length[rid] = n0 + n
        width = max(len(self.table[rid]) for rid, _ in entries) + 1
        table = torch.full((E, width), -1, dtype=torch.int32)
        for e, (rid, _) in enumerate(entries):
            table[e, :len(self.table[rid])] = torch.tensor(self.table[rid], dtype=torch.int32)
        table = table.to(DEV)
        ctx = types.SimpleNamespace(
            act_dtype=self.td, device=DEV, n_tokens=len(tok_entry), n_entries=E, positions=_i32(positions), tok_entry=_i32(tok_entry),
            entry_q_start=_i32(q_start), entry_q_len=_i32(q_len), entry_pos0=_i32(pos0), entry_slot=_i32(slots),
            h_q_start=np.array(q_start, dtype=np.int32), h_q_len=np.array(q_len, dtype=np.int32), h_pos0=np.array(pos0, dtype=np.int32),
            kv_bound=None, decode_only=all(n == 1 for n in q_len), max_kv_len=max(p + n for p, n in zip(pos0, q_len)),
            kv_cache=lambda slot: self.kv, block_table=lambda group: table, state=lambda slot: self.state)
        h = torch.cat([rows for _, rows in entries]).to(self.td).to(DEV)
        out = self.part.forward(ctx, h, types.SimpleNamespace(cache=0, write_cache=write_cache))
        if hasattr(out, "materialize"):
            out = out.materialize(torch.float32)
        out = out.float().cpu()
        return {rid: out[q_start[e]:q_start[e] + q_len[e]] for e, (rid, _) in enumerate(entries)}


def _window_spec(H, G, D, V, window, d, scale=0.3, dims=None, ramp=None, borrows=False, keep=None):
    from infero_b200.config.spec import MixerSpec, PositionSpec
    dims = D if dims is None else dims
    pos = PositionSpec("rope_neox", 700.0, dims, yarn=ramp) if dims else None
    return MixerSpec(kind="normed_attention", hidden=d, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=V, qkv_bias=True,
                     scale=scale, window=window, keep_window=keep or window, position=pos, qk_norm_kind="projection", sink=True,
                     borrows_cache=borrows, norm_eps=1e-5, weight_suffix="")


def _window_dict(H, G, D, V, window, scale=0.3, dims=None, ramp=None):
    rot = {"base": 700.0, "dims": D if dims is None else dims}
    if ramp:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), ramp))
    return {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale, "mask": {"size": window}, "rot": rot}


def _plain_window(a, h, m, borrowed_from=None):
    w = a.weights()
    kv = PB.window_keys_values(h.double(), borrowed_from.weights() if borrowed_from else w, "mix", m, 1e-5)
    return PB.window_attention(h.double(), w, "mix", m, 1e-5, kv)[:, :m["heads"] * m["vdim"]]


WINDOW_SHAPES = [(2, 1, 8, 8, 5), (6, 2, 6, 10, 7), (4, 2, 64, 64, 24), (3, 3, 16, 24, 33), (4, 1, 128, 128, 100), (1, 1, 12, 5, 1)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,window", WINDOW_SHAPES)
def test_windowed_attention_with_a_sink_in_portions_and_single_tokens(dtype, H, G, D, V, window):
    d = max(64, H * V)
    m = _window_dict(H, G, D, V, window, ramp=(4.0, 32, 8.0, 1.0) if D >= 8 else None)
    a = _Alone(_window_spec(H, G, D, V, window, d, ramp=(4.0, 32, 8.0, 1.0) if D >= 8 else None), dtype)
    g = torch.Generator().manual_seed(7)
    n = 3 * window + 40
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
    assert _rel(torch.cat(outs)[:, :H * V], _plain_window(a, h1, m)) < tol
    assert _rel(torch.cat([got1[0]["b"], got1[1]["b"]])[:, :H * V], _plain_window(a, h2, m)) < tol
    # a request that starts on pages and in a slot another gave back
    a.close("b")
    assert _rel(a.step([("c", h2[:20])])["c"][:, :H * V], _plain_window(a, h2[:20], m)) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("back", [0, 1, 15, 16, 17, 38, 39, 40, 41, 47, 48, 49])
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_stands_out_inside_the_window_and_vanishes_outside_it(dtype, back, decode):
    """One key is made to carry almost all the weight for the last query; it sits `back` tokens before it.  Inside a window
    of 40 (back <= 39) the result is that key's value; one further back and it is gone.  In a portion and token by token."""
    H, G, D, V, window, d = 2, 1, 64, 64, 40, 128
    m = _window_dict(H, G, D, V, window, scale=0.4, dims=0)
    a = _Alone(_window_spec(H, G, D, V, window, d, scale=0.4, dims=0), dtype, seed=back)
    # every query head is projected as the key head is, but from the input with its second half negated: the query of
    # a token whose input is an earlier token's with that half negated is that token's key (score scale * D), while
    # its own key points elsewhere
    for leaf in ("", ".b", ".norm"):
        a.w["l0.mix.q" + leaf] = torch.cat([a.w["l0.mix.k" + leaf]] * H)
    a.w["l0.mix.q"][:, d // 2:] *= -1
    a.part.bind({k: v.to(DEV) for k, v in a.w.items()})
    g = torch.Generator().manual_seed(back)
    n = 70
    h = torch.randn(n, d, generator=g)
    h[n - 1] = h[n - 1 - back]
    h[n - 1, d // 2:] *= -1
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    want = _plain_window(a, h, m)
    if decode:
        got = torch.cat([a.step([("r", h[:n - 50])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 50, n)])
    else:
        got = torch.cat([a.step([("r", h[:11])])["r"], a.step([("r", h[11:])])["r"]])
    assert _rel(got[:, :H * V], want) < (3e-5 if dtype == "float32" else 4e-2)
    h2 = h.clone()
    h2[n - 1 - back] = 0.0
    moved = _rel(_plain_window(a, h2, m)[-1:], want[-1:])
    assert (moved > 0.3) if back < window else (moved < 1e-9)


def test_the_sink_takes_the_weight_when_every_score_is_low():
    """Queries that point away from every key: the softmax's sum is almost all sink, the result almost nothing; without the
    sink's term it would be an average of the values."""
    H, G, D, V, window, d = 2, 2, 16, 16, 30, 64
    m = _window_dict(H, G, D, V, window, scale=3.0, dims=0)
    a = _Alone(_window_spec(H, G, D, V, window, d, scale=3.0, dims=0), "float32")
    for k in ("l0.mix.q", "l0.mix.k", "l0.mix.q.b", "l0.mix.k.b"):
        a.w[k] = a.w[k].abs()
    a.w["l0.mix.q"], a.w["l0.mix.q.b"] = -a.w["l0.mix.q"], -a.w["l0.mix.q.b"]
    a.w["l0.mix.q.norm"], a.w["l0.mix.k.norm"] = a.w["l0.mix.q.norm"].abs(), a.w["l0.mix.k.norm"].abs()
    a.part.bind({k: v.to(DEV) for k, v in a.w.items()})
    h = torch.rand(25, d, generator=torch.Generator().manual_seed(1)) + 0.2
    want = _plain_window(a, h, m)
    got = a.step([("r", h)])["r"][:, :H * V]
    values = (h.double() @ a.weights()["mix.v"].T + a.weights()["mix.v.b"])
    assert float(want.abs().max()) < 0.02 * float(values.abs().max())
    assert float((got.double() - want).abs().max()) < 1e-5 * float(values.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_that_borrows_keys_and_values_looks_further_back_than_their_owner(dtype):
    H, G, D, V, d = 4, 2, 16, 24, 96
    ramp = (4.0, 32, 8.0, 1.0)
    owner = _Alone(_window_spec(H, G, D, V, 9, d, ramp=ramp, keep=21), dtype, seed=1)
    reader = _Alone(_window_spec(2, G, D, V, 21, d, ramp=ramp, borrows=True, keep=21), dtype, seed=2, cache=owner.kv)
    assert not any(".k" in n or ".v" in n for n in reader.w)
    h = torch.randn(60, d, generator=torch.Generator().manual_seed(3))
    if dtype == "bfloat16":
        h = h.bfloat16().float()
    outs = []
    for lo, hi in ((0, 13), (13, 14), (14, 16), (16, 47), (47, 48), (48, 60)):
        owner.step([("r", h[lo:hi])])
        reader.table, reader.free = owner.table, [p for p in reader.free if p not in owner.table["r"]]
        reader.length = {"r": lo}
        reader.slot = dict(owner.slot)
        outs.append(reader.step([("r", h[lo:hi])], write_cache=False)["r"])
    m = _window_dict(2, G, D, V, 21, ramp=ramp)
    assert _rel(torch.cat(outs)[:, :2 * V], _plain_window(reader, h, m, borrowed_from=owner)) < (2e-5 if dtype == "float32" else 3e-2)


def _parallel_spec(H, G, D, C, blocks, taps, d, dims=None, bands=None, ls=0.7, rs=1.1):
    from infero_b200.config.spec import MixerSpec, NORMED_ATTENTION_NAMES, PositionSpec, RGLRU_NAMES
    dims = D if dims is None else dims
    ren = lambda table, side: tuple((r, leaf.replace("mix.", f"mix.{side}.", 1)) for r, leaf in table)      # noqa: E731
    left = MixerSpec(kind="normed_attention", hidden=d, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=D, qkv_bias=True,
                     scale=0.3, position=PositionSpec("rope_neox", 700.0, dims, bands=bands) if dims else None,
                     qk_norm_kind="head_unit", value_from_key=True, out_gate=True, norm_eps=1e-5,
                     names=ren(NORMED_ATTENTION_NAMES, "left"), weight_suffix="")
    right = MixerSpec(kind="rglru", hidden=d, rec_width=C, rec_blocks=blocks, rec_slope=8.0, conv_taps=taps,
                      names=ren(RGLRU_NAMES, "right"), weight_suffix="")
    return MixerSpec(kind="parallel", hidden=d, branches=(left, right), branch_scales=(ls, rs), weight_suffix="")


def _parallel_dict(H, G, D, C, blocks, taps, dims=None, bands=None, ls=0.7, rs=1.1):
    rot = {"base": 700.0, "dims": D if dims is None else dims}
    if bands:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": 0.3, "rot": rot},
            "right": {"width": C, "blocks": blocks, "conv": taps}, "left_scale": ls, "right_scale": rs}


PARALLEL_SHAPES = [(2, 1, 8, 12, 3, 2), (4, 2, 64, 64, 2, 4), (3, 3, 10, 30, 1, 1), (2, 2, 128, 128, 4, 4), (1, 1, 16, 40, 5, 7)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,C,blocks,taps", PARALLEL_SHAPES)
def test_the_two_mixers_side_by_side_in_portions_and_single_tokens(dtype, H, G, D, C, blocks, taps):
    """The stacked activations [gated heads * left scale | state * gate branch * right scale]: the recurrence and the
    convolution's tail carried from portion to portion and token to token, beside a second request, in slots used again."""
    d = H * D + C
    bands = (4.0, 1.0, 3.0, 48) if D >= 16 else None
    a = _Alone(_parallel_spec(H, G, D, C, blocks, taps, d, dims=D // 2 if D >= 16 else None, bands=bands), dtype, slots=2)
    m = _parallel_dict(H, G, D, C, blocks, taps, dims=D // 2 if D >= 16 else None, bands=bands)
    g = torch.Generator().manual_seed(11)
    h1, h2 = torch.randn(90, d, generator=g), torch.randn(30, d, generator=g)
    if dtype == "bfloat16":
        h1, h2 = h1.bfloat16().float(), h2.bfloat16().float()
    w = a.weights()

    def plain(h):
        return torch.cat([0.7 * PB.left_attention(h.double(), w, "mix.left", m["left"], 1e-5)[:, :H * D],
                          1.1 * PB.right_recurrent(h.double(), w, "mix.right", m["right"])[:, H * D:H * D + C]], dim=1)
    outs, at = [], 0
    first = a.step([("a", h1[:1]), ("b", h2[:7])])
    outs.append(first["a"])
    at = 1
    for size in (1, 2, 1, 3, taps, 1, 1, 33, 2):
        step = [("a", h1[at:at + size])]
        if at == 2:
            step.append(("b", h2[7:]))
        res = a.step(step)
        if at == 2:
            second_b = res["b"]
        outs.append(res["a"])
        at += size
    while at < 90:
        outs.append(a.step([("a", h1[at:at + 1])])["a"])
        at += 1
    tol = 3e-5 if dtype == "float32" else 3e-2
    assert _rel(torch.cat(outs)[:, :H * D + C], plain(h1)) < tol
    assert _rel(torch.cat([first["b"], second_b])[:, :H * D + C], plain(h2)) < tol
    a.close("b")
    assert _rel(a.step([("c", h2[:9])])["c"][:, :H * D + C], plain(h2[:9])) < tol        # b's slot, zeroed


def test_a_state_lasts_for_hundreds_of_tokens():
    """A decay close to one: what the first tokens wrote is still most of the state 300 tokens on, so a state that was
    lost or zeroed on the way shows; the portion is cut at every size between 1 and 4 tokens around the taps."""
    H, G, D, C, blocks, taps, d = 1, 1, 8, 32, 2, 4, 40
    a = _Alone(_parallel_spec(H, G, D, C, blocks, taps, d), "float32", pages=40)
    a.w["l0.mix.right.lam"] = a.w["l0.mix.right.lam"] - 4.0
    for leaf in ("x.b", "conv.b"):                       # (a constant input would drown the first tokens)
        a.w["l0.mix.right." + leaf] = torch.zeros_like(a.w["l0.mix.right." + leaf])
    a.part.bind({k: v.to(DEV) for k, v in a.w.items()})
    m = _parallel_dict(H, G, D, C, blocks, taps)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(320, d, generator=g) * 0.1
    h[:6] *= 40.0
    w = a.weights()
    want = PB.right_recurrent(h.double(), w, "mix.right", m["right"])[:, H * D:H * D + C] * 1.1
    quiet = h.clone()
    quiet[:6] = 0.0
    assert _rel(PB.right_recurrent(quiet.double(), w, "mix.right", m["right"])[-1:, H * D:H * D + C] * 1.1, want[-1:]) > 0.3
    outs, at = [], 0
    for size in [3, 1, 2, 4, 1, 1, 3, 2] + [1] * 280 + [23]:
        outs.append(a.step([("r", h[at:at + size])])["r"])
        at += size
    assert at == 320
    assert _rel(torch.cat(outs)[:, H * D:H * D + C], want) < 3e-5


@pytest.mark.parametrize("C,blocks,taps,out_dtype", [(64, 2, 4, torch.float32), (256, 1, 1, torch.float32), (48, 6, 2, torch.float32),
                                                     (512, 2, 3, torch.bfloat16)])
def test_single_token_steps_in_one_launch_with_bf16_gate_matrices(C, blocks, taps, out_dtype):
    """Steps of single tokens with bf16 gate matrices take one kernel for convolution, gates and state.  Three requests
    in shuffled slots decode twelve tokens each after a two-token portion (which takes the three-kernel path); every
    result is held to a 64-bit recurrence written out here."""
    from infero_b200.kernels import layer_ops as L
    g = torch.Generator().manual_seed(C + taps)
    bs, E, n = C // blocks, 3, 14
    rnd = lambda *sh, k=1.0: torch.randn(*sh, generator=g) * k                                  # noqa: E731
    yx = rnd(E, n, 2 * C)
    cw, cb = rnd(C, taps, k=0.5), rnd(C, k=0.1)
    wg = (rnd(blocks, 2 * bs, bs, k=2.0 * bs ** -0.5)).bfloat16()
    rb, ib, lam = rnd(C, k=0.3), rnd(C, k=0.3), rnd(C) - 2.0
    # plain, in 64-bit
    want = torch.zeros(E, n, C, dtype=torch.float64)
    W = wg.double()
    for e in range(E):
        x = torch.cat([torch.zeros(taps - 1, C, dtype=torch.float64), yx[e, :, C:].double()])
        S = torch.zeros(C, dtype=torch.float64)
        for t in range(n):
            u = cb.double() + sum(cw[:, j].double() * x[t + j] for j in range(taps))
            ub = u.view(blocks, bs)
            pre = torch.einsum("bnk,bk->bn", W, ub)
            r = torch.sigmoid(pre[:, :bs].reshape(C) + rb.double())
            i = torch.sigmoid(pre[:, bs:].reshape(C) + ib.double())
            a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
            S = a * S + torch.sqrt(1.0 - a * a) * i * u
            y = yx[e, t, :C].double()
            want[e, t] = 0.9 * S * 0.5 * y * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
    dev = lambda t: t.to(DEV)                                                                  # noqa: E731
    state = torch.full((5, taps, C), 7.0, device=DEV)
    slots = [4, 1, 2]
    for sl in slots:
        state[sl].zero_()
    cwd, cbd, wgd, rbd, ibd, lamd = dev(cw), dev(cb), dev(wg), dev(rb), dev(ib), dev(lam)
    got = torch.zeros(E, n, C, dtype=torch.float64)

    def step(at, size):
        rows = dev(torch.cat([yx[e, at:at + size] for e in range(E)]).contiguous())
        out = torch.empty(E * size, C, dtype=out_dtype, device=DEV)
        L.rglru(rows, 0, C, cwd, cbd, wgd, rbd, ibd, lamd, 8.0, state, _i32(np.repeat(np.arange(E), size)),
                _i32(np.arange(E) * size), _i32([size] * E), _i32(slots), E, out, 0.9, max_q_len=size)
        got[:, at:at + size] = out.double().cpu().view(E, size, C)
    step(0, 2)
    for t in range(2, n):
        step(t, 1)
    assert _rel(got, want) < (2e-5 if out_dtype == torch.float32 else 1e-2)
    assert float(state[0].min()) == 7.0 and float(state[3].max()) == 7.0            # other requests' slots untouched


def test_a_far_key_is_found_by_the_left_mixer():
    """Causal attention over all keys: the key that carries the weight is hundreds of tokens back, at page borders."""
    H, G, D, C, d = 2, 1, 64, 64, 192
    for back in (1, 255, 256, 257, 300):
        a = _Alone(_parallel_spec(H, G, D, C, 1, 2, d, dims=0), "bfloat16", seed=back, pages=40)
        m = _parallel_dict(H, G, D, C, 1, 2, dims=0)
        g = torch.Generator().manual_seed(back)
        n = 330
        h = (torch.randn(n, d, generator=g) * 0.2)
        h[n - 1 - back] *= 8.0
        h[n - 1] = h[n - 1 - back]
        h = h.bfloat16().float()
        w = a.weights()
        # sharpen: unit-RMS queries and keys give scores within +-scale*D; the design's scale is a parameter
        want = 0.7 * PB.left_attention(h.double(), w, "mix.left", m["left"], 1e-5)[:, :H * D]
        got = torch.cat([a.step([("r", h[:n - 3])])["r"]] + [a.step([("r", h[p:p + 1])])["r"] for p in range(n - 3, n)])
        assert _rel(got[:, :H * D], want) < 4e-2


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


ALL = [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("C", "float32"), ("D", "bfloat16"), ("D", "float32")]


@pytest.mark.parametrize("name,dtype", ALL + [("B", "bfloat16")])
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
    PB.forward(cfg, w, toks, trail)
    runner = make_runner(mdir, "float32", 64)
    seen = []
    orig = PreNormBlock.forward

    def spy(self, ctx, x, delta, slot):
        pending = orig(self, ctx, x, delta, slot)
        val, scale = (pending.value, pending.scale) if isinstance(pending, K.Scaled) else (pending, 1.0)
        if isinstance(val, K.Partials):
            val = val.materialize(torch.float32)
        seen.append((x + scale * val.float()).cpu())
        return pending
    PreNormBlock.forward = spy
    try:
        runner.open("a")
        runner.step([StepEntry("a", toks, [len(toks) - 1])])
    finally:
        PreNormBlock.forward = orig
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert _rel(got, trail[i]) < 1e-5, i


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
    """Portions longer than the tiles of the product and attention kernels, cut beside their edges."""
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
        toks.append(int(PB.forward(cfg, w, toks)[-1].argmax()))
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


def test_the_trace_runner_replays_a_banelix_folder(tmp_path):
    mdir = model_dir("A")
    reqs = make_requests("A", [70, 30], seed=2)
    steps = R.steps_mixed(reqs, seed=3, max_live=2)
    got = R.replay_subprocess(mdir, "float32", steps, R.max_live_tokens(steps, reqs), str(tmp_path), CONFIGS["A"]["vocab"])
    worst, where = R.compare(got, plain_logits(mdir, reqs))
    assert worst <= TOL["float32"], (worst, where)


def test_the_generate_command_line_on_a_banelix_folder():
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
